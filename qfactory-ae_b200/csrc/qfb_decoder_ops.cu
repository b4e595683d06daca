// Small element-wise neighbours of the quantized linears in a decoder layer: RMSNorm, SiLU * up,
// rotary embedding with the key / value cache write.  Each replaces a chain of framework kernels
// (eight for the norm) by one launch; all are HBM / launch bound and hold no state.
//
// The reference runs these through its serving stack's own kernels
// (third_party/vllm-bitblas/vllm/model_executor/models/llama.py:60-120, 260-285); they sit on
// either side of the quantized linears this library replaces.
#include <algorithm>

#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

// y[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * w     (fp16 in / out, fp32 arithmetic;
// the product with rstd is rounded to fp16 before the weight multiply, as x.half() * w does)
// With `res` the row is first updated in place, x[r, :] += res[r, :] (one fp16 addition, as the
// framework's x + o), and the norm is taken of the sum: the residual add and the next norm in one pass.
__global__ void __launch_bounds__(256) rmsnorm_kernel(__half* __restrict__ x, const __half* __restrict__ res,
                                                      const __half* __restrict__ w, __half* __restrict__ y, int d,
                                                      float eps) {
  // programmatic dependent launch: the next kernel (a quantized linear, which fetches its weights
  // before it waits for this one) may start now; nothing is read or written before the wait
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  uint4* xr = reinterpret_cast<uint4*>(x + (size_t)row * d);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * d) : nullptr;
  const int nv = d >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 v = xr[i];
    if (rr) {
      const uint4 r = rr[i];
      v.x = as_u32(__hadd2(as_h2(v.x), as_h2(r.x)));
      v.y = as_u32(__hadd2(as_h2(v.y), as_h2(r.y)));
      v.z = as_u32(__hadd2(as_h2(v.z), as_h2(r.z)));
      v.w = as_u32(__hadd2(as_h2(v.w), as_h2(r.w)));
      xr[i] = v;  // re-read below by the same thread
    }
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(as_h2(u[j]));
      ss += f.x * f.x + f.y * f.y;
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += (i < (int)(blockDim.x >> 5)) ? red[i] : 0.f;
  const float rstd = rsqrtf(tot / (float)d + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * d);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const uint4 v = xr[i], g = wr[i];
    const uint32_t u[4] = {v.x, v.y, v.z, v.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(as_h2(u[j]));
      const __half2 n = __floats2half2_rn(f.x * rstd, f.y * rstd);
      o[j] = as_u32(__hmul2(n, as_h2(gw[j])));
    }
    yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// The same norm for rows of up to 16384 features, as a chain of two memory round trips instead of
// eight: up to 1024 threads hold the whole row in registers (VPT 16-byte vectors each), so the
// loads of the row, of the residual and of the weight are all in flight together, the sum of
// squares is one block reduction, and nothing is read twice.  A decode step has one row per batch
// entry and two norms per layer: with one 256-thread CTA looping over the row the kernel took 7 us,
// a fixed cost on the critical path between two linears.
template <int VPT>
__global__ void __launch_bounds__(1024) rmsnorm_row_kernel(__half* __restrict__ x, const __half* __restrict__ res,
                                                           const __half* __restrict__ w, __half* __restrict__ y, int d,
                                                           float eps) {
  grid_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x, nv = d >> 3;
  // the norm weight never depends on the preceding kernel: fetched before the wait
  uint4 g[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
    g[i] = v < nv ? reinterpret_cast<const uint4*>(w)[v] : make_uint4(0, 0, 0, 0);
  }
  grid_dependency_wait();
  uint4* xr = reinterpret_cast<uint4*>(x + (size_t)row * d);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * d) : nullptr;
  uint4 xv[VPT], rv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
    xv[i] = v < nv ? xr[v] : make_uint4(0, 0, 0, 0);
    rv[i] = (rr && v < nv) ? rr[v] : make_uint4(0, 0, 0, 0);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
    if (rr) {
      xv[i].x = as_u32(__hadd2(as_h2(xv[i].x), as_h2(rv[i].x)));
      xv[i].y = as_u32(__hadd2(as_h2(xv[i].y), as_h2(rv[i].y)));
      xv[i].z = as_u32(__hadd2(as_h2(xv[i].z), as_h2(rv[i].z)));
      xv[i].w = as_u32(__hadd2(as_h2(xv[i].w), as_h2(rv[i].w)));
      if (v < nv) xr[v] = xv[i];
    }
    const uint32_t u[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(as_h2(u[j]));
      ss += f.x * f.x + f.y * f.y;
    }
  }
  __shared__ float red[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  const int nwarps = (blockDim.x + 31) >> 5;
  for (int i = 0; i < nwarps; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)d + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * d);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
    if (v >= nv) continue;
    const uint32_t u[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, gw[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(as_h2(u[j]));
      const __half2 n = __floats2half2_rn(f.x * rstd, f.y * rstd);
      o[j] = as_u32(__hmul2(n, as_h2(gw[j])));
    }
    yr[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// out[r, j] = silu(gu[r, j]) * gu[r, half + j]   for j < half   (fp16, silu and product as fp16 ops)
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ out, int half,
                                                       long long total_vec) {
  grid_launch_dependents();
  grid_dependency_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one 8-element vector each
  if (i >= total_vec) return;
  const int vec_per_row = half >> 3;
  const long long r = i / vec_per_row;
  const int j = (int)(i - r * vec_per_row);
  const uint4 a = reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * half)[j];
  const uint4 b = reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * half + half)[j];
  const uint32_t ua[4] = {a.x, a.y, a.z, a.w}, ub[4] = {b.x, b.y, b.z, b.w};
  uint32_t o[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __half22float2(as_h2(ua[q]));
    // silu in fp32, rounded to fp16, then the fp16 product (what F.silu(g) * u computes)
    const __half2 s = __floats2half2_rn(f.x / (1.f + __expf(-f.x)), f.y / (1.f + __expf(-f.y)));
    o[q] = as_u32(__hmul2(s, as_h2(ub[q])));
  }
  reinterpret_cast<uint4*>(out + (size_t)r * half)[j] = make_uint4(o[0], o[1], o[2], o[3]);
}

// Rotary embedding of the query and key heads of a fused QKV activation, in place, and the write
// of the rotated keys and the values into the static caches at positions pos[t]:
//   qkv      fp16 [B, T, hq + 2 hkv, hd]     (pairs (2i, 2i+1) rotate by the angle of pos[t], frequency i)
//   cos/sin  fp16 [max_len, hd / 2]
//   k_cache, v_cache  fp16 [B, hkv, max_len, hd]
// Every product and sum is an fp16 operation, as the framework expression t1*c - t2*s computes.
__global__ void __launch_bounds__(256) rope_cache_kernel(__half* __restrict__ qkv, const __half* __restrict__ cosv,
                                                         const __half* __restrict__ sinv, const long long* __restrict__ pos,
                                                         __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                                         int T, int hq, int hkv, int hd, int max_len, long long total) {
  grid_launch_dependents();
  grid_dependency_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one pair of elements each
  if (idx >= total) return;
  const int hp = hd >> 1, H = hq + 2 * hkv;
  const int i = (int)(idx % hp);
  long long r = idx / hp;
  const int h = (int)(r % H);
  r /= H;
  const int t = (int)(r % T);
  const int b = (int)(r / T);
  const long long p = pos[t];
  // a position outside the tables and the caches (a graph replayed past max_len, a bad caller)
  // is skipped: no rotation, no cache write
  if (p < 0 || p >= max_len) return;
  __half2* src = reinterpret_cast<__half2*>(qkv + (((size_t)b * T + t) * H + h) * hd) + i;
  __half2 v = *src;
  if (h < hq + hkv) {
    const __half c = cosv[(size_t)p * hp + i], s = sinv[(size_t)p * hp + i];
    const __half x1 = __low2half(v), x2 = __high2half(v);
    // (_rn forms: the compiler must not contract a product and a sum into one fused multiply-add)
    v = __halves2half2(__hsub_rn(__hmul_rn(x1, c), __hmul_rn(x2, s)), __hadd_rn(__hmul_rn(x1, s), __hmul_rn(x2, c)));
    *src = v;
  }
  if (h >= hq) {
    const bool is_k = h < hq + hkv;
    __half* cache = is_k ? k_cache : v_cache;
    const int hh = is_k ? h - hq : h - hq - hkv;
    reinterpret_cast<__half2*>(cache + (((size_t)b * hkv + hh) * max_len + (size_t)p) * hd)[i] = v;
  }
}

// Every kernel of this file is launched with programmatic stream serialisation: it may become
// resident while its predecessor drains, and waits (griddepcontrol.wait) before touching memory.
template <class... KArgs, class... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

cudaError_t launch_rope_cache(__half* qkv, const __half* cosv, const __half* sinv, const long long* pos, __half* k_cache,
                              __half* v_cache, int B, int T, int hq, int hkv, int hd, int max_len, cudaStream_t st) {
  const long long total = (long long)B * T * (hq + 2 * hkv) * (hd >> 1);
  return launch_pdl(rope_cache_kernel, (unsigned)((total + 255) / 256), 256, st, qkv, cosv, sinv, pos, k_cache, v_cache, T, hq,
                    hkv, hd, max_len, total);
}

cudaError_t launch_rmsnorm(__half* x, const __half* res, const __half* w, __half* y, int rows, int d, float eps,
                           cudaStream_t st) {
  const int nv = d >> 3;
  // few rows (a decode step): one CTA per row holding the row in registers; many rows or very long
  // rows: the looping kernel, which keeps more CTAs per SM
  if (rows <= 64 && nv <= 2048) {
    const int vpt = nv > 1024 ? 2 : 1;
    const unsigned block = (unsigned)std::min(1024, (((nv + vpt - 1) / vpt + 31) / 32) * 32);
    if (vpt == 1) return launch_pdl(rmsnorm_row_kernel<1>, (unsigned)rows, block, st, x, res, w, y, d, eps);
    return launch_pdl(rmsnorm_row_kernel<2>, (unsigned)rows, block, st, x, res, w, y, d, eps);
  }
  return launch_pdl(rmsnorm_kernel, (unsigned)rows, 256, st, x, res, w, y, d, eps);
}

cudaError_t launch_silu_mul(const __half* gu, __half* out, int rows, int half, cudaStream_t st) {
  const long long total = (long long)rows * (half >> 3);
  return launch_pdl(silu_mul_kernel, (unsigned)((total + 255) / 256), 256, st, gu, out, half, total);
}

}  // namespace qfb
