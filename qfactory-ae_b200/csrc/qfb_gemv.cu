// Split-K GEMV / skinny GEMM on CUDA cores for small activation batches.
//
// Replaces the reference's kernel_gptq / kernel_gemv templates
// (qfactory/include/gptq_gemv.h:14-154, qfactory/include/gemv.h:12-94).
//
// Mapping.  A CTA owns one 128-row tile of the packed weight and a contiguous range of
// K units; thread (row r, k-way w) owns row r and a sub-range of those units, so a warp's
// 128-bit loads cover 512 contiguous bytes and NO cross-lane reduction is needed: each
// lane accumulates its own output row.  The activation slice of the CTA is staged once in
// shared memory and read back with warp-uniform (broadcast) 128-bit loads.  Partial sums of
// the k-ways are combined in shared memory; partial sums of the K splits go through an fp32
// workspace and are summed in split order by the last CTA of the tile to arrive
// (deterministic, no atomics on data, counters reset themselves).
//
// Numerics.  (q - z) is exact in fp16; x * (q - z) is accumulated in fp16x2 chains of at most 8
// terms, flushed into an fp32 sum per quantisation group, and the group sum is multiplied by the
// scale once, in fp32 (the reference's "deferred decode", qfactory/include/utils.h:193-213, with
// fp32 instead of fp16 group sums).  fp16x2 arithmetic issues at half rate on B200, so every
// fp16 instruction removed from the inner loop counts double.
//
// Ordering under programmatic dependent launch: weight, scale and zero loads (which never
// depend on the preceding kernel) are issued first; activations, the workspace and the
// output are only touched after griddepcontrol.wait.
#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

template <int BITS, int MB, int U>
__global__ void __launch_bounds__(256, (MB <= 2 ? 3 : 2)) gemv_splitk_kernel(const GemvParams p) {
  using G = Geo<BITS>;
  using C = Codec<BITS>;
  constexpr int XV = G::kUnitK / 8;  // uint4 (8 halfs) of activations per unit
  constexpr int NV = G::kUnitVecs;

  extern __shared__ uint4 smem[];

  const int tid = threadIdx.x;
  const int r = tid & (kTileRows - 1);
  const int kw = tid >> 7;
  const int KW = blockDim.x >> 7;
  const int tile = blockIdx.y;
  const int split = blockIdx.x;
  const int S = gridDim.x;

  // unit range of the CTA and of this thread's k-way (no divisions: the host passes the strides)
  const int ub = min(split * p.max_units_per_cta, p.units);
  const int ue = min(ub + p.max_units_per_cta, p.units);
  const int ncta = ue - ub;
  const int tb = min(ub + kw * p.units_per_kway, ue);
  const int te = min(tb + p.units_per_kway, ue);

  const uint4* wrow = p.qw + ((size_t)tile * p.units * NV) * kTileRows + r;
  const __half* srow = p.qs + (size_t)tile * p.groups * kTileRows + r;
  const uint8_t* zrow = p.qz + (size_t)tile * p.groups * kTileRows + r;

  // position of unit `tb` inside its quantisation group (one division per thread)
  int g_load = tb / p.units_per_group;
  int gpos_load = tb - g_load * p.units_per_group;

  uint4 wv[U][NV];
  __half sc[U];
  uint32_t zr[U];
  bool newg[U];

  auto load_batch = [&](int base) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int un = base + u;
      newg[u] = false;
      if (un < te) {
#pragma unroll
        for (int v = 0; v < NV; ++v) wv[u][v] = ldg_stream_v4(wrow + ((size_t)un * NV + v) * kTileRows);
        newg[u] = (u == 0) || (gpos_load == 0);
        if (newg[u]) {  // first unit of a group (or of the batch): fetch the group's scale and zero
          sc[u] = p.qs ? srow[(size_t)g_load * kTileRows] : __ushort_as_half(0x3C00);
          zr[u] = p.qz ? (uint32_t)zrow[(size_t)g_load * kTileRows] : p.zconst;
        }
        if (++gpos_load == p.units_per_group) {
          gpos_load = 0;
          ++g_load;
        }
      }
    }
  };

  load_batch(tb);
  grid_launch_dependents();
  grid_dependency_wait();

  // stage the CTA's activation slice: MB rows x (ncta * kUnitK) halfs; rows >= m read as 0
  const int xs_stride = p.max_units_per_cta * XV;
  {
    const int nvec = ncta * XV;
    for (int i = tid; i < nvec * MB; i += blockDim.x) {
      const int m = i / nvec, j = i - m * nvec;
      uint4* dst = smem + m * xs_stride + j;
      if (m < p.m) {
        cp_async_16(dst, p.x + (size_t)m * p.k + (size_t)ub * G::kUnitK + (size_t)j * 8);
      } else {
        *dst = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit_wait_all();
  }
  __syncthreads();

  // acc: fp32 results; gacc: fp32 sum of x * (q - z) over the current group, scaled once per group
  float acc[MB], gacc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = gacc[m] = 0.f;
  float s_cur = 0.f;
  typename C::ZM zm = C::zmagic(0);

  for (int base = tb; base < te; base += U) {
    if (base != tb) load_batch(base);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (base + u < te) {
        if (newg[u]) {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            acc[m] = fmaf(s_cur, gacc[m], acc[m]);
            gacc[m] = 0.f;
          }
          s_cur = __half2float(sc[u]);
          zm = C::zmagic(zr[u]);
        }
        const uint4* xs = smem + (base + u - ub) * XV;
        __half2 a0[MB], a1[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) a0[m] = a1[m] = __half2half2(__ushort_as_half(0));
        C::unit(wv[u], zm, [&](int j8, __half2(&d)[4]) {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            const uint4 xv = xs[m * xs_stride + j8];
            a0[m] = __hfma2(d[0], as_h2(xv.x), a0[m]);
            a1[m] = __hfma2(d[1], as_h2(xv.y), a1[m]);
            a0[m] = __hfma2(d[2], as_h2(xv.z), a0[m]);
            a1[m] = __hfma2(d[3], as_h2(xv.w), a1[m]);
          }
          if ((j8 & 3) == 3 || j8 == XV - 1) {  // flush the fp16 chains (<= 8 terms each) into fp32
#pragma unroll
            for (int m = 0; m < MB; ++m) {
              const float2 f = __half22float2(__hadd2(a0[m], a1[m]));
              gacc[m] += f.x + f.y;
              a0[m] = a1[m] = __half2half2(__ushort_as_half(0));
            }
          }
        });
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = fmaf(s_cur, gacc[m], acc[m]);

  // combine the k-ways of this CTA
  __syncthreads();  // everyone is done reading the activation stage
  float* red = reinterpret_cast<float*>(smem);
  if (KW > 1) {
    if (kw > 0) {
#pragma unroll
      for (int m = 0; m < MB; ++m) red[((kw - 1) * MB + m) * kTileRows + r] = acc[m];
    }
    __syncthreads();
    if (kw == 0) {
      for (int w = 1; w < KW; ++w)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] += red[((w - 1) * MB + m) * kTileRows + r];
    }
  }

  const int n = tile * kTileRows + r;
  if (S == 1) {
    if (kw == 0 && n < p.n) {
#pragma unroll
      for (int m = 0; m < MB; ++m)
        if (m < p.m) p.y[(size_t)m * p.n + n] = __float2half_rn(acc[m]);
    }
    return;
  }

  // split-K: publish this CTA's partial, the last CTA of the tile sums them in split order
  if (kw == 0) {
#pragma unroll
    for (int m = 0; m < MB; ++m)
      if (m < p.m) p.partial[((size_t)split * p.m + m) * p.npad + n] = acc[m];
  }
  __threadfence();
  __syncthreads();
  __shared__ int is_last;
  if (tid == 0) {
    const unsigned prev = atomicAdd(p.counters + tile, 1u);
    is_last = (prev == (unsigned)(S - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (kw == 0) {
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m < p.m) {
        // eight independent loads in flight per step; the additions stay in split order
        const float* base = p.partial + (size_t)m * p.npad + n;
        const size_t sstride = (size_t)p.m * p.npad;
        float s = 0.f;
        int sp = 0;
        for (; sp + 8 <= S; sp += 8) {
          float t[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) t[u] = __ldcg(base + (size_t)(sp + u) * sstride);
#pragma unroll
          for (int u = 0; u < 8; ++u) s += t[u];
        }
        for (; sp < S; ++sp) s += __ldcg(base + (size_t)sp * sstride);
        if (n < p.n) p.y[(size_t)m * p.n + n] = __float2half_rn(s);
      }
    }
  }
  if (tid == 0) p.counters[tile] = 0u;
}

template <int BITS, int MB>
static cudaError_t launch_one(const GemvParams& p, dim3 grid, int block, size_t smem, bool pdl, cudaStream_t st) {
  constexpr int U = (BITS == 3) ? 2 : (BITS == 2 ? 4 : 8);
  auto kern = gemv_splitk_kernel<BITS, MB, U>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int BITS>
static cudaError_t launch_bits(const GemvParams& p, int mb, dim3 grid, int block, size_t smem, bool pdl,
                               cudaStream_t st) {
  switch (mb) {
    case 1: return launch_one<BITS, 1>(p, grid, block, smem, pdl, st);
    case 2: return launch_one<BITS, 2>(p, grid, block, smem, pdl, st);
    case 4: return launch_one<BITS, 4>(p, grid, block, smem, pdl, st);
    default: return launch_one<BITS, 8>(p, grid, block, smem, pdl, st);
  }
}

cudaError_t launch_gemv(const GemvParams& p, int bits, int mb, dim3 grid, int block, size_t smem, bool pdl,
                        cudaStream_t st) {
  switch (bits) {
    case 2: return launch_bits<2>(p, mb, grid, block, smem, pdl, st);
    case 3: return launch_bits<3>(p, mb, grid, block, smem, pdl, st);
    case 4: return launch_bits<4>(p, mb, grid, block, smem, pdl, st);
    case 8: return launch_bits<8>(p, mb, grid, block, smem, pdl, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace qfb
