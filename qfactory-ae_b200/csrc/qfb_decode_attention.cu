// Single-query (decode step) attention over the static key / value cache: the neighbour of the
// quantized linears between the QKV and the O projection of a decoder layer.  One launch replaces
// the framework's masked attention over the whole cache (mask construction, grouped-query
// expansion, attention, transpose copy: ~12 us per layer in the CUDA-graph decode step).
//
// The reference runs this step through its serving stack's paged-attention kernels
// (third_party/vllm-bitblas/vllm/model_executor/models/llama.py:150-175); it is not part of the
// quantized path itself.
//
//   qkv      fp16 [B, hq + 2 hkv, 128]   (queries already rotated; only the hq query heads are read)
//   k_cache, v_cache  fp16 [B, hkv, max_len, 128]; the keys 0 .. pos[0] are attended
//   out      fp16 [B, hq * 128]          (the O projection's input layout)
//
// Grid (hkv, B, NS): the NS CTAs of a (batch row, key/value head) form a thread-block cluster and
// split the keys; each CTA computes the scores of the G = hq / hkv query heads of its head group
// against its keys with mma.sync (queries as the A operand, zero-padded to 16 rows, keys as B,
// fp32 accumulation), a softmax over its range in shared memory, and P * V with 16-byte loads of
// the value rows; the partial (max, sum, output) of every CTA is pushed into the first
// CTA's shared memory, one cluster barrier, and the first CTA merges and stores.
#include <math.h>

#include <algorithm>

#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

namespace {

constexpr int kHD = 128;           // head dimension
constexpr int kQStride = kHD + 8;  // halfs; +16 bytes per row keeps the fragment loads conflict-free
constexpr int kRecvStride = kHD + 2;  // floats per (split, head): the output row, its max and its sum

__device__ __forceinline__ void attn_mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // rows 8..15 of the A operand are padding: a1 = a3 = 0
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void attn_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void attn_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void attn_st_cluster(uint32_t local_addr, int rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// rotary embedding of one pair (x1, x2) by (c, s): every product and sum an fp16 operation, as
// rope_cache_kernel computes it (the _rn forms keep the compiler from fusing product and sum)
__device__ __forceinline__ uint32_t rope_pair(uint32_t x, __half c, __half s) {
  const __half x1 = __low2half(as_h2(x)), x2 = __high2half(as_h2(x));
  return as_u32(__halves2half2(__hsub_rn(__hmul_rn(x1, c), __hmul_rn(x2, s)), __hadd_rn(__hmul_rn(x1, s), __hmul_rn(x2, c))));
}
// 8 consecutive halfs (4 pairs, frequencies i0 .. i0 + 3) rotated by the angles of one position
__device__ __forceinline__ uint4 rope_vec(uint4 v, const __half* cosp, const __half* sinp, int i0) {
  const uint2 c = *reinterpret_cast<const uint2*>(cosp + i0), s = *reinterpret_cast<const uint2*>(sinp + i0);
  const __half2 c01 = as_h2(c.x), c23 = as_h2(c.y), s01 = as_h2(s.x), s23 = as_h2(s.y);
  v.x = rope_pair(v.x, __low2half(c01), __low2half(s01));
  v.y = rope_pair(v.y, __high2half(c01), __high2half(s01));
  v.z = rope_pair(v.z, __low2half(c23), __low2half(s23));
  v.w = rope_pair(v.w, __high2half(c23), __high2half(s23));
  return v;
}

// ROPE: the kernel also does what rope_cache_kernel does for a single new token: the queries are
// rotated as they are staged, the new key is rotated and, with the new value, used from shared
// memory by the CTAs whose key range holds the new position, and ONE CTA of the cluster writes
// both into the caches for the steps to come.  (qkv itself is left un-rotated.)
template <int G, bool ROPE>
__global__ void __launch_bounds__(128) decode_attention_kernel(const __half* __restrict__ qkv, __half* __restrict__ kc,
                                                               __half* __restrict__ vc,
                                                               const long long* __restrict__ pos, __half* __restrict__ out,
                                                               int hq, int hkv, int max_len, int chunk_max,
                                                               float scale_log2e, const __half* __restrict__ cosv,
                                                               const __half* __restrict__ sinv) {
  static_assert(G >= 1 && G <= 8, "one 16-row MMA tile holds the query heads of a group");
  extern __shared__ uint4 smem_raw[];
  __half* q_s = reinterpret_cast<__half*>(smem_raw);                          // [8][kQStride]
  float* s_s = reinterpret_cast<float*>(q_s + 8 * kQStride);                  // [G][chunk_max] scores, then probabilities
  float* stat = s_s + G * chunk_max;                                          // [G] max, [G] sum
  float* pv = stat + 16;                                                      // [4 warps][G][128] partial outputs
  float* recv = pv + 4 * G * kHD;                                             // [NS][G][kRecvStride] (used in the first CTA)
  __shared__ __align__(16) __half knew_s[kHD], vnew_s[kHD];                   // ROPE: the new token's rotated key, its value

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kvh = blockIdx.x, b = blockIdx.y, z = blockIdx.z, NS = gridDim.z;
  if (NS > 1) attn_cluster_arrive();  // (waited for before the first remote store)
  // (No programmatic dependent launch here: letting the O projection become resident while this
  // latency-bound kernel runs made the decode step 10 % slower; launched in plain stream order it
  // was the fastest of the four variants measured.)

  // this CTA's keys: [k0, k0 + nk) of the n = pos + 1 attended ones, in chunks of a multiple of 8
  const long long p_new = pos[0];
  const int n = min((int)p_new + 1, max_len);
  const int chunk = min(chunk_max, (((n + NS - 1) / NS) + 7) & ~7);
  const int k0 = z * chunk;
  const int nk = max(0, min(n, k0 + chunk) - k0);
  const int H = hq + 2 * hkv;
  const __half* kbase = kc + ((size_t)b * hkv + kvh) * (size_t)max_len * kHD;
  const __half* vbase = vc + ((size_t)b * hkv + kvh) * (size_t)max_len * kHD;

  // the G query rows of this head group, rows G..7 zero
  for (int i = tid; i < 8 * (kHD / 8); i += blockDim.x) {
    const int r = i / (kHD / 8), c = i % (kHD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) {
      v = *reinterpret_cast<const uint4*>(qkv + ((size_t)b * H + (size_t)kvh * G + r) * kHD + c * 8);
      if (ROPE && p_new >= 0 && p_new < max_len) v = rope_vec(v, cosv + (size_t)p_new * (kHD / 2), sinv + (size_t)p_new * (kHD / 2), c * 4);
    }
    *reinterpret_cast<uint4*>(q_s + r * kQStride + c * 8) = v;
  }
  // the key position of the new token inside this CTA's range (or -1): taken from shared memory, not from the cache
  int j_new = -1;
  if (ROPE && p_new >= 0 && p_new < max_len) {
    const int pn = (int)p_new;
    if (pn >= k0 && pn < k0 + nk) j_new = pn - k0;
    if (j_new >= 0 && tid < 32) {   // 16 threads rotate the key, 16 copy the value
      const int c = tid & 15;
      const __half* src = qkv + ((size_t)b * H + hq + (tid < 16 ? 0 : hkv) + kvh) * kHD + c * 8;
      uint4 v = *reinterpret_cast<const uint4*>(src);
      if (tid < 16) v = rope_vec(v, cosv + (size_t)pn * (kHD / 2), sinv + (size_t)pn * (kHD / 2), c * 4);
      *reinterpret_cast<uint4*>((tid < 16 ? knew_s : vnew_s) + c * 8) = v;
      // the CTA that owns the position also stores both for the steps to come
      __half* dst = (tid < 16 ? kc : vc) + (((size_t)b * hkv + kvh) * (size_t)max_len + (size_t)pn) * kHD + c * 8;
      *reinterpret_cast<uint4*>(dst) = v;
    }
  }
  __syncthreads();

  // the value rows of the first P * V pass are requested now: they do not depend on the scores,
  // and their round trip then overlaps the one of the keys
  const int rg = tid >> 4, cg = tid & 15;
  const __half* vr = vbase + (size_t)k0 * kHD + cg * 8;
  uint4 v_first[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int j = rg + 8 * u;
    v_first[u] = j < nk ? (ROPE && j == j_new ? *reinterpret_cast<const uint4*>(vnew_s + cg * 8)
                                              : *reinterpret_cast<const uint4*>(vr + (size_t)j * kHD))
                        : make_uint4(0, 0, 0, 0);
  }

  // ---- scores: S[head][key] = q . k * scale, 8 keys per MMA tile, the warps take alternate tiles ----
  {
    uint32_t qa[8][2];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(q_s + g * kQStride + ks * 16 + 2 * t);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(q_s + g * kQStride + ks * 16 + 8 + 2 * t);
    }
    const int ntiles = (nk + 7) >> 3;
    for (int ti = warp; ti < ntiles; ti += 4) {
      const int key = min(k0 + ti * 8 + g, n - 1);  // (keys past the range are read in bounds and masked below)
      const __half* kr = (ROPE && key - k0 == j_new) ? knew_s + 2 * t : kbase + (size_t)key * kHD + 2 * t;
      uint32_t kb[8][2];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        kb[ks][0] = *reinterpret_cast<const uint32_t*>(kr + ks * 16);
        kb[ks][1] = *reinterpret_cast<const uint32_t*>(kr + ks * 16 + 8);
      }
      float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) attn_mma(d, qa[ks][0], qa[ks][1], kb[ks][0], kb[ks][1]);
      if (g < G) {  // d[0], d[1]: head g, keys 2t and 2t + 1 of the tile
        const int j = ti * 8 + 2 * t;
        s_s[g * chunk_max + j] = j < nk ? d[0] * scale_log2e : -1e30f;
        s_s[g * chunk_max + j + 1] = j + 1 < nk ? d[1] * scale_log2e : -1e30f;
      }
    }
  }
  __syncthreads();

  // ---- softmax over this CTA's keys (base-2 exponent; the 1 / sum is applied at the end) ----
  for (int h = warp; h < G; h += 4) {
    float* row = s_s + h * chunk_max;
    float m = -1e30f;
    for (int j = lane; j < nk; j += 32) m = fmaxf(m, row[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (int j = lane; j < nk; j += 32) {
      const float p = exp2f(row[j] - m);
      row[j] = p;
      l += p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) {
      stat[h] = m;
      stat[8 + h] = l;
    }
  }
  __syncthreads();

  // ---- O[head][c] = sum_j P[head][j] * V[j][c] ----
  // Sixteen threads read one 256-byte value row (16 bytes each), so the eight row groups of the
  // CTA have eight rows in flight per pass and four passes unrolled: one memory round trip covers
  // 32 keys.  (One thread per column with 2-byte loads had 4 rows in flight and paid a round trip
  // per 4 keys: 5 us of a 9 us launch.)  The row groups are then summed: the two of a warp by a
  // shuffle, the four warps through shared memory.
  float o[G];
  {
    float acc[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
    for (int j0 = rg; j0 < nk; j0 += 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + 8 * u;
        if (j0 == rg) v[u] = v_first[u];
        else v[u] = j < nk ? (ROPE && j == j_new ? *reinterpret_cast<const uint4*>(vnew_s + cg * 8)
                                                 : *reinterpret_cast<const uint4*>(vr + (size_t)j * kHD))
                           : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = min(j0 + 8 * u, nk - 1);  // (a row past the range was read as zeros)
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t2 = __half22float2(as_h2(w[e]));
          f[2 * e] = t2.x;
          f[2 * e + 1] = t2.y;
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float p = s_s[h * chunk_max + j];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(p, f[e], acc[h][e]);
        }
      }
    }
    // lanes 0-15 and 16-31 of a warp hold two row groups of the same columns
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], 16);
    if (lane < 16) {
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float* dst = pv + (warp * G + h) * kHD + cg * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < G; ++h)
      o[h] = (pv[(0 * G + h) * kHD + tid] + pv[(1 * G + h) * kHD + tid]) + (pv[(2 * G + h) * kHD + tid] + pv[(3 * G + h) * kHD + tid]);
  }

  __half* orow = out + ((size_t)b * hq + (size_t)kvh * G) * kHD + tid;
  if (NS == 1) {
#pragma unroll
    for (int h = 0; h < G; ++h) orow[(size_t)h * kHD] = __float2half_rn(o[h] / stat[8 + h]);
    return;
  }

  // ---- merge the splits in the first CTA of the cluster ----
  const uint32_t recv_addr = static_cast<uint32_t>(__cvta_generic_to_shared(recv));
  attn_cluster_wait();  // pairs with the arrive at kernel start: every CTA of the cluster runs
#pragma unroll
  for (int h = 0; h < G; ++h) attn_st_cluster(recv_addr + ((z * G + h) * kRecvStride + tid) * 4, 0, o[h]);
  if (tid < G) {
    attn_st_cluster(recv_addr + ((z * G + tid) * kRecvStride + kHD) * 4, 0, stat[tid]);
    attn_st_cluster(recv_addr + ((z * G + tid) * kRecvStride + kHD + 1) * 4, 0, stat[8 + tid]);
  }
  attn_cluster_arrive();
  attn_cluster_wait();
  if (z != 0) return;
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float m = -1e30f;
    for (int s = 0; s < NS; ++s) m = fmaxf(m, recv[(s * G + h) * kRecvStride + kHD]);
    float num = 0.f, den = 0.f;
    for (int s = 0; s < NS; ++s) {
      const float* r = recv + (s * G + h) * kRecvStride;
      const float w = exp2f(r[kHD] - m);  // 0 for an empty split (its max is the -1e30 sentinel, its sum 0)
      num = fmaf(w, r[tid], num);
      den = fmaf(w, r[kHD + 1], den);
    }
    orow[(size_t)h * kHD] = __float2half_rn(num / den);
  }
}

template <int G, bool ROPE>
cudaError_t launch_g(const __half* qkv, __half* kc, __half* vc, const long long* pos, __half* out, int B, int hq,
                     int hkv, int max_len, const __half* cosv, const __half* sinv, cudaStream_t st) {
  // up to 8 key splits, at least 64 keys of capacity each, no more than fill the device
  // (more CTAs than about four per SM only add launch and merge work: measured at 16 rows);
  // but never so few that the scores of a split outgrow the shared memory of a CTA
  const int by_len = std::max(1, max_len / 64), by_fill = std::max(1, (148 * 4) / std::max(1, hkv * B));
  int ns = std::min(8, std::min(by_len, by_fill));
  auto smem_for = [&](int nsplit, int* chunk) {
    const int cm = (((max_len + nsplit - 1) / nsplit) + 7) & ~7;
    if (chunk) *chunk = cm;
    return (size_t)8 * kQStride * sizeof(__half) + ((size_t)G * cm + 16 + 4 * G * kHD) * sizeof(float) +
           (size_t)nsplit * G * kRecvStride * sizeof(float);
  };
  constexpr size_t kSmemBudget = 200 * 1024;
  while (ns < 8 && smem_for(ns, nullptr) > kSmemBudget) ++ns;
  int chunk_max = 0;
  const size_t smem = smem_for(ns, &chunk_max);
  if (smem > kSmemBudget) return cudaErrorInvalidConfiguration;  // (not reachable for max_len <= 16384)
  auto kern = decode_attention_kernel<G, ROPE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(hkv, B, ns);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = ns;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float scale_log2e = 1.4426950408889634f / sqrtf((float)kHD);
  return cudaLaunchKernelEx(&cfg, kern, qkv, kc, vc, pos, out, hq, hkv, max_len, chunk_max, scale_log2e, cosv, sinv);
}

}  // namespace

bool decode_attention_supported(int hq, int hkv, int hd, int max_len) {
  if (hd != kHD || hkv <= 0 || hq % hkv != 0 || max_len <= 0 || max_len > 16384) return false;
  const int gq = hq / hkv;
  return gq == 1 || gq == 2 || gq == 4 || gq == 8;
}

cudaError_t launch_decode_attention(const __half* qkv, __half* kc, __half* vc, const long long* pos, __half* out,
                                    int B, int hq, int hkv, int max_len, const __half* cosv, const __half* sinv,
                                    cudaStream_t st) {
#define QFB_ATTN_CASE(GQ)                                                                                         \
  case GQ:                                                                                                        \
    return cosv ? launch_g<GQ, true>(qkv, kc, vc, pos, out, B, hq, hkv, max_len, cosv, sinv, st)                 \
                : launch_g<GQ, false>(qkv, kc, vc, pos, out, B, hq, hkv, max_len, nullptr, nullptr, st);
  switch (hq / hkv) {
    QFB_ATTN_CASE(1)
    QFB_ATTN_CASE(2)
    QFB_ATTN_CASE(4)
    QFB_ATTN_CASE(8)
    default: return cudaErrorInvalidValue;
  }
#undef QFB_ATTN_CASE
}

}  // namespace qfb
