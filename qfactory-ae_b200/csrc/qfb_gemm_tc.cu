// Tensor-core path: y^T[n, m] = W[n, :] . x[m, :] with the WEIGHT rows as the UMMA M dimension
// (128) and the activation batch as the UMMA N dimension (16..256), so that even a single
// activation row fills the 5th-generation tensor core.  No counterpart in the reference, whose
// kernels are CUDA-core GEMVs only (qfactory/include/gptq_gemv.h:14-154).
//
// Data flow of one CTA (one 128-row weight tile x one batch tile x one K split):
//
//   TMA (warp 0)      packed weights (contiguous bulk copy), zeros, scales, and the fp16
//                     activation tile (128-byte-swizzled tensor copy) -> shared-memory ring
//   decode (8 warps)  packed codes -> exact (q - z) fp16 pairs in registers (LOP3 / PRMT magic
//                     numbers) -> tcgen05.st into TENSOR MEMORY as the A operand.  The fp16
//                     weights never touch shared memory, whose bandwidth could not carry the
//                     4x-expanded stream at HBM rate.
//   MMA (1 thread)    tcgen05.mma kind::f16, A from tensor memory, B (activations) from shared
//                     memory, fp32 accumulators in tensor memory
//   scale (4 warps)   POST mode (small batches): one accumulator per quantisation group; the
//                     group's fp32 partial is read back with tcgen05.ld and folded into register
//                     accumulators with ONE fp32 FMA by the row's scale, so the decode needs a
//                     single fp16 instruction per code pair.  PRE mode (large batches): the
//                     decode multiplies by the scale and one accumulator spans all of K.
//
// Every mbarrier wait is bounded: on a time-out the CTA raises a flag, all roles drain, tensor
// memory is released and a status word is written for the host.
#include "qfb_common.cuh"
#include "qfb_kernels.h"
#include "qfb_ptx.cuh"

namespace qfb {

using namespace ptx;

constexpr int kTcThreads = 512;
constexpr int kASlots = 4;         // A-operand slots in tensor memory, 32 columns (64 k) each
constexpr int kAColsTotal = kASlots * 32;
constexpr int kDecodeWarps = 8;

template <int BITS, int NB, bool POST>
struct TcCfg {
  static constexpr int kWBytes = 128 * 64 * BITS / 8;
  static constexpr int kXBytes = NB * 128;
  static constexpr int kZBytes = 128;
  static constexpr int kSBytes = 256;
  static constexpr int kStageBytes = kWBytes + kXBytes + kZBytes + kSBytes;
  static constexpr int kBudget = (NB <= 64) ? 100 * 1024 : 200 * 1024;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : (kStagesRaw < 3 ? 3 : kStagesRaw);
  static constexpr int kDBufs = POST ? 2 : 1;
  static constexpr int kColsNeeded = kAColsTotal + kDBufs * NB;
  static constexpr int kTmemCols = kColsNeeded <= 256 ? 256 : 512;
  static constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes;
};

// ---- decode of the 32 codes one thread owns in a 64-k stage ---------------------------
template <int BITS> struct StageDecode;
template <> struct StageDecode<4> {
  // stage = [2 units][128 rows][16 B]; thread (row, h) owns unit h
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[16]) {
    const uint4 v = *reinterpret_cast<const uint4*>(w + ((h * kTileRows + row) << 4));
    const Codec<4>::ZM zm = Codec<4>::zmagic(z);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 t[4];
      Codec<4>::word(ww[j], zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[4 * j + i] = t[i];
    }
  }
};
template <> struct StageDecode<8> {
  // stage = [4 units][128 rows][16 B]; thread (row, h) owns units 2h, 2h+1
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[16]) {
    const Codec<8>::ZM zm = Codec<8>::zmagic(z);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint4 v = *reinterpret_cast<const uint4*>(w + (((2 * h + u) * kTileRows + row) << 4));
      const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        d[8 * u + 2 * j] = __hsub2(as_h2(prmt(ww[j], 0x64646464u, 0x4140u)), as_h2(zm.m));
        d[8 * u + 2 * j + 1] = __hsub2(as_h2(prmt(ww[j], 0x64646464u, 0x4342u)), as_h2(zm.m));
      }
    }
  }
};
template <> struct StageDecode<2> {
  // stage = [1 unit][128 rows][16 B]; thread (row, h) owns words 2h, 2h+1 of the row's vector
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[16]) {
    const uint2 v = *reinterpret_cast<const uint2*>(w + (row << 4) + (h << 3));
    const Codec<2>::ZM zm = Codec<2>::zmagic(z);
    const uint32_t ww[2] = {v.x, v.y};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      __half2 t[4];
      Codec<2>::half_word(ww[j], zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[8 * j + i] = t[i];
      Codec<2>::half_word(ww[j] >> 8, zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[8 * j + 4 + i] = t[i];
    }
  }
};

template <int BITS, int NB, bool POST>
__global__ void __launch_bounds__(kTcThreads, (POST && NB <= 16) ? 2 : 1) qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                  const TcParams p) {
  using Cfg = TcCfg<BITS, NB, POST>;
  constexpr int NS = Cfg::kStages;
  constexpr int NA = kASlots;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[NS], bar_empty[NS], bar_afull[NA], bar_aempty[NA], bar_dfull[2], bar_dempty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, mtile = blockIdx.y, split = blockIdx.z, S = gridDim.z;
  const int kb0 = (int)(((long long)split * p.kblocks) / S);
  const int kb1 = (int)(((long long)(split + 1) * p.kblocks) / S);
  const int nkb = kb1 - kb0;

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t x_off = 0;
  const uint32_t w_off = NS * Cfg::kXBytes;
  const uint32_t z_off = w_off + NS * Cfg::kWBytes;
  const uint32_t s_off = z_off + NS * Cfg::kZBytes;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&bar_full[i]), 1);
      mbar_init(smem_u32(&bar_empty[i]), 1);
    }
    for (int i = 0; i < NA; ++i) {
      mbar_init(smem_u32(&bar_afull[i]), kDecodeWarps);
      mbar_init(smem_u32(&bar_aempty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bar_dfull[i]), 1);
      mbar_init(smem_u32(&bar_dempty[i]), 4);
    }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_holder), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  volatile int* abortp = &abort_flag;
  grid_launch_dependents();

  const bool has_z = p.qz != nullptr;
  const bool has_s = p.qs != nullptr;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_x);
      const uint32_t tx = Cfg::kWBytes + Cfg::kXBytes + (has_z ? Cfg::kZBytes : 0) + ((!POST && has_s) ? Cfg::kSBytes : 0);
      const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(p.qw) + (size_t)tile * p.kblocks * Cfg::kWBytes;
      auto issue_weights = [&](int i) {
        const int s = i % NS, kb = kb0 + i;
        const uint32_t bar = smem_u32(&bar_full[s]);
        mbar_arrive_expect_tx(bar, tx);
        tma_bulk_g2s(sbase + w_off + s * Cfg::kWBytes, wsrc + (size_t)kb * Cfg::kWBytes, Cfg::kWBytes, bar);
        const int g = kb / p.kb_per_group;
        if (has_z)
          tma_bulk_g2s(sbase + z_off + s * Cfg::kZBytes, p.qz + ((size_t)tile * p.groups + g) * kTileRows, Cfg::kZBytes, bar);
        if (!POST && has_s)
          tma_bulk_g2s(sbase + s_off + s * Cfg::kSBytes, p.qs + ((size_t)tile * p.groups + g) * kTileRows, Cfg::kSBytes, bar);
      };
      auto issue_x = [&](int i) {
        const int s = i % NS, kb = kb0 + i;
        tma_tensor_2d_g2s(sbase + x_off + s * Cfg::kXBytes, &tmap_x, kb * 64, mtile * NB, smem_u32(&bar_full[s]));
      };
      // weights never depend on the preceding kernel: start them before the dependency wait
      const int pro = nkb < NS ? nkb : NS;
      for (int i = 0; i < pro; ++i) issue_weights(i);
      grid_dependency_wait();
      for (int i = 0; i < pro; ++i) issue_x(i);
      for (int i = NS; i < nkb; ++i) {
        const int s = i % NS;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ((i / NS) & 1) ^ 1, abortp)) break;
        issue_weights(i);
        issue_x(i);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16_m128(NB);
      int seg = 0;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % NS, a = i % NA, kb = kb0 + i;
        const bool new_seg = (i == 0) || (POST && (kb % p.kb_per_group == 0));
        const bool end_seg = (i == nkb - 1) || (POST && ((kb + 1) % p.kb_per_group == 0));
        const int d = POST ? (seg & 1) : 0;
        if (!mbar_wait(smem_u32(&bar_full[s]), (i / NS) & 1, abortp)) break;
        if (!mbar_wait(smem_u32(&bar_afull[a]), (i / NA) & 1, abortp)) break;
        if (POST && new_seg) {
          if (!mbar_wait(smem_u32(&bar_dempty[d]), ((seg >> 1) & 1) ^ 1, abortp)) break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + kAColsTotal + d * NB;
        const uint32_t a_tmem = tmem_base + a * 32;
        const uint64_t bdesc = smem_desc_k_sw128(sbase + x_off + s * Cfg::kXBytes);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma_f16_ts(d_tmem, a_tmem + 8 * j, bdesc + (uint64_t)(2 * j), idesc, (new_seg && j == 0) ? 0u : 1u);
        mma_commit(smem_u32(&bar_empty[s]));
        mma_commit(smem_u32(&bar_aempty[a]));
        if (end_seg) {
          mma_commit(smem_u32(&bar_dfull[d]));
          ++seg;
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 4 + kDecodeWarps) {
    // ------------------------------ decode warps ------------------------------
    const int q = warp & 3, h = (warp - 4) >> 2;
    const int row = q * 32 + lane;
    for (int i = 0; i < nkb; ++i) {
      const int s = i % NS, a = i % NA;
      if (!mbar_wait(smem_u32(&bar_full[s]), (i / NS) & 1, abortp)) break;
      const uint32_t z = has_z ? (uint32_t)gbase[z_off + s * Cfg::kZBytes + row] : p.zconst;
      __half2 d[16];
      StageDecode<BITS>::run(gbase + w_off + s * Cfg::kWBytes, row, h, z, d);
      uint32_t r[16];
      if (!POST && has_s) {
        const __half2 s2 = __half2half2(*reinterpret_cast<const __half*>(gbase + s_off + s * Cfg::kSBytes + row * 2));
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = as_u32(__hmul2(d[j], s2));
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = as_u32(d[j]);
      }
      if (!mbar_wait(smem_u32(&bar_aempty[a]), ((i / NA) & 1) ^ 1, abortp)) break;
      tc_fence_after();
      tmem_st_x16(tmem_base + ((uint32_t)(q * 32) << 16) + a * 32 + h * 16, r);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_afull[a]));
    }
  } else if (warp >= 12) {
    // ------------------------------ scale / epilogue warps --------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int n = tile * kTileRows + row;
    const int m0 = mtile * NB;
    // one 16-column chunk of results: fp16 output, or fp32 split-K partial
    auto store_chunk = [&](int c, const float* v) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int m = m0 + c + j;
        if (m < p.m) {
          if (S == 1) {
            if (n < p.n) p.y[(size_t)m * p.n + n] = __float2half_rn(v[j]);
          } else {
            p.partial[((size_t)split * p.m + m) * p.npad + n] = v[j];
          }
        }
      }
    };
    bool ok = true;
    if (POST) {
      float acc[NB];
#pragma unroll
      for (int j = 0; j < NB; ++j) acc[j] = 0.f;
      int seg = 0;
      for (int i = 0; i < nkb; ++i) {
        const int kb = kb0 + i;
        const bool end_seg = (i == nkb - 1) || ((kb + 1) % p.kb_per_group == 0);
        if (!end_seg) continue;
        const int g = kb / p.kb_per_group;
        const float sval = has_s ? __half2float(p.qs[((size_t)tile * p.groups + g) * kTileRows + row]) : 1.f;
        const int d = seg & 1;
        if (!mbar_wait(smem_u32(&bar_dfull[d]), (seg >> 1) & 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + kAColsTotal + d * NB;
#pragma unroll
        for (int c = 0; c < NB; c += 16) {
          uint32_t v[16];
          tmem_ld_x16(taddr + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c + j] = fmaf(sval, __uint_as_float(v[j]), acc[c + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_dempty[d]));
        ++seg;
      }
      if (ok) {
        grid_dependency_wait();  // y and the workspace may still be in use by the preceding kernel
#pragma unroll
        for (int c = 0; c < NB; c += 16) store_chunk(c, &acc[c]);
      }
    } else {
      ok = mbar_wait(smem_u32(&bar_dfull[0]), 0, abortp);
      if (ok) {
        tc_fence_after();
        grid_dependency_wait();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + kAColsTotal;
#pragma unroll 1
        for (int c = 0; c < NB; c += 16) {
          uint32_t v[16];
          tmem_ld_x16(taddr + c, v);
          tmem_wait_ld();
          float f[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
          store_chunk(c, f);
        }
        tc_fence_before();
      }
    }
    if (ok && S > 1) {
      // split-K: every epilogue warp publishes its 32 rows, the LAST warp to arrive (over all
      // splits and all four row quarters) sums the partials of the whole tile in split order.
      __threadfence();
      __syncwarp();
      unsigned prev = 0;
      unsigned* ctr = p.counters + (mtile * gridDim.x + tile);
      if (lane == 0) prev = atomicAdd(ctr, 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev == (unsigned)(4 * S - 1)) {
        __threadfence();
        for (int qq = 0; qq < 4; ++qq) {
          const int nn = tile * kTileRows + qq * 32 + lane;
          for (int j = 0; j < NB; ++j) {
            const int m = m0 + j;
            if (m >= p.m) break;
            float sum = 0.f;
            for (int sp = 0; sp < S; ++sp) sum += __ldcg(p.partial + ((size_t)sp * p.m + m) * p.npad + nn);
            if (nn < p.n) p.y[(size_t)m * p.n + nn] = __float2half_rn(sum);
          }
        }
        if (lane == 0) *ctr = 0u;
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  if (*abortp) {
    // give bulk copies still in flight time to land before shared memory is released (bounded)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 1u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
template <int BITS, int NB, bool POST>
static cudaError_t launch_cfg(const CUtensorMap& tm, const TcParams& p, dim3 grid, bool pdl, cudaStream_t st) {
  using Cfg = TcCfg<BITS, NB, POST>;
  auto kern = qgemm_tc_kernel<BITS, NB, POST>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tm, p);
}

template <int BITS>
static cudaError_t launch_nb(const CUtensorMap& tm, const TcParams& p, int nb, bool post, dim3 grid, bool pdl,
                             cudaStream_t st) {
  if (post) {
    switch (nb) {
      case 16: return launch_cfg<BITS, 16, true>(tm, p, grid, pdl, st);
      case 32: return launch_cfg<BITS, 32, true>(tm, p, grid, pdl, st);
      case 64: return launch_cfg<BITS, 64, true>(tm, p, grid, pdl, st);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (nb) {
    case 16: return launch_cfg<BITS, 16, false>(tm, p, grid, pdl, st);
    case 64: return launch_cfg<BITS, 64, false>(tm, p, grid, pdl, st);
    case 128: return launch_cfg<BITS, 128, false>(tm, p, grid, pdl, st);
    case 256: return launch_cfg<BITS, 256, false>(tm, p, grid, pdl, st);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_gemm_tc(const CUtensorMap& tmap_x, const TcParams& p, int bits, int nb, bool post, dim3 grid,
                           bool pdl, cudaStream_t st) {
  switch (bits) {
    case 2: return launch_nb<2>(tmap_x, p, nb, post, grid, pdl, st);
    case 4: return launch_nb<4>(tmap_x, p, nb, post, grid, pdl, st);
    case 8: return launch_nb<8>(tmap_x, p, nb, post, grid, pdl, st);
    default: return cudaErrorInvalidValue;
  }
}

size_t gemm_tc_smem_bytes(int bits, int nb, bool post) {
  auto stage = [&](int wb) { return wb + nb * 128 + 128 + 256; };
  const int wb = 128 * 64 * bits / 8;
  const int budget = nb <= 64 ? 100 * 1024 : 200 * 1024;
  int ns = budget / stage(wb);
  ns = ns > 12 ? 12 : (ns < 3 ? 3 : ns);
  (void)post;
  return 1024 + (size_t)ns * stage(wb);
}

}  // namespace qfb
