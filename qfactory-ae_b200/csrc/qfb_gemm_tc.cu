// Tensor-core path: y^T[n, m] = W[n, :] . x[m, :] with the WEIGHT rows as the UMMA M dimension
// (128) and the activation batch as the UMMA N dimension (16..256), so that even a single
// activation row fills the 5th-generation tensor core.  No counterpart in the reference, whose
// kernels are CUDA-core GEMVs only (qfactory/include/gptq_gemv.h:14-154).
//
// Data flow of one CTA (one 128-row weight tile x one batch tile x one K split), in stages
// of 128 k:
//
//   TMA (2 threads)   packed weights (one contiguous bulk copy per stage) and the fp16
//                     activation tile (two 128-byte-swizzled tensor boxes) -> two independent
//                     shared-memory rings; the weight ring is released by the decode warps as
//                     soon as the codes are in registers, the activation ring by MMA completion
//   decode (8 or 16 warps)  packed codes -> exact (q - z) fp16 pairs in registers (LOP3 / PRMT magic
//                     numbers) -> tcgen05.st into TENSOR MEMORY as the A operand.  The fp16
//                     weights never touch shared memory, whose bandwidth could not carry the
//                     4x-expanded stream at HBM rate.  Thread (row, half) owns 64 codes of a stage.
//   MMA (1-2 threads) tcgen05.mma kind::f16, A from tensor memory, B (activations) from shared
//                     memory, fp32 accumulators in tensor memory.  ONE tcgen05.commit per stage
//                     feeds every consumer of "stage done".  With per-stage accumulators (POST)
//                     two threads issue alternate stages, since a skinny MMA costs more to issue
//                     than to execute.
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

constexpr int kStageK = 128;              // k per pipeline stage
constexpr int kStepsPerStage = kStageK / 16;
constexpr int kAColsPerSlot = kStageK / 2;  // one 32-bit column holds two fp16 k
constexpr int kDecodeWarps = 8;
// sleep between polls of a barrier that is not ready yet, per role (ns)
constexpr unsigned kSleepScale = 100, kSleepProducer = 100, kSleepMma = 20, kSleepDecode = 20;

// DG = decode groups: 1 -> 8 decode warps (512 threads, two CTAs per SM for the smallest batch
// tile), 2 -> two groups of 8 decode warps that take alternate stages (768 threads, one CTA per SM).
template <int BITS, int NB, bool POST, int DG>
struct TcCfg {
  static constexpr int kThreads = 128 + 256 * DG + 128;
  static constexpr int kScaleWarp0 = 4 + 8 * DG;
  static constexpr int kWBytes = 128 * kStageK * BITS / 8;
  static constexpr int kXBytes = NB * kStageK * 2;
  static constexpr int kZSlot = 256;   // effective zeros of a stage: 128 rows x up to 2 groups
  static constexpr int kSSlot = 512;   // fp16 scales of a stage (PRE mode only)
  static constexpr int kQBytes = kZSlot + (POST ? 0 : kSSlot);
  // two CTAs share an SM (98 KB of shared memory, 256 tensor-memory columns, 64 registers each):
  // the narrow per-stage-accumulator tiles, and with one decode group the scale-in-the-decode tiles
  // up to 128 columns (two independent pipelines hide each other's hand-off latencies)
  static constexpr bool kTwoPerSM = DG == 1 && (POST ? NB <= 32 : NB <= 128);
  static constexpr int kBudget = kTwoPerSM ? 98 * 1024 : 224 * 1024;
  static constexpr int kXStages = (kTwoPerSM && !POST) ? (NB <= 32 ? 6 : NB <= 64 ? 3 : 2)
                                  : NB <= 16 ? 6 : NB <= 32 ? (POST ? 4 : 8) : NB <= 64 ? 6 : NB <= 128 ? 4 : (BITS == 8 ? 2 : 3);
  static constexpr int kWStagesRaw = (kBudget - kXStages * kXBytes) / (kWBytes + kQBytes);
  static constexpr int kWStages = kWStagesRaw > 16 ? 16 : kWStagesRaw;
  static constexpr int kTmemCols = kTwoPerSM ? 256 : 512;
  // ring of R slots in tensor memory: A operand (64 columns) + in POST mode one accumulator each
  static constexpr int kSlotCols = kAColsPerSlot + (POST ? NB : 0);
  // PRE mode with skinny MMAs (N <= 128) is issue-bound too: two issuers, one accumulator each
  static constexpr int kIssuers = POST ? 2 : ((NB <= 128 && !(kTwoPerSM && NB > 64)) ? 2 : 1);
  static constexpr int kRingRaw = (kTmemCols - (POST ? 0 : kIssuers * NB)) / kSlotCols;
  static constexpr int kRingCap = kXStages < 6 ? kXStages : 6;   // never deeper than the activation ring
  static constexpr int kRing = kRingRaw > kRingCap ? kRingCap : kRingRaw;
  static constexpr int kDBase = kRing * kAColsPerSlot;
  static constexpr size_t kSmemBytes = 1024 + (size_t)kXStages * kXBytes + (size_t)kWStages * (kWBytes + kQBytes);
  static_assert(kWStages >= 2, "weight ring too shallow");
  static_assert(kRing >= 2, "need at least two tensor-memory slots");
  static_assert(kDBase + (POST ? kRing * NB : kIssuers * NB) <= kTmemCols, "tensor memory over-subscribed");
};

// ---- decode of the 64 codes thread (row, h) owns in a 128-k stage -> 32 fp16 pairs ------
template <int BITS> struct StageDecode;
template <> struct StageDecode<4> {
  // stage = [4 units][128 rows][16 B]; thread owns units 2h, 2h+1
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const Codec<4>::ZM zm = Codec<4>::zmagic(z);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint4 v = *reinterpret_cast<const uint4*>(w + (((2 * h + u) * kTileRows + row) << 4));
      const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 t[4];
        Codec<4>::word(ww[j], zm, t);
#pragma unroll
        for (int i = 0; i < 4; ++i) d[16 * u + 4 * j + i] = t[i];
      }
    }
  }
};
// Fragment layouts: stage = [2 halves of 64 rows][8 k-steps of 128 * BITS bytes] (qfb_common.cuh).
// Row wt*64 + rb*16 + hh*8 + g owns, in the word frag_word_of(rb, hh) of lane g*4+t, the codes of
// k 4t..4t+3 of a step: two exact fp16 pairs in k order per word.
template <int BITS> struct StageDecodeFragment;
template <> struct StageDecodeFragment<4> {
  // nibbles 0,4,2,6 (hh = 0) or 1,5,3,7 (hh = 1): two LOP3 with the row's mask / magic
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const Codec<4>::ZM zm = Codec<4>::zmagic(z);
    const int wt = row >> 6, rb = (row >> 4) & 3, hh = (row >> 3) & 1, g = row & 7;
    const uint32_t mask = hh ? 0x00f000f0u : 0x000f000fu, magic = hh ? 0x54005400u : 0x64006400u;
    const __half2 zs = as_h2(hh ? zm.hi : zm.lo);
    const uint8_t* base = w + wt * 4096 + (4 * h) * 512 + g * 64 + rb * 4;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t word = *reinterpret_cast<const uint32_t*>(base + ks * 512 + t * 16);
        d[ks * 8 + t * 2] = __hsub2(as_h2(lop3_and_or(word, mask, magic)), zs);
        d[ks * 8 + t * 2 + 1] = __hsub2(as_h2(lop3_and_or(word >> 8, mask, magic)), zs);
      }
  }
};
template <> struct StageDecodeFragment<8> {
  // one word = the row's four bytes of k 4t..4t+3
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const Codec<8>::ZM zm = Codec<8>::zmagic(z);
    const int wt = row >> 6, rb = (row >> 4) & 3, hh = (row >> 3) & 1, g = row & 7;
    const uint8_t* base = w + wt * 8192 + (4 * h) * 1024 + frag_word_offset(8, g * 4, rb * 2 + hh);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t word = *reinterpret_cast<const uint32_t*>(base + ks * 1024 + t * 16);
        d[ks * 8 + t * 2] = __hsub2(as_h2(prmt(word, 0x64646464u, 0x4140u)), as_h2(zm.m));
        d[ks * 8 + t * 2 + 1] = __hsub2(as_h2(prmt(word, 0x64646464u, 0x4342u)), as_h2(zm.m));
      }
  }
};
template <> struct StageDecodeFragment<2> {
  // one word = two row blocks; the row's fields sit at bit o = 4 (rb & 1) + 2 hh of each byte pair
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const Codec<2>::ZM zm = Codec<2>::zmagic(z);
    const int wt = row >> 6, rb = (row >> 4) & 3, hh = (row >> 3) & 1, g = row & 7;
    const int oi = (rb & 1) * 2 + hh;  // bit offset / 2
    const uint32_t mask = 0x00030003u << (2 * oi);
    const uint32_t magic = oi == 0 ? 0x64006400u : oi == 1 ? 0x5C005C00u : oi == 2 ? 0x54005400u : 0x4C004C00u;
    const __half2 zs = as_h2(oi == 0 ? zm.m[0] : oi == 1 ? zm.m[1] : oi == 2 ? zm.m[2] : zm.m[3]);
    const uint8_t* base = w + wt * 2048 + (4 * h) * 256 + g * 32 + (rb >> 1) * 4;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t word = *reinterpret_cast<const uint32_t*>(base + ks * 256 + t * 8);
        d[ks * 8 + t * 2] = __hsub2(as_h2(lop3_and_or(word, mask, magic)), zs);
        d[ks * 8 + t * 2 + 1] = __hsub2(as_h2(lop3_and_or(word >> 8, mask, magic)), zs);
      }
  }
};
template <> struct StageDecodeFragment<3> {
  // word j of lane g*4+t sits in plane j (128 bytes) of the k-step (384 bytes).  Row blocks 0..2: word rb, the
  // row's fields at bit offset 0 (rows g) or 3 (rows g + 8) for k 4t, 4t+1 and 9 bits higher for k 4t+2, 4t+3.
  // Row block 3: offset 6 of words 0 / 1 (rows g) and of word 2 (rows g + 8, k 4t, 4t+1); rows g + 8,
  // k 4t+2, 4t+3 are collected from the spare bits 15 / 31 of the three words.
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const int wt = row >> 6, rb = (row >> 4) & 3, hh = (row >> 3) & 1, g = row & 7;
    const uint8_t* base = w + wt * 3072 + (4 * h) * 384 + g * 16;
    if (rb < 3) {
      // the field as the low mantissa bits of 2^(10 - offset): exact q + 2^(10 - offset), minus the same with z
      const uint32_t mask = hh ? 0x00380038u : 0x00070007u, magic = hh ? 0x58005800u : 0x64006400u;
      const __half2 zs = as_h2(magic | ((z << (hh ? 3 : 0)) * 0x00010001u));
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint32_t word = *reinterpret_cast<const uint32_t*>(base + ks * 384 + rb * 128 + t * 4);
          d[ks * 8 + t * 2] = __hsub2(as_h2(lop3_and_or(word, mask, magic)), zs);
          d[ks * 8 + t * 2 + 1] = __hsub2(as_h2(lop3_and_or(word >> 9, mask, magic)), zs);
        }
    } else {
      const uint32_t mask = 0x01C001C0u, magic = 0x4C004C00u;
      const __half2 zs = as_h2(magic | ((z << 6) * 0x00010001u));
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint8_t* p = base + ks * 384 + t * 4;
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(p), w1 = *reinterpret_cast<const uint32_t*>(p + 128),
                         w2 = *reinterpret_cast<const uint32_t*>(p + 256);
          const uint32_t spare = ((w0 >> 9) & 0x00400040u) | ((w1 >> 8) & 0x00800080u) | ((w2 >> 7) & 0x01000100u);
          const uint32_t lo = hh ? (w2 & mask) : (w0 & mask), hi = hh ? spare : (w1 & mask);
          d[ks * 8 + t * 2] = __hsub2(as_h2(lo | magic), zs);
          d[ks * 8 + t * 2 + 1] = __hsub2(as_h2(hi | magic), zs);
        }
    }
  }
};
template <> struct StageDecode<8> {
  // stage = [8 units][128 rows][16 B]; thread owns units 4h .. 4h+3
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const Codec<8>::ZM zm = Codec<8>::zmagic(z);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint4 v = *reinterpret_cast<const uint4*>(w + (((4 * h + u) * kTileRows + row) << 4));
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
  // stage = [2 units][128 rows][16 B]; thread owns unit h
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const uint4 v = *reinterpret_cast<const uint4*>(w + ((h * kTileRows + row) << 4));
    const Codec<2>::ZM zm = Codec<2>::zmagic(z);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
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
template <> struct StageDecode<3> {
  // stage = one 3-bit unit = [3 vectors][128 rows][16 B]: two 2-bit-plane vectors and the
  // 1-bit-plane vector; thread owns 2-bit vector h and words 2h, 2h+1 of the plane vector
  __device__ static __forceinline__ void run(const uint8_t* w, int row, int h, uint32_t z, __half2 (&d)[32]) {
    const uint4 a = *reinterpret_cast<const uint4*>(w + ((h * kTileRows + row) << 4));
    const uint2 b = *reinterpret_cast<const uint2*>(w + ((2 * kTileRows + row) << 4) + (h << 3));
    const Codec<3>::ZM zm = Codec<3>::zmagic(z);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    const uint32_t bw[2] = {b.x, b.y};
#pragma unroll
    for (int j = 0; j < 2; ++j) {  // 32 codes: 2-bit words aw[2j], aw[2j+1] with plane word bw[j]
      __half2 t[4];
      Codec<3>::half_word(aw[2 * j], bw[j] << 2, zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[16 * j + i] = t[i];
      Codec<3>::half_word(aw[2 * j] >> 8, bw[j] << 1, zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[16 * j + 4 + i] = t[i];
      Codec<3>::half_word(aw[2 * j + 1], bw[j] >> 6, zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[16 * j + 8 + i] = t[i];
      Codec<3>::half_word(aw[2 * j + 1] >> 8, bw[j] >> 7, zm, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) d[16 * j + 12 + i] = t[i];
    }
  }
};

// Sum of the split-K partials of one warp's 32 rows (lane = row) over all S splits, in split order,
// rounded to fp16 into y.  base0 -> partial of split 0, batch column 0, this lane's row; `sstride`
// floats between splits, `cstride` between batch columns; ydst -> y[first batch row][this lane's
// output feature], `ystride` halfs between batch rows; `cols` = valid batch columns.
// Loads in flight per round: 32 batch columns of one split where one accumulator spans K (this
// warp's own sums, the same bits it published, are re-read from tensor memory at taddr_own instead,
// plus the second issuer's accumulator when `two`); 8 columns of four splits for the narrow
// per-stage-accumulator tiles, which have many splits.  (A column at a time cost one round trip per
// column: the reduce of a wide tile then took longer than its MMAs.  Measured against 16 columns of
// two splits and against a non-inlined function: this form is 2-7 % faster on every batch size.)
template <int NB, bool POST>
__device__ __forceinline__ void splitk_reduce(const float* base0, size_t sstride, size_t cstride, int S, int split, int cols,
                                           bool row_ok, __half* ydst, size_t ystride, uint32_t taddr_own, bool two) {
  constexpr int CW = POST ? 8 : 32, SPB = POST ? 4 : 1;
#pragma unroll 1
  for (int c0 = 0; c0 < NB; c0 += CW) {
    if (c0 >= cols) break;
    float sum[CW];
#pragma unroll
    for (int j = 0; j < CW; ++j) sum[j] = 0.f;
#pragma unroll 1
    for (int sp = 0; sp < S; sp += SPB) {
      float t[SPB][CW];
#pragma unroll
      for (int u = 0; u < SPB; ++u) {
        if (!POST && sp + u == split) continue;   // filled below, without a load
#pragma unroll
        for (int j = 0; j < CW; ++j)
          t[u][j] = (sp + u < S && c0 + j < cols) ? __ldcg(base0 + (size_t)(sp + u) * sstride + (size_t)(c0 + j) * cstride) : 0.f;
      }
      if (!POST) {
#pragma unroll
        for (int u = 0; u < SPB; ++u)
          if (sp + u == split) {
#pragma unroll
            for (int c = 0; c < CW; c += 16) {
              uint32_t v[16], v2[16];
              tmem_ld_x16(taddr_own + c0 + c, v);
              if (two) tmem_ld_x16(taddr_own + NB + c0 + c, v2);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) t[u][c + j] = __uint_as_float(v[j]) + (two ? __uint_as_float(v2[j]) : 0.f);
            }
          }
      }
#pragma unroll
      for (int u = 0; u < SPB; ++u)
#pragma unroll
        for (int j = 0; j < CW; ++j)
          if (sp + u < S) sum[j] += t[u][j];
    }
#pragma unroll
    for (int j = 0; j < CW; ++j)
      if (c0 + j < cols && row_ok) ydst[(size_t)(c0 + j) * ystride] = __float2half_rn(sum[j]);
  }
}

// FRAG = the layer is in the fragment layout (a build of its own: with both decoders behind a run-time branch in
// the decode loop the compiler allots registers for the larger of the two)
// ASYM = the layer has scales AND zero points (the common case; a build of its own for the same reason; used
// where the scale is applied in the decode)
template <int BITS, int NB, bool POST, int DG, bool FRAG, bool ASYM>
__global__ void __launch_bounds__(TcCfg<BITS, NB, POST, DG>::kThreads, (TcCfg<BITS, NB, POST, DG>::kTwoPerSM ? 2 : 1))
qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const TcParams p) {
  using Cfg = TcCfg<BITS, NB, POST, DG>;
  constexpr int NS = Cfg::kWStages;   // weight ring
  constexpr int NX = Cfg::kXStages;   // activation ring
  constexpr int R = Cfg::kRing;       // tensor-memory slot ring

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_wfull[NS], bar_wempty[NS], bar_xfull[NX], bar_xempty[NX];
  __shared__ uint64_t bar_afull[R], bar_done[R], bar_dempty[R], bar_final;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Two grid shapes.  Uniform: grid (row tiles, batch tiles, K splits).  Tail-split (p.tail_split > 0,
  // one-dimensional grid): the first p.full_units CTAs own a whole (row tile, batch tile) unit each,
  // the remaining units (the last, partly filled wave of a launch) are cut into p.tail_split K ranges
  // of one CTA each, so that the tail costs a fraction of a wave.
  int tile = blockIdx.x, mtile = blockIdx.y, split = blockIdx.z, S = gridDim.z;
  int unit_ctr = mtile * gridDim.x + tile;   // index of this unit's arrival counters
  int tail_unit = -1;                        // >= 0: this CTA writes compact partials of tail unit `tail_unit`
  if (p.tail_split > 0) {
    const int c = blockIdx.x;
    int unit = c;
    split = 0;
    S = 1;
    if (c >= p.full_units) {
      const int j = c - p.full_units;
      tail_unit = j / p.tail_split;
      unit = p.full_units + tail_unit;
      split = j - tail_unit * p.tail_split;
      S = p.tail_split;
      unit_ctr = tail_unit;
    }
    tile = unit / p.mtiles;
    mtile = unit - tile * p.mtiles;
  }
  const int kb0 = (int)(((long long)split * p.kblocks) / S);
  const int kb1 = (int)(((long long)(split + 1) * p.kblocks) / S);
  const int nkb = kb1 - kb0;

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
  constexpr uint32_t x_off = 0;
  constexpr uint32_t w_off = NX * Cfg::kXBytes;
  constexpr uint32_t z_off = w_off + NS * Cfg::kWBytes;
  constexpr uint32_t s_off = z_off + NS * Cfg::kZSlot;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&bar_wfull[i]), 1);
      mbar_init(smem_u32(&bar_wempty[i]), kDecodeWarps);  // the eight warps of the group that decodes the stage
    }
    for (int i = 0; i < NX; ++i) {
      mbar_init(smem_u32(&bar_xfull[i]), 1);
      mbar_init(smem_u32(&bar_xempty[i]), 1);
    }
    for (int i = 0; i < R; ++i) {
      mbar_init(smem_u32(&bar_afull[i]), kDecodeWarps);
      mbar_init(smem_u32(&bar_done[i]), 1);
      mbar_init(smem_u32(&bar_dempty[i]), 4);
    }
    mbar_init(smem_u32(&bar_final), Cfg::kIssuers);
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
  const long long wait_limit = p.stall_test ? 200000LL : kWaitLimitCycles;
  grid_launch_dependents();

  const bool has_z = ASYM || p.qz != nullptr;
  const bool has_s = ASYM || p.qs != nullptr;

  if (warp == 0) {
    // ------------------------------ weight producer ---------------------------
    // (never depends on the preceding kernel: no dependency wait on this path)
    if (lane == 0) {
      const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(p.qw) + ((size_t)tile * p.kblocks + kb0) * Cfg::kWBytes;
      int s = 0;
      uint32_t ph = 1;  // first pass over the ring: parity 1 of a fresh barrier passes at once
      // group of the stage's first 64 k, tracked without divisions in the loop
      const int hpg = p.halfstages_per_group;
      int g0 = (kb0 * 2) / hpg, gpos = (kb0 * 2) % hpg;
      const uint32_t ng = hpg == 1 ? 2u : 1u;
      const uint32_t zb = has_z ? ng * 128u : 0u, sb = (!POST && has_s) ? ng * 256u : 0u;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(smem_u32(&bar_wempty[s]), ph, abortp, kSleepProducer, wait_limit)) break;
        const uint32_t bar = smem_u32(&bar_wfull[s]);
        // zeros / scales of the groups this stage touches: one group, or two when the group is 64
        mbar_arrive_expect_tx(bar, Cfg::kWBytes + zb + sb + ((p.stall_test && i == 0) ? 16u : 0u));
        if (FRAG) {
          // the stage is two runs: 8 k-steps (128 * BITS bytes each) of the upper and of the lower 64 rows
          const uint8_t* f0 = reinterpret_cast<const uint8_t*>(p.qw) +
                              (((size_t)tile * 2) * (size_t)(p.kblocks * 8) + (size_t)(kb0 + i) * 8) * (128 * BITS);
          tma_bulk_g2s(sbase + w_off + s * Cfg::kWBytes, f0, Cfg::kWBytes / 2, bar);
          tma_bulk_g2s(sbase + w_off + s * Cfg::kWBytes + Cfg::kWBytes / 2,
                       f0 + (size_t)p.kblocks * 8 * (128 * BITS), Cfg::kWBytes / 2, bar);
        } else {
          tma_bulk_g2s(sbase + w_off + s * Cfg::kWBytes, wsrc + (size_t)i * Cfg::kWBytes, Cfg::kWBytes, bar);
        }
        if (zb) tma_bulk_g2s(sbase + z_off + s * Cfg::kZSlot, p.qz + ((size_t)tile * p.groups + g0) * kTileRows, zb, bar);
        if (sb) tma_bulk_g2s(sbase + s_off + s * Cfg::kSSlot, p.qs + ((size_t)tile * p.groups + g0) * kTileRows, sb, bar);
        gpos += 2;
        if (hpg == 1) { g0 += 2; gpos = 0; } else if (gpos >= hpg) { gpos = 0; ++g0; }
        if (++s == NS) { s = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    // ------------------------------ activation producer -----------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_x);
      grid_dependency_wait();
      int s = 0;
      uint32_t ph = 1;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(smem_u32(&bar_xempty[s]), ph, abortp, kSleepProducer, wait_limit)) break;
        const uint32_t bar = smem_u32(&bar_xfull[s]);
        const uint32_t dst = sbase + x_off + s * Cfg::kXBytes;
        mbar_arrive_expect_tx(bar, Cfg::kXBytes);
        tma_tensor_2d_g2s(dst, &tmap_x, (kb0 + i) * kStageK, mtile * NB, bar);
        tma_tensor_2d_g2s(dst + NB * 128, &tmap_x, (kb0 + i) * kStageK + 64, mtile * NB, bar);
        if (++s == NX) { s = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1 || (warp == 2 && Cfg::kIssuers == 2)) {
    // ------------------------------ MMA issuer(s) -----------------------------
    // Issuer e takes stages e, e + kIssuers, ...  POST: every stage has its own accumulator.
    // PRE: every issuer has its own accumulator over all its stages; the epilogue adds them.
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16_m128(NB);
      const int e = (warp == 1) ? 0 : 1;
      for (int i = e; i < nkb; i += Cfg::kIssuers) {
        const int xs = i % NX, r = i % R;
        const uint32_t phx = (uint32_t)(i / NX) & 1u, phr = (uint32_t)(i / R) & 1u;
        if (!mbar_wait(smem_u32(&bar_xfull[xs]), phx, abortp, kSleepMma, wait_limit)) break;
        if (!mbar_wait(smem_u32(&bar_afull[r]), phr, abortp, kSleepMma, wait_limit)) break;
        if (POST) {
          if (!mbar_wait(smem_u32(&bar_dempty[r]), phr ^ 1u, abortp, kSleepMma, wait_limit)) break;
        }
        tc_fence_after();
        const uint32_t a_tmem = tmem_base + r * kAColsPerSlot;
        const uint32_t d_tmem = tmem_base + Cfg::kDBase + (POST ? r * NB : e * NB);
        const uint32_t xsm = sbase + x_off + xs * Cfg::kXBytes;
        const uint64_t bd0 = smem_desc_k_sw128(xsm), bd1 = smem_desc_k_sw128(xsm + NB * 128);
        mma_f16_ts_stage8(d_tmem, a_tmem, (uint32_t)bd0, (uint32_t)bd1, (uint32_t)(bd0 >> 32), idesc,
                          POST ? 0u : (i >= Cfg::kIssuers ? 1u : 0u));
        mma_commit(smem_u32(&bar_done[r]));
      }
      mma_commit(smem_u32(&bar_final));  // every MMA this thread issued is complete
    }
    __syncwarp();
  } else if (warp >= 4 && warp < Cfg::kScaleWarp0) {
    // ------------------------------ decode warps ------------------------------
    // group `grp` takes stages grp, grp + DG, ...; inside a group thread (row, h) owns 64 codes
    const int grp = (warp - 4) >> 3;
    const int q = warp & 3, h = ((warp - 4) >> 2) & 1;
    const int row = q * 32 + lane;
    // with groups of 64 the two halves of a stage belong to different groups: half h reads
    // the second record of the stage's zero / scale slot
    const int qsel = (p.halfstages_per_group == 1 && h == 1) ? kTileRows : 0;
    constexpr bool frag = FRAG;
    // position of the row's scale / zero inside the tile's 128 (fragment layers keep them in fragment order)
    const int qrow = qsel + (frag ? frag_pos_of_row(row) : row);
    for (int i = grp; i < nkb; i += DG) {
      // ring positions and phases of stage i (NS, R, NX are compile-time constants: multiply-shift, no division)
      const int s = i % NS, r = i % R;
      const uint32_t phs = (uint32_t)(i / NS) & 1u, phr = ((uint32_t)(i / R) & 1u) ^ 1u;
      if (!mbar_wait(smem_u32(&bar_wfull[s]), phs, abortp, kSleepDecode, wait_limit)) break;
      const uint32_t z = has_z ? (uint32_t)gbase[z_off + s * Cfg::kZSlot + qrow] : p.zconst;
      __half2 d[32];
      if constexpr (FRAG) StageDecodeFragment<BITS>::run(gbase + w_off + s * Cfg::kWBytes, row, h, z, d);
      else StageDecode<BITS>::run(gbase + w_off + s * Cfg::kWBytes, row, h, z, d);
      uint32_t rr[32];
      if (!POST && has_s) {
        const __half2 s2 = __half2half2(reinterpret_cast<const __half*>(gbase + s_off + s * Cfg::kSSlot)[qrow]);
#pragma unroll
        for (int j = 0; j < 32; ++j) rr[j] = as_u32(__hmul2(d[j], s2));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) rr[j] = as_u32(d[j]);
      }
      // the packed stage is in registers: hand the shared-memory slot back to the producer
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_wempty[s]));
      // slot r was last read by the MMAs of stage i - R
      if (!mbar_wait(smem_u32(&bar_done[r]), phr, abortp, kSleepDecode, wait_limit)) break;
      // ... and the activation tile of that stage is free as well: tell its producer.  The
      // decode warps cannot fall behind the commits (the MMAs need their stores), so this
      // relay never misses a phase; R <= NX makes it reach every tile that is still needed.
      if (i >= R && (warp & 7) == 4 && lane == 0) mbar_arrive(smem_u32(&bar_xempty[(i - R) % NX]));
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + r * kAColsPerSlot + h * 32;
      tmem_st_x16(taddr, reinterpret_cast<const uint32_t(&)[16]>(rr[0]));
      tmem_st_x16(taddr + 16, reinterpret_cast<const uint32_t(&)[16]>(rr[16]));
      // publish at once: the MMAs of this stage start a whole decode earlier than with a deferred
      // hand-off, which matters more than the store latency exposed here (measured)
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_afull[r]));
    }
  } else if (warp >= Cfg::kScaleWarp0) {
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
            if (tail_unit >= 0) p.partial[(((size_t)split * p.tail_units + tail_unit) * NB + (c + j)) * kTileRows + row] = v[j];
            else p.partial[((size_t)split * p.m + m) * p.npad + n] = v[j];
          }
        }
      }
    };
    bool ok = true;
    // split-K: every epilogue warp publishes its 32 rows; per row quarter, the LAST warp to arrive
    // over all splits sums that quarter's partials in split order (splitk_reduce)
    auto finish_split = [&](uint32_t taddr_own, bool two) {
      if (S <= 1) return;
      __threadfence();
      __syncwarp();
      unsigned prev = 0;
      unsigned* ctr = p.counters + (unit_ctr * 4 + q);
      if (lane == 0) prev = atomicAdd(ctr, 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev != (unsigned)(S - 1)) return;
      __threadfence();
      const size_t sstride = tail_unit >= 0 ? (size_t)p.tail_units * NB * kTileRows : (size_t)p.m * p.npad;
      const size_t cstride = tail_unit >= 0 ? (size_t)kTileRows : (size_t)p.npad;
      const float* base0 = tail_unit >= 0 ? p.partial + (size_t)tail_unit * NB * kTileRows + row
                                          : p.partial + (size_t)m0 * p.npad + n;
      splitk_reduce<NB, POST>(base0, sstride, cstride, S, split, p.m - m0, n < p.n, p.y + (size_t)m0 * p.n + n, (size_t)p.n,
                              taddr_own, two);
      if (lane == 0) *ctr = 0u;
    };
    if (POST) {
      float acc[NB];
#pragma unroll
      for (int j = 0; j < NB; ++j) acc[j] = 0.f;
      const size_t sz_row = (size_t)tile * p.groups * kTileRows +
                            (FRAG ? frag_pos_of_row(row) : row);
      const int stages_per_group = p.halfstages_per_group >> 1;  // POST needs groups of whole stages
      int r = 0;
      uint32_t phr = 0;
      // scales are fetched two stages ahead of their use
      // group of stage kb0 + j, advanced without divisions: (gq, gr) = divmod(kb0 + j, stages_per_group)
      int gq = (kb0 + 2) / stages_per_group, gr = (kb0 + 2) % stages_per_group;
      auto scale_at = [&](int j, int grp) -> __half {
        return (has_s && j < nkb) ? p.qs[sz_row + (size_t)grp * kTileRows] : __ushort_as_half(0x3C00);
      };
      __half sc0 = scale_at(0, kb0 / stages_per_group), sc1 = scale_at(1, (kb0 + 1) / stages_per_group);
      for (int i = 0; i < nkb; ++i) {
        const float sval = __half2float(sc0);
        sc0 = sc1;
        sc1 = scale_at(i + 2, gq);
        if (++gr == stages_per_group) { gr = 0; ++gq; }
        if (!mbar_wait(smem_u32(&bar_done[r]), phr, abortp, kSleepScale, wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + Cfg::kDBase + r * NB;
        constexpr int CH = NB < 32 ? NB : 32;  // columns read back per wait
#pragma unroll
        for (int c0 = 0; c0 < NB; c0 += CH) {
          uint32_t v[CH];
#pragma unroll
          for (int c = 0; c < CH; c += 16) tmem_ld_x16(taddr + c0 + c, reinterpret_cast<uint32_t(&)[16]>(v[c]));
          tmem_wait_ld();
          if (c0 + CH == NB) {  // the accumulator is free as soon as its last chunk is in registers
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_dempty[r]));
          }
#pragma unroll
          for (int j = 0; j < CH; ++j) acc[c0 + j] = fmaf(sval, __uint_as_float(v[j]), acc[c0 + j]);
        }
        if (++r == R) { r = 0; phr ^= 1; }
      }
      if (ok) {
        grid_dependency_wait();  // y and the workspace may still be in use by the preceding kernel
#pragma unroll
        for (int c = 0; c < NB; c += 16) store_chunk(c, &acc[c]);
        finish_split(0u, false);
      }
    } else {
      ok = mbar_wait(smem_u32(&bar_final), 0, abortp, 500, wait_limit) && !*abortp;  // (an abandoned launch stores nothing)
      if (ok) {
        tc_fence_after();
        grid_dependency_wait();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + Cfg::kDBase;
        const bool two = Cfg::kIssuers == 2 && nkb >= 2;  // the second accumulator holds something
#pragma unroll 1
        for (int c = 0; c < NB; c += 16) {
          uint32_t v[16], v2[16];
          tmem_ld_x16(taddr + c, v);
          if (two) tmem_ld_x16(taddr + NB + c, v2);
          tmem_wait_ld();
          float f[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]) + (two ? __uint_as_float(v2[j]) : 0.f);
          store_chunk(c, f);
        }
        finish_split(taddr, two);
        tc_fence_before();
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();   // every role has left its loop (a role that ran out of work early must not
                     // look at the abort flag before the others had the chance to raise it)
  if (*abortp) {
    // give bulk copies still in flight time to land before shared memory is released (bounded)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 1u);
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
template <int BITS, int NB, bool POST, int DG, bool FRAG>
static cudaError_t launch_cfg_layout(const CUtensorMap& tm, const TcParams& p, dim3 grid, bool pdl, cudaStream_t st);

template <int BITS, int NB, bool POST, int DG>
static cudaError_t launch_cfg(const CUtensorMap& tm, const TcParams& p, dim3 grid, bool pdl, cudaStream_t st) {
  if (p.layout == QFB_LAYOUT_FRAGMENT) return launch_cfg_layout<BITS, NB, POST, DG, true>(tm, p, grid, pdl, st);
  return launch_cfg_layout<BITS, NB, POST, DG, false>(tm, p, grid, pdl, st);
}

template <int BITS, int NB, bool POST, int DG, bool FRAG>
static cudaError_t launch_cfg_layout(const CUtensorMap& tm, const TcParams& p, dim3 grid, bool pdl, cudaStream_t st) {
  using Cfg = TcCfg<BITS, NB, POST, DG>;
  auto kern = qgemm_tc_kernel<BITS, NB, POST, DG, FRAG, false>;
  // scale-in-the-decode mode: the common case of scales and zero points present has a build of its own (measured:
  // 2-6 % faster from 64 rows up; with per-stage accumulators the same specialisation was 3 % slower, not used)
  if constexpr (!POST) {
    if (p.qz && p.qs) kern = qgemm_tc_kernel<BITS, NB, POST, DG, FRAG, true>;
  }
  // the attribute belongs to the (function, device) pair: set it on every launch, it is cheap
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tm, p);
}

template <int BITS, int DG>
static cudaError_t launch_nb(const CUtensorMap& tm, const TcParams& p, int nb, bool post, dim3 grid, bool pdl,
                             cudaStream_t st) {
  if (post) {
    if (DG != 1) return cudaErrorInvalidValue;  // (narrow batch tiles: one decode group only)
    switch (nb) {
      case 16: return launch_cfg<BITS, 16, true, 1>(tm, p, grid, pdl, st);
      case 32: return launch_cfg<BITS, 32, true, 1>(tm, p, grid, pdl, st);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (nb) {
    case 64: return launch_cfg<BITS, 64, false, DG>(tm, p, grid, pdl, st);
    case 128: return launch_cfg<BITS, 128, false, DG>(tm, p, grid, pdl, st);
    case 256: return launch_cfg<BITS, 256, false, DG>(tm, p, grid, pdl, st);
    default: return cudaErrorInvalidValue;
  }
}

template <int DG>
static cudaError_t launch_bits(const CUtensorMap& tmap_x, const TcParams& p, int bits, int nb, bool post, dim3 grid,
                               bool pdl, cudaStream_t st) {
  switch (bits) {
    case 2: return launch_nb<2, DG>(tmap_x, p, nb, post, grid, pdl, st);
    case 3: return launch_nb<3, DG>(tmap_x, p, nb, post, grid, pdl, st);
    case 4: return launch_nb<4, DG>(tmap_x, p, nb, post, grid, pdl, st);
    case 8: return launch_nb<8, DG>(tmap_x, p, nb, post, grid, pdl, st);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_gemm_tc(const CUtensorMap& tmap_x, const TcParams& p, int bits, int nb, bool post, int decode_groups,
                           dim3 grid, bool pdl, cudaStream_t st) {
  // two decode groups (768 threads, one CTA per SM) where the scale is applied in the decode:
  // measured +10-17 % from 33 rows up, bit-identical results; three groups (1024 threads, 64
  // registers) were 3-6 % slower than two, and the narrow per-stage-accumulator tiles gain nothing
  if (decode_groups == 2 && !post) return launch_bits<2>(tmap_x, p, bits, nb, post, grid, pdl, st);
  return launch_bits<1>(tmap_x, p, bits, nb, post, grid, pdl, st);
}

}  // namespace qfb
