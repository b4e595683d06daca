// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernel uses:
// mbarriers, bulk (TMA) copies, tensor memory (TMEM) management and tcgen05 MMA.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qfb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A waiting thread may stay suspended in hardware for up to this long per attempt (it resumes
// at once when the phase completes), so idle roles do not burn issue slots polling.
constexpr uint32_t kSuspendHintNs = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after ~1 s of polling (or as soon as another thread of the CTA
// has given up), raising *abort_flag so every role of the CTA drains and exits.
constexpr long long kWaitLimitCycles = 2000000000LL;
// `backoff_ns` > 0 puts the warp to sleep between attempts: a polling warp otherwise spends
// issue slots and ALU-pipe cycles that the decode warps of the same SM need (measured: idle
// roles polled away more instructions than the decode itself executed).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned backoff_ns = 0, long long limit_cycles = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (backoff_ns) __nanosleep(backoff_ns);
    if ((++it & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// ---- async-proxy fences ------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- TMA ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_tensor_2d_g2s(uint32_t dst, const CUtensorMap* tmap, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- tensor memory -----------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// each lane writes 16 consecutive 32-bit columns of its own TMEM lane
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// each lane reads 16 consecutive 32-bit columns of its own TMEM lane
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---- tcgen05 MMA -------------------------------------------------------------------
// D[tmem] (+)= A[tmem] * B[smem descriptor]; A is 128 x 16 fp16 (8 columns), K-major.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The eight k16 steps of one 128-k stage in a single block: A advances 8 columns per step,
// B walks two 128-byte-swizzled 64-k atoms (descriptor low words b0_lo / b1_lo, +32 bytes per
// step).  `first_accumulates` = 0 makes step 0 overwrite D.
__device__ __forceinline__ void mma_f16_ts_stage8(uint32_t d_tmem, uint32_t a_tmem, uint32_t b0_lo, uint32_t b1_lo,
                                                  uint32_t b_hi, uint32_t idesc, uint32_t first_accumulates) {
  asm volatile(
      "{\n\t"
      ".reg .pred p0, p1;\n\t"
      ".reg .b64 bd;\n\t"
      ".reg .b32 a, bl;\n\t"
      "setp.ne.b32 p0, %6, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "mov.b64 bd, {%2, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %5, p0;\n\t"
      "add.u32 a, %1, 8;\n\t  add.u32 bl, %2, 2;\n\t  mov.b64 bd, {bl, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "add.u32 a, %1, 16;\n\t add.u32 bl, %2, 4;\n\t  mov.b64 bd, {bl, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "add.u32 a, %1, 24;\n\t add.u32 bl, %2, 6;\n\t  mov.b64 bd, {bl, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "add.u32 a, %1, 32;\n\t mov.b64 bd, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "add.u32 a, %1, 40;\n\t add.u32 bl, %3, 2;\n\t  mov.b64 bd, {bl, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "add.u32 a, %1, 48;\n\t add.u32 bl, %3, 4;\n\t  mov.b64 bd, {bl, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "add.u32 a, %1, 56;\n\t add.u32 bl, %3, 6;\n\t  mov.b64 bd, {bl, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, p1;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b0_lo), "r"(b1_lo), "r"(b_hi), "r"(idesc), "r"(first_accumulates)
      : "memory");
}
// arrive on an mbarrier once every tcgen05 operation issued so far by this thread is done
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// K-major, 128-byte-swizzled shared-memory operand descriptor (8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                          // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                          // layout type: SWIZZLE_128B
  return d;
}
// fp16 x fp16 -> fp32, both operands K-major, M = 128
__host__ __device__ constexpr uint32_t idesc_f16_m128(int n) {
  return (1u << 4) /* D = f32 */ | (0u << 7) /* A = f16 */ | (0u << 10) /* B = f16 */ |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

}  // namespace ptx
}  // namespace qfb
