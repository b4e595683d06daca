// Split-K GEMV / skinny GEMM for batches of at most 16 activation rows on the warp-level
// tensor-core instruction (mma.sync m16n8k16), reading the "fragment" packed layout.
//
// Replaces the reference's kernel_gptq / kernel_gemv templates
// (qfactory/include/gptq_gemv.h:14-154, qfactory/include/gemv.h:12-94) for 2-, 3-, 4- and 8-bit layers.
//
// Why a third kernel.  On B200 the fp16x2 CUDA-core instructions and the integer/logic pipe both
// issue at half rate, so a CUDA-core GEMV that spends LOP3 + HSUB2 + HFMA2 per code pair is
// bound by instruction issue at about a third of the HBM rate.  Here the dot product moves to
// the tensor core and the zero-point subtraction moves out of the inner loop:
//
//   * the 16 weight rows of a row block are the M side of the MMA, the (at most 8) activation
//     rows its N side, so one 32-bit word of eight 4-bit codes is exactly one thread's A
//     fragment (rows g and g+8, four k each) and costs one shift and four AND instructions;
//   * a masked nibble is used AS IT IS as an fp16 bit pattern: the subnormal q * 2^-24 (nibble at
//     bits 0-3 of a half) or q * 2^-20 (bits 4-7).  The tensor core multiplies subnormals
//     exactly and accumulates in fp32; the two powers of two belong to different ROWS (g and
//     g+8), so they are folded into the row's scale;
//   * per quantisation group  sum_k x_k (q_k - z) s = s * sum_k x_k q_k - s z * sum_k x_k :
//     the first sum is the MMA accumulator, sum_k x_k is computed once per CTA by MMAs whose
//     A fragment is all ones, and both products are applied in fp32 once per group.
//
// Mapping.  A CTA owns one 128-row tile and a range of 128-k batches; warp (wt, kw) owns the
// 64-row half wt and the k-way kw of that range.  One 128-bit load per thread brings the words
// of four row blocks for one 16-k step, so consecutive steps of a warp are consecutive 512-byte
// runs.  The CTA's activation slice arrives by one bulk (TMA) copy per batch row.  Partial sums
// of the k-ways are combined in shared memory, those of the K splits either inside a thread-block
// cluster (pushed into the owner's shared memory, one cluster barrier) or through the fp32
// workspace by the last CTA of the tile to arrive; both in split order (deterministic; the
// counters reset themselves).
//
// Ordering under programmatic dependent launch: weight, scale and zero loads are issued before
// griddepcontrol.wait; activations, workspace and output are only touched after it.
#include <map>
#include <mutex>

#include "qfb_common.cuh"
#include "qfb_kernels.h"
#include "qfb_ptx.cuh"

namespace qfb {

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// thread-block-cluster helpers: barrier across the CTAs of a cluster, store into the shared memory
// of CTA `rank` of the cluster at the offset that `addr` has in this CTA
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_barrier() {
  cluster_arrive();
  cluster_wait();
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, int rank, float v) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t local_addr, int rank, const float4& v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

constexpr int kRedStride = 132;  // floats per (k-way, batch row) line of the k-way reduction

// first MMA of a segment: the accumulator starts from zero
__device__ __forceinline__ void mma_m16n8k16_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// the words of one lane and k-step a warp holds: 4 (16 bytes), 2 or 1
template <int NW> struct Words;
// load_if keeps the predicate inside the instruction (no branch around the load), so that the
// k-steps of a batch stay one basic block the compiler can schedule across
template <> struct Words<4> {
  uint32_t v[4];
  __device__ __forceinline__ void load(const void* p) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(p));
  }
  __device__ __forceinline__ void load_if(const void* p, int pred) {
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %5, 0;\n@q ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n}"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]) : "l"(p), "r"(pred));
  }
};
template <> struct Words<3> {  // (3-bit: the three words of a lane sit in three 128-byte planes of the k-step)
  uint32_t v[3];
  __device__ __forceinline__ void load(const void* p) {
    const char* c = static_cast<const char*>(p);
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v[0]) : "l"(c));
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v[1]) : "l"(c + 128));
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v[2]) : "l"(c + 256));
  }
  __device__ __forceinline__ void load_if(const void* p, int pred) {
    const char* c = static_cast<const char*>(p);
    asm volatile(
        "{\n.reg .pred q;\nsetp.ne.b32 q, %4, 0;\n@q ld.global.nc.L1::no_allocate.u32 %0, [%3];\n"
        "@q ld.global.nc.L1::no_allocate.u32 %1, [%3+128];\n@q ld.global.nc.L1::no_allocate.u32 %2, [%3+256];\n}"
        : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]) : "l"(c), "r"(pred));
  }
};
template <> struct Words<2> {
  uint32_t v[2];
  __device__ __forceinline__ void load(const void* p) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "l"(p));
  }
  __device__ __forceinline__ void load_if(const void* p, int pred) {
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %3, 0;\n@q ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n}"
                 : "+r"(v[0]), "+r"(v[1]) : "l"(p), "r"(pred));
  }
};

template <> struct Words<1> {
  uint32_t v[1];
  __device__ __forceinline__ void load(const void* p) {
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v[0]) : "l"(p));
  }
  __device__ __forceinline__ void load_if(const void* p, int pred) {
    if (pred) load(p);
  }
};

// raw scales (one half2 = rows g, g+8 per row block) and zeros (one byte per row) of a thread's rows
template <int RB> struct ScaleZero {
  uint32_t s[RB];
  uint32_t z[RB / 2];
  __device__ __forceinline__ void load(const __half* qs, const uint8_t* qz, size_t o) {
    if (RB == 4) {
      if (qs) { const uint4 v = ldg_v4(qs + o); s[0] = v.x; s[1] = v.y; s[RB - 2] = v.z; s[RB - 1] = v.w; }
      if (qz) { const uint2 v = ldg_v2(qz + o); z[0] = v.x; z[RB / 2 - 1] = v.y; }
    } else {
      if (qs) { const uint2 v = ldg_v2(qs + o); s[0] = v.x; s[1] = v.y; }
      if (qz) z[0] = __ldg(reinterpret_cast<const unsigned*>(qz + o));
    }
  }
};

// BITS  = 4, 8 or 2 (FragCodec in qfb_common.cuh)
// NT    = number of 8-column batch tiles (m <= 8 * NT)
// RB    = 16-row blocks per warp: 4 (a warp owns 64 rows) or 2 (32 rows)
// SEG64 = quantisation groups of 64 (a segment = 4 k-steps) instead of >= 128 (8 k-steps)
// A segment is the run of k-steps whose MMA accumulator is folded into the results at once
// with one scale and zero per row: min(group, 128) k.
// PUSH  = the results are also sent to the peers of a tensor-parallel group (MmaParams::push); a build of its
//         own, so that the plain kernel carries none of that code (measured: as a run-time branch in the
//         store path it cost the 4-us launches of the small layers 0.6 us)
// LEAN  = a build without the fused-activation staging and without the reduction through the workspace, for
//         the launches that need neither (measured: 1-3 % faster; the compiler schedules the common path
//         better when the rare ones are not in the same function)
// NORM  = the activations are rmsnorm(x + r) * w of a residual stream (MmaParams::norm_*), made while they are
//         staged: every CTA adds and weights its K slice and sums its squares; the sums of a tile's K splits
//         meet where the partial results meet (in the cluster, or in the one CTA of an unsplit tile), and
//         1 / rms, a scalar per batch row, is applied to the result instead of to every activation.  A
//         build of its own; launched with in-cluster reduction or no split only.
// ASYM  = the layer is known to have scales and zero points (the common case: their null checks and the
//         symmetric / group-less fold leave the loop)
// ONE   = one activation row (m = 1): the threads fetch the slice with
//         plain loads and sum it on the way in (one barrier and one pass less than the bulk copy + all-ones MMA
//         that serve every m), and only batch column 0 is folded and reduced
template <int BITS, int NT, int RB, bool SEG64, bool PUSH, bool LEAN, bool NORM, bool ASYM, bool ONE>
__device__ __forceinline__ void gemv_mma_body(const MmaParams& p) {
  using FC = FragCodec<BITS>;
  constexpr int KS = SEG64 ? 4 : 8;    // k-steps per segment
  constexpr int NSEG = SEG64 ? 2 : 1;  // segments per 128-k batch
  constexpr int NW = RB * BITS / 4;    // words of a lane and k-step this warp holds
  constexpr int NSLOT = NW >= 3 ? 1 : 2;  // register buffers of one batch each (32 registers in all, 24 for NW = 3, 16 for NW = 1)
  constexpr int WPK = 8 / RB;          // warps per k-way: 128 rows / (16 * RB)
  extern __shared__ uint4 smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wt = warp & 1;                    // 64-row half of the tile
  const int sub = (warp >> 1) & (WPK / 2 - 1);  // which RB row blocks of that half (RB = 2 only)
  const int kw = warp / WPK;
  const int KW = (blockDim.x >> 5) / WPK;
  const int tile = blockIdx.y, split = blockIdx.x, S = gridDim.x;
  // Shared memory of another CTA of the cluster may only be touched once that CTA has started:
  // every CTA arrives here, at its start, and waits for the others just before its first remote
  // store, a whole main loop later (the wait is free by then).
  if (p.cluster) cluster_arrive();

  // balanced ranges of 128-k batches: CTA [bb, be), this warp's k-way [wb, we); no divisions on
  // this path (the host passes batches / S and batches % S, the k-ways are a power of two)
  const int bb = split * p.batches_div + min(split, p.batches_mod);
  const int be = bb + p.batches_div + (split < p.batches_mod ? 1 : 0);
  const int ncta = be - bb;
  const int kw_shift = KW == 4 ? 2 : (KW == 2 ? 1 : 0);
  const int wb = bb + ((kw * ncta) >> kw_shift);
  const int we = bb + (((kw + 1) * ncta) >> kw_shift);

  // 4 * BITS bytes per lane and k-step for the four row blocks; this warp reads the words of
  // its RB row blocks (for RB = 2: the lower or upper half of them)
  constexpr int kStepBytes = 128 * BITS, kBatchBytes = 8 * kStepBytes;
  const char* wp = reinterpret_cast<const char*>(p.qw) +
                   ((size_t)(tile * 2 + wt) * p.ksteps + (size_t)wb * 8) * kStepBytes +
                   frag_word_offset(BITS, lane, sub * NW);

  // quantisation group of the warp's first segment, and the position inside it
  const int segs_per_group = SEG64 ? p.chunks_per_group : (p.chunks_per_group >> 1);
  int grp = wb * NSEG, gpos = 0;
  int grp_last = we * NSEG - 1;  // last group this warp touches
  if (segs_per_group != 1) {     // (one segment per group, the common case, needs no division)
    grp = (wb * NSEG) / segs_per_group;
    gpos = wb * NSEG - grp * segs_per_group;
    grp_last = (we * NSEG - 1) / segs_per_group;
  }

  // scales and zeros of the group being accumulated: loaded one segment ahead (right after the
  // fold that consumed the previous group's), into the same registers
  ScaleZero<RB> sz_cur;
#pragma unroll
  for (int i = 0; i < RB; ++i) sz_cur.s[i] = 0;
#pragma unroll
  for (int i = 0; i < RB / 2; ++i) sz_cur.z[i] = 0;
  auto sz_offset = [&](int gi) { return (((size_t)tile * p.groups + gi) * 2 + wt) * 64 + g * 8 + sub * 4; };

  Words<NW> w[NSLOT][8];
#pragma unroll
  for (int sl = 0; sl < NSLOT; ++sl)
    if (wb + sl < we) {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[sl][i].load(wp + sl * kBatchBytes + i * kStepBytes);
    }
  wp += NSLOT * kBatchBytes;  // from here on: the batch NSLOT ahead of the one being processed
  if (wb < we) sz_cur.load(p.qs, p.qz, sz_offset(grp));
  grid_launch_dependents();
  grid_dependency_wait();

  // ---- stage the CTA's activation slice ------------------------------------------------------
  const int xstride = p.batches_per_cta * 128 + 16;  // halfs; +16 keeps the fragment loads conflict-free
  __half* x_s = reinterpret_cast<__half*>(smem);
  // one bulk copy per row (256 bytes per batch: sizes and both addresses are multiples of 16),
  // lane r of warp 0 issues row r; warp 0 waits for the bytes, the barrier below publishes them
  __shared__ __align__(8) uint64_t xbar;
  __shared__ int xabort;
  __shared__ unsigned push_epoch[16];   // epoch of the reduction this launch feeds, per batch row
  __shared__ float nss_warp[8][16];     // NORM: per-warp sums of squares of the slice, per batch row
  __shared__ float nss_recv[8][16];     // NORM: the sums of the K splits of the tile (written by every CTA of the cluster)
  __shared__ float nrstd[16];           // NORM: 1 / rms per batch row
  // With p.act == 1 the activations are silu(gate) * up of a fused gate/up tensor [m, 2k]: the gate
  // and the up slices arrive by one bulk copy each and are combined in shared memory, with the
  // arithmetic of the stand-alone kernel (silu in fp32 rounded to fp16, then one fp16 product).
  __half* u_s = reinterpret_cast<__half*>(reinterpret_cast<char*>(smem) + p.act_offset);
  constexpr bool direct = ONE;
  if (NORM) {
    // x + r (one fp16 addition, as the stand-alone kernel), written back by the CTAs of tile 0 (whose K splits
    // cover the row once), times the norm weight (one fp16 product) into the slice; squares summed in fp32 per
    // thread and batch row, then per warp, in a fixed order
    const int vec_row = ncta * 16;  // 16-byte vectors per row of the slice
    float ss[8 * NT];
#pragma unroll
    for (int r = 0; r < 8 * NT; ++r) ss[r] = 0.f;
    const bool collect = p.collect.local != nullptr;
    const unsigned cep = collect ? (0x80000000u | (__ldcg(p.collect.step) << 8) | p.collect.idx) : 0u;
    for (int j = tid; j < vec_row; j += blockDim.x) {
      const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + (size_t)bb * 128 + (size_t)j * 8);
      const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int r = 0; r < 8 * NT; ++r) {
        if (r < p.m) {
          const size_t go = (size_t)r * p.k + (size_t)bb * 128 + (size_t)j * 8;
          uint4 xv = __ldcg(reinterpret_cast<const uint4*>(p.norm_x + go));
          uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
          if (collect) {
            // the addend: the partials of all ranks summed in rank order in fp32 and rounded to fp16 (what the
            // reduction kernel computes, bit for bit); a peer's words are polled until they carry the epoch
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
            for (int rk = 0; rk < 8; ++rk) {
              if (rk < p.collect.world) {
                uint4 p4;
                if (rk == p.collect.rank) {
                  p4 = __ldcg(reinterpret_cast<const uint4*>(p.collect.local + p.collect.own_offset + go * 2));
                } else {
                  const char* src = p.collect.local + p.collect.recv_offset + (size_t)rk * p.collect.region_bytes + go * 4;
                  uint4 lo, hi;
                  unsigned long long t0 = 0;
                  while (true) {
                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w) : "l"(src) : "memory");
                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(src + 16) : "memory");
                    if (lo.y == cep && lo.w == cep && hi.y == cep && hi.w == cep) break;
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > p.collect.timeout_ns) {   // bounded: record it and go on with what is there
                      atomicExch(p.collect.status, 1u);
                      break;
                    }
                  }
                  p4 = make_uint4(lo.x, lo.z, hi.x, hi.z);
                }
                const uint32_t pu[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float2 f = __half22float2(as_h2(pu[q]));
                  acc[2 * q] += f.x;
                  acc[2 * q + 1] += f.y;
                }
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) xu[q] = as_u32(__hadd2(as_h2(xu[q]), __floats2half2_rn(acc[2 * q], acc[2 * q + 1])));
          } else if (p.norm_r) {
            const uint4 rv = __ldcg(reinterpret_cast<const uint4*>(p.norm_r + go));
            const uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) xu[q] = as_u32(__hadd2(as_h2(xu[q]), as_h2(ru[q])));
          }
          if (p.norm_out && tile == 0) *reinterpret_cast<uint4*>(p.norm_out + go) = make_uint4(xu[0], xu[1], xu[2], xu[3]);
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(as_h2(xu[q]));
            ss[r] += f.x * f.x + f.y * f.y;
            o[q] = as_u32(__hmul2(as_h2(xu[q]), as_h2(wu[q])));
          }
          *reinterpret_cast<uint4*>(x_s + (size_t)r * xstride + (size_t)j * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 8 * NT; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], o);
      if (lane == 0) nss_warp[warp][r] = ss[r];
    }
  } else if (direct) {
    // one activation row: every thread fetches 16 bytes of the slice itself, stores them and adds them up; the 16
    // (8) lanes that hold a 128-k (64-k) segment combine their sums with shuffles and one of them writes the
    // segment's sum.  One barrier instead of two and no pass over the staged slice.
    constexpr int SEGL = SEG64 ? 8 : 16;  // lanes (16-byte vectors) per segment
    const int nvec = ncta * 16;
    float* xs_sum = reinterpret_cast<float*>(x_s + xstride);
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)bb * 128);
    if (PUSH && tid == 0)
      push_epoch[0] = p.push.idx >= 0 ? (0x80000000u | (__ldcg(p.push.step) << 8) | (unsigned)p.push.idx)
                                      : __ldcg(p.push.epochs) + 1u;
    for (int base = 0; base < nvec; base += (int)blockDim.x) {  // (nvec is a multiple of 16: a segment's lanes agree)
      const int j = base + tid;
      uint4 v = j < nvec ? __ldcg(src + j) : make_uint4(0u, 0u, 0u, 0u);
      if (!LEAN && p.act) {  // silu(gate) * up, the arithmetic of the pass over the staged slices below
        const uint4 up = j < nvec ? __ldcg(src + (p.k >> 3) + j) : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t ua[4] = {v.x, v.y, v.z, v.w}, ub[4] = {up.x, up.y, up.z, up.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(as_h2(ua[q]));
          const __half2 sg = __floats2half2_rn(f.x / (1.f + __expf(-f.x)), f.y / (1.f + __expf(-f.y)));
          o[q] = as_u32(__hmul2(sg, as_h2(ub[q])));
        }
        v = make_uint4(o[0], o[1], o[2], o[3]);
      }
      const float2 f0 = __half22float2(as_h2(v.x)), f1 = __half22float2(as_h2(v.y));
      const float2 f2 = __half22float2(as_h2(v.z)), f3 = __half22float2(as_h2(v.w));
      float sum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
      for (int o = SEGL / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (j < nvec) {
        *(reinterpret_cast<uint4*>(x_s) + j) = v;
        if ((j & (SEGL - 1)) == 0) xs_sum[(j / SEGL) * (8 * NT)] = sum;
      }
    }
  } else if (warp == 0) {
    const uint32_t bar = ptx::smem_u32(&xbar);
    const uint32_t row_bytes = (uint32_t)ncta * 256u;
    if (lane == 0) {
      xabort = 0;
      ptx::mbar_init(bar, 1);
      ptx::fence_barrier_init();
      ptx::mbar_arrive_expect_tx(bar, row_bytes * (uint32_t)p.m * (p.act ? 2u : 1u) + (p.stall_test ? 16u : 0u));
    }
    __syncwarp();
    // (the reduction kernel that finished the previous epoch of these rows precedes this launch)
    if (PUSH && lane < p.m)
      push_epoch[lane] = p.push.idx >= 0 ? (0x80000000u | (__ldcg(p.push.step) << 8) | (unsigned)p.push.idx)
                                         : __ldcg(p.push.epochs + lane) + 1u;
    if (lane < p.m) {
      const __half* src = p.x + (size_t)lane * p.x_stride + (size_t)bb * 128;
      ptx::tma_bulk_g2s(ptx::smem_u32(x_s + (size_t)lane * xstride), src, row_bytes, bar);
      if (p.act) ptx::tma_bulk_g2s(ptx::smem_u32(u_s + (size_t)lane * xstride), src + p.k, row_bytes, bar);
    }
    // bounded: a copy that never lands raises the status word instead of hanging the CTA
    if (!ptx::mbar_wait(bar, 0, &xabort, 0, p.stall_test ? 200000LL : ptx::kWaitLimitCycles) && lane == 0 && p.status)
      atomicExch(p.status, 1u);
  }
  __syncthreads();
  if (!LEAN && !direct && p.act) {
    const int vec_row = ncta * 16;  // 16-byte vectors per row of the slice
    for (int i = tid; i < p.m * vec_row; i += blockDim.x) {
      const int r = i / vec_row, j = i - r * vec_row;
      uint4* gp = reinterpret_cast<uint4*>(x_s + (size_t)r * xstride) + j;
      const uint4 a = *gp, b = *(reinterpret_cast<const uint4*>(u_s + (size_t)r * xstride) + j);
      const uint32_t ua[4] = {a.x, a.y, a.z, a.w}, ub[4] = {b.x, b.y, b.z, b.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(as_h2(ua[q]));
        const __half2 sg = __floats2half2_rn(f.x / (1.f + __expf(-f.x)), f.y / (1.f + __expf(-f.y)));
        o[q] = as_u32(__hmul2(sg, as_h2(ub[q])));
      }
      *gp = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();
  }

  // activation row each batch tile of this thread reads (rows >= m repeat the last valid row;
  // their output columns are never stored)
  const __half* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) xrow[nt] = x_s + (size_t)min(g + 8 * nt, p.m - 1) * xstride + 4 * t;

  // ---- sum of the activations over every segment of the slice: an MMA whose A fragment is all
  // ones yields, in every row, the column sums of the B fragment.  The warps share the segments.
  float* xsum_s = reinterpret_cast<float*>(x_s + (size_t)p.m * xstride);  // [segments][8 * NT]
  if (!direct) {
    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};  // fp16 1.0
    const int nwarps = blockDim.x >> 5;
    // two segments per pass and two accumulators per segment (even / odd k-steps): independent
    // MMA chains, so the latency of a dependent accumulate is paid KS / 2 times, not KS per segment
    const int nsegs = ncta * NSEG;
    for (int sg0 = warp; sg0 < nsegs; sg0 += 2 * nwarps) {
      float dx[2][NT][2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int sg = min(sg0 + u * nwarps, nsegs - 1);  // (a clamped duplicate is computed and dropped)
#pragma unroll
        for (int k4 = 0; k4 < KS; ++k4) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint2 v = *reinterpret_cast<const uint2*>(xrow[nt] + (sg * KS + k4) * 16);
            if (k4 < 2) mma_m16n8k16_zero(dx[u][nt][k4 & 1], ones, v.x, v.y);
            else mma_m16n8k16(dx[u][nt][k4 & 1], ones, v.x, v.y);
          }
        }
      }
      if (g == 0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int sg = sg0 + u * nwarps;
          if (sg < nsegs) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
              *reinterpret_cast<float2*>(xsum_s + sg * (8 * NT) + nt * 8 + 2 * t) =
                  make_float2(dx[u][nt][0][0] + dx[u][nt][1][0], dx[u][nt][0][1] + dx[u][nt][1][1]);
          }
        }
      }
    }
    __syncthreads();
  }

  float acc[RB][NT][4];
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rb][nt][i] = 0.f;

  const float zc = (float)p.zconst;

  for (int b0 = wb; b0 < we; b0 += NSLOT) {
#pragma unroll
    for (int sl = 0; sl < NSLOT; ++sl) {
      const int b = b0 + sl;
      if (b >= we) break;
      const int lb = b - bb;
      const int more = b + NSLOT < we ? 1 : 0;
#pragma unroll
      for (int seg = 0; seg < NSEG; ++seg) {
        float d[RB][NT][4];
#pragma unroll
        for (int k4 = 0; k4 < KS; ++k4) {
          const int ks = seg * KS + k4;
          uint32_t bf[NT][2];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint2 v = *reinterpret_cast<const uint2*>(xrow[nt] + lb * 128 + ks * 16);
            bf[nt][0] = v.x;
            bf[nt][1] = v.y;
          }
#pragma unroll
          for (int rb = 0; rb < RB; ++rb) {
            uint32_t a[4];
            FC::decode(w[sl][ks].v, rb, a);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              if (k4 == 0) mma_m16n8k16_zero(d[rb][nt], a, bf[nt][0], bf[nt][1]);
              else mma_m16n8k16(d[rb][nt], a, bf[nt][0], bf[nt][1]);
            }
          }
          // the words of this k-step are consumed: fetch the same step of a later batch into them
          if (NSLOT == 1) w[sl][ks].load_if(wp + ks * kStepBytes, more);  // (measured: a gain with one buffer only)
          else if (more) w[sl][ks].load(wp + ks * kStepBytes);
        }
        // fold the segment's accumulators into the results: s * 2^24 * D - s * z * sum(x)
        float dx[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float2 v = *reinterpret_cast<const float2*>(xsum_s + (lb * NSEG + seg) * (8 * NT) + nt * 8 + 2 * t);
          dx[nt][0] = v.x;
          dx[nt][1] = v.y;
        }
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
          float2 sf = make_float2(1.f, 1.f);
          if (ASYM || p.qs) sf = __half22float2(as_h2(sz_cur.s[rb]));
          float z0 = zc, z1 = zc;
          if (ASYM || p.qz) {
            const uint32_t zb = sz_cur.z[rb >> 1] >> ((rb & 1) * 16);
            z0 = (float)(zb & 0xffu);
            z1 = (float)((zb >> 8) & 0xffu);
          }
          // undo the power of two of the subnormal fields: 2^(24 - bit offset inside the half)
          const float a0 = sf.x * (float)(1 << (24 - FC::shift_lo(rb))), a1 = sf.y * (float)(1 << (24 - FC::shift_hi(rb)));
          const float b0 = -sf.x * z0, b1 = -sf.y * z1;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            acc[rb][nt][0] = fmaf(b0, dx[nt][0], fmaf(a0, d[rb][nt][0], acc[rb][nt][0]));
            acc[rb][nt][2] = fmaf(b1, dx[nt][0], fmaf(a1, d[rb][nt][2], acc[rb][nt][2]));
            if (!ONE) {  // (one activation row: only batch column 0 is stored)
              acc[rb][nt][1] = fmaf(b0, dx[nt][1], fmaf(a0, d[rb][nt][1], acc[rb][nt][1]));
              acc[rb][nt][3] = fmaf(b1, dx[nt][1], fmaf(a1, d[rb][nt][3], acc[rb][nt][3]));
            }
          }
        }
        if (++gpos == segs_per_group) {  // the next segment starts a new group
          gpos = 0;
          ++grp;
          if (grp <= grp_last) sz_cur.load(p.qs, p.qz, sz_offset(grp));
        }
      }
      wp += kBatchBytes;
    }
  }

  // ---- combine the k-ways of the CTA ----------------------------------------------------
  __syncthreads();  // everyone is done reading the staged activations
  float* red = reinterpret_cast<float*>(smem);
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int mm = nt * 8 + 2 * t + (i & 1);
        const int r = wt * 64 + (sub * RB + rb) * 16 + (i >> 1) * 8 + g;
        if (ONE && (i & 1)) continue;
        if (mm < p.m) red[(kw * p.m + mm) * kRedStride + r] = acc[rb][nt][i];
      }
  __syncthreads();

  // From here on the outputs of the tile are handled as quads: four consecutive rows of one
  // batch column (quad q: column q / 32, rows 4 * (q % 32) ...), 16-byte shared-memory accesses.
  const int nout = p.m * kTileRows;
  const int nq = p.m * (kTileRows / 4);
  auto kway_sum4 = [&](int q) {
    const int mm = q >> 5, r = (q & 31) * 4;
    float4 v = *reinterpret_cast<const float4*>(red + mm * kRedStride + r);
    for (int w = 1; w < KW; ++w) {
      const float4 u = *reinterpret_cast<const float4*>(red + (w * p.m + mm) * kRedStride + r);
      v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
    }
    return v;
  };
  // the four fp16 results of a quad as two {data, epoch} words in this rank's receive region of every peer
  auto push_quad = [&](int mm, int n, uint32_t lo, uint32_t hi) {
    const unsigned ep = push_epoch[mm];
    const size_t off = p.push.recv_offset + (size_t)mm * p.n * 4 + (size_t)(n >> 3) * 32 + (size_t)((n >> 2) & 1) * 16;
#pragma unroll
    for (int r = 0; r < 8; ++r)   // (compile-time indices: the pointer array stays in the parameter bank)
      if (r < p.push.world && r != p.push.rank)
        asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p.push.base[r] + off), "r"(lo), "r"(ep),
                     "r"(hi), "r"(ep)
                     : "memory");
  };
  auto store_quad = [&](int q, const float4& v0) {
    const int mm = q >> 5, n = tile * kTileRows + (q & 31) * 4;
    __half* dst = p.y + (size_t)mm * p.n + n;
    float4 v = v0;
    if (NORM) {  // the scalar of the norm, applied to the result
      const float rs = nrstd[mm];
      v.x *= rs; v.y *= rs; v.z *= rs; v.w *= rs;
    }
    if (n + 3 < p.n && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
      const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
      *reinterpret_cast<uint2*>(dst) = make_uint2(as_u32(lo), as_u32(hi));
      if (PUSH) push_quad(mm, n, as_u32(lo), as_u32(hi));   // (such layers have whole, aligned quads only)
    } else {
      const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (n + i < p.n) dst[i] = __float2half_rn(e[i]);
    }
  };
  // NORM: this CTA's sum of squares of a batch row (its warps' sums in a fixed order)
  auto norm_cta_sum = [&](int r) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += nss_warp[w][r];
    return t;
  };
  if (S == 1) {
    if (NORM) {
      if (tid < p.m) nrstd[tid] = rsqrtf(norm_cta_sum(tid) / (float)p.k + p.norm_eps);
      __syncthreads();
    }
    for (int q = tid; q < nq; q += blockDim.x) store_quad(q, kway_sum4(q));
    return;
  }

  if (p.cluster) {
    // split-K inside a thread-block cluster (the S splits of a tile are one cluster): CTA r owns
    // the quads [r * qper, (r + 1) * qper).  Every CTA pushes its k-way-reduced partial of a quad
    // into a receive buffer in the OWNER's shared memory (slot = the sender's split), one cluster
    // barrier makes the pushes visible, and each owner sums its S slots in split order.  The
    // receive buffer is a region of its own: a fast CTA may push while a slow one still computes.
    float4* recv = reinterpret_cast<float4*>(reinterpret_cast<char*>(smem) + p.recv_offset);
    const uint32_t recv_addr = static_cast<uint32_t>(__cvta_generic_to_shared(recv));
    const int qper = p.quads_per_owner;
    cluster_wait();  // pairs with the arrive at kernel start: every CTA of the cluster runs
    if (NORM && tid < p.m) {  // every CTA of the tile learns every split's sum of squares
      const float t = norm_cta_sum(tid);
      const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(&nss_recv[split][tid]));
      for (int c = 0; c < S; ++c) st_cluster_f32(a, c, t);
    }
    for (int q = tid; q < nq; q += blockDim.x) {
      const float4 v = kway_sum4(q);
      const int owner = (int)__umulhi((unsigned)q, p.qper_magic);  // q / qper (q < 2^9, qper <= 2^9)
      st_cluster_v4(recv_addr + (split * qper + (q - owner * qper)) * 16, owner, v);
    }
    cluster_barrier();
    if (NORM) {
      if (tid < p.m) {
        float t = 0.f;
        for (int u = 0; u < S; ++u) t += nss_recv[u][tid];   // split order: the same bits in every CTA
        nrstd[tid] = rsqrtf(t / (float)p.k + p.norm_eps);
      }
      __syncthreads();
    }
    for (int j = tid; j < qper; j += blockDim.x) {
      const int q = split * qper + j;
      if (q < nq) {
        float4 v = recv[j];
        for (int u = 1; u < S; ++u) {
          const float4 w = recv[u * qper + j];
          v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        store_quad(q, v);
      }
    }
    return;
  }

  if (LEAN) return;  // (the lean build is only launched for S == 1 and in-cluster reductions)
  // split-K through the workspace: publish this CTA's partial, the last CTA of the tile to
  // arrive sums them in split order
  for (int q = tid; q < nq; q += blockDim.x) {
    const int mm = q >> 5, r = (q & 31) * 4;
    *reinterpret_cast<float4*>(p.partial + ((size_t)split * p.m + mm) * p.npad + tile * kTileRows + r) = kway_sum4(q);
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
  const size_t sstride = (size_t)p.m * p.npad;
  // every thread sums its (at most 16) outputs in split order, with either the loads of one split
  // for all its outputs or those of eight splits for two outputs in flight together, whichever
  // makes the shorter chain of round trips
  constexpr int kMaxOut = 16;  // 16 rows x 128 outputs over at least 128 threads, 8 x 128 over at least 64
  const int J = (nout + blockDim.x - 1) / blockDim.x;
  float s[kMaxOut];
  const float* src[kMaxOut];
#pragma unroll
  for (int j = 0; j < kMaxOut; ++j) {
    const int i = min(tid + j * (int)blockDim.x, nout - 1);
    src[j] = p.partial + (size_t)(i >> 7) * p.npad + tile * kTileRows + (i & 127);
    s[j] = 0.f;
  }
  if (2 * S > J) {  // few outputs per thread: two outputs at a time, eight splits in flight each
    for (int j0 = 0; j0 < J; j0 += 2) {
      const float* a0 = src[0];
      const float* a1 = src[0];
#pragma unroll
      for (int j = 0; j < kMaxOut; j += 2)
        if (j == j0) {
          a0 = src[j];
          a1 = src[j + 1];
        }
      float s0 = 0.f, s1 = 0.f;
      int sp = 0;
      for (; sp + 8 <= S; sp += 8) {
        float v0[8], v1[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          v0[u] = __ldcg(a0 + (size_t)(sp + u) * sstride);
          v1[u] = __ldcg(a1 + (size_t)(sp + u) * sstride);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          s0 += v0[u];
          s1 += v1[u];
        }
      }
      for (; sp < S; ++sp) {
        const float v0 = __ldcg(a0 + (size_t)sp * sstride), v1 = __ldcg(a1 + (size_t)sp * sstride);
        s0 += v0;
        s1 += v1;
      }
#pragma unroll
      for (int j = 0; j < kMaxOut; j += 2)
        if (j == j0) {
          s[j] = s0;
          s[j + 1] = s1;
        }
    }
  } else {
    for (int sp = 0; sp < S; ++sp) {
      float v[kMaxOut];
#pragma unroll
      for (int j = 0; j < kMaxOut; ++j) v[j] = (j < J) ? __ldcg(src[j] + (size_t)sp * sstride) : 0.f;
#pragma unroll
      for (int j = 0; j < kMaxOut; ++j) s[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxOut; ++j) {
    const int i = tid + j * (int)blockDim.x;
    const int n = tile * kTileRows + (i & 127);
    if (j < J && i < nout && n < p.n) p.y[(size_t)(i >> 7) * p.n + n] = __float2half_rn(s[j]);
  }
  if (tid == 0) p.counters[tile] = 0u;
  if (PUSH) {
    // this path stores single outputs: send the tile's results from where they were just written
    __syncthreads();
    for (int q = tid; q < nq; q += blockDim.x) {
      const int mm = q >> 5, n = tile * kTileRows + (q & 31) * 4;
      const uint2 yv = __ldcg(reinterpret_cast<const uint2*>(p.y + (size_t)mm * p.n + n));
      push_quad(mm, n, yv.x, yv.y);
    }
  }
}

// Two register budgets of the same body: CTAs of up to 256 threads with 128 registers per thread
// (two per SM, 16 warps), and CTAs of up to 128 threads with 96 (five per SM, 20 warps: measured
// 7-9 % faster on layers with many row tiles, slower as 256-thread CTAs, which fit only twice
// either way).  Tighter budgets that would leave room for the next launch's CTAs to become
// resident early (three CTAs of 256 threads at 80 registers, six of 128 at 80) spill inside the
// k-step loop and were 5-70 % slower on every Llama-7B layer shape.
template <int BITS, int NT, int RB, bool SEG64, bool PUSH = false, bool LEAN = false, bool NORM = false, bool ASYM = false,
          bool ONE = false>
__global__ void __launch_bounds__(256, 2) gemv_mma_kernel(const MmaParams p) {
  gemv_mma_body<BITS, NT, RB, SEG64, PUSH, LEAN, NORM, ASYM, ONE>(p);
}
template <int BITS, int NT, int RB, bool SEG64, bool PUSH = false, bool LEAN = false, bool NORM = false, bool ASYM = false,
          bool ONE = false>
__global__ void __launch_bounds__(128, 5) gemv_mma_kernel_small(const MmaParams p) {
  gemv_mma_body<BITS, NT, RB, SEG64, PUSH, LEAN, NORM, ASYM, ONE>(p);
}

template <int BITS, int NT, int RB, bool SEG64>
static cudaError_t launch_cfg(const MmaParams& p, dim3 grid, int block, size_t smem, bool pdl, cudaStream_t st) {
  auto kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, NT, RB, SEG64> : gemv_mma_kernel<BITS, NT, RB, SEG64>;
  if (!p.act && (p.cluster || grid.x == 1) && !p.push.world) {
    kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, NT, RB, SEG64, false, true>
                                   : gemv_mma_kernel<BITS, NT, RB, SEG64, false, true>;
    // (measured: 1-2 % faster with one batch tile, 2-5 % slower with two, where it is not used)
    if constexpr (NT == 1) {
      // one activation row (and no test of a copy that never lands, which needs the copy): its own build
      if (p.m == 1 && !p.stall_test)
        kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, NT, RB, SEG64, false, true, false, false, true>
                                       : gemv_mma_kernel<BITS, NT, RB, SEG64, false, true, false, false, true>;
      if (p.qs && p.qz) {
        kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, NT, RB, SEG64, false, true, false, true>
                                       : gemv_mma_kernel<BITS, NT, RB, SEG64, false, true, false, true>;
        if (p.m == 1 && !p.stall_test)
          kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, NT, RB, SEG64, false, true, false, true, true>
                                         : gemv_mma_kernel<BITS, NT, RB, SEG64, false, true, false, true, true>;
      }
    }
  }
  if constexpr (NT == 1) {
    // one activation row through the general build (fused activation, reduction through the workspace): every
    // path of one row sums its activations the same way, so they keep giving the same bits
    if (p.m == 1 && !p.stall_test && (p.act || !(p.cluster || grid.x == 1)))
      kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, 1, RB, SEG64, false, false, false, false, true>
                                     : gemv_mma_kernel<BITS, 1, RB, SEG64, false, false, false, false, true>;
  }
  if (p.norm_w) {
    // the build with the fused residual add + RMS norm: the same layers, in-cluster reduction or no split
    if (p.push.world || p.act || !(p.cluster || grid.x == 1)) return cudaErrorInvalidValue;
    if constexpr (BITS == 4 && !SEG64)
      kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<4, NT, RB, false, false, true, true>
                                     : gemv_mma_kernel<4, NT, RB, false, false, true, true>;
    else
      return cudaErrorNotSupported;
  }
  if (p.push.world) {
    // the sending build: 4-bit layers with groups of 128 and more (what the decoder's row-parallel layers are)
    if constexpr (BITS == 4 && !SEG64) {
      kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<4, NT, RB, false, true> : gemv_mma_kernel<4, NT, RB, false, true>;
      if constexpr (NT == 1) {
        if (p.m == 1 && !p.stall_test)
          kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<4, 1, RB, false, true, false, false, false, true>
                                         : gemv_mma_kernel<4, 1, RB, false, true, false, false, false, true>;
      }
    } else {
      return cudaErrorNotSupported;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.cluster) {  // the K splits of one tile form a cluster
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = grid.x;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return cudaLaunchKernelEx(&cfg, kern, p);
}

// How many clusters of `cluster` CTAs (block threads, smem bytes of dynamic shared memory each)
// the current device holds at once; cached per configuration.  0 when the query fails.
template <int BITS, int NT, int RB, bool SEG64>
static int query_clusters(int block, size_t smem, int cluster) {
  auto kern = block <= kMmaSmallBlock ? gemv_mma_kernel_small<BITS, NT, RB, SEG64> : gemv_mma_kernel<BITS, NT, RB, SEG64>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster, 1024);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

// one instantiation per (bit width, batch tiles, group mode); RB follows: 64-row warps for one
// batch tile of 2-, 3- and 4-bit layers, 32-row warps otherwise (3-bit: that one build only)
#define QFB_MMA_DISPATCH(FN, ...)                                                                     \
  do {                                                                                                \
    if (bits == 4 && nt == 1) return seg64 ? FN<4, 1, 4, true>(__VA_ARGS__) : FN<4, 1, 4, false>(__VA_ARGS__); \
    if (bits == 4 && nt == 2) return seg64 ? FN<4, 2, 2, true>(__VA_ARGS__) : FN<4, 2, 2, false>(__VA_ARGS__); \
    if (bits == 8 && nt == 1) return seg64 ? FN<8, 1, 2, true>(__VA_ARGS__) : FN<8, 1, 2, false>(__VA_ARGS__); \
    if (bits == 8 && nt == 2) return seg64 ? FN<8, 2, 2, true>(__VA_ARGS__) : FN<8, 2, 2, false>(__VA_ARGS__); \
    if (bits == 2 && nt == 1) return seg64 ? FN<2, 1, 4, true>(__VA_ARGS__) : FN<2, 1, 4, false>(__VA_ARGS__); \
    if (bits == 3 && nt == 1 && !seg64) return FN<3, 1, 4, false>(__VA_ARGS__);                               \
    if (bits == 2 && nt == 2) return seg64 ? FN<2, 2, 2, true>(__VA_ARGS__) : FN<2, 2, 2, false>(__VA_ARGS__); \
  } while (0)

int mma_rows_per_warp(int bits, int nt) {
  return (nt == 1 && bits != 8) ? 64 : 32;
}

static int query_any(int bits, int nt, bool seg64, int block, size_t sm, int cluster) {
  QFB_MMA_DISPATCH(query_clusters, block, sm, cluster);
  return 0;
}

int mma_max_active_clusters(int bits, int nt, bool seg64, int block, size_t smem, int cluster) {
  static std::mutex mu;
  static std::map<unsigned long long, int> cache;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  const size_t smem_kb = (smem + 1023) / 1024;  // the answer only changes with the shared-memory footprint
  const unsigned long long key = ((unsigned long long)dev << 52) | ((unsigned long long)bits << 48) |
                                 ((unsigned long long)nt << 44) | ((unsigned long long)seg64 << 43) |
                                 ((unsigned long long)block << 28) | ((unsigned long long)smem_kb << 8) |
                                 (unsigned long long)cluster;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  const int n = query_any(bits, nt, seg64, block, smem_kb * 1024, cluster);
  cache[key] = n;
  return n;
}

cudaError_t launch_gemv_mma(const MmaParams& p, int bits, int nt, dim3 grid, int block, size_t smem, bool pdl,
                            cudaStream_t st) {
  const bool seg64 = p.chunks_per_group == 1;
  QFB_MMA_DISPATCH(launch_cfg, p, grid, block, smem, pdl, st);
  return cudaErrorInvalidValue;
}

}  // namespace qfb
