// One-shot all-reduce over peer memory for the row-parallel linears of a tensor-parallel decoder
// (O and down projections), fused with what follows it in a decoder layer: the residual add and
// the next RMSNorm.
//
// The reference's serving stack sums the partial results of a row-parallel linear with a
// collective call (third_party/vllm-bitblas/vllm/model_executor/layers/linear.py:1100-1124) and
// prefers a one-shot peer-memory kernel over NCCL for small messages
// (third_party/vllm-bitblas/csrc/custom_all_reduce.cuh:133-150 flags, :210-226 one-shot;
// dispatch in vllm/distributed/device_communicators/custom_all_reduce.py:242-255).  A decode step
// of the 80-layer decoder has 160 such reductions of 16 KiB per batch row: their latency, not
// their bandwidth, is what matters.
//
// Protocol.  Every rank owns one symmetric buffer (same layout on every rank, mapped into every
// peer): a header and two data slots; a slot holds this rank's own partial (plain fp16, written by
// the row-parallel GEMV as its output) and one RECEIVE region per source rank.  The reduction
// kernel runs one thread-block cluster per batch row (a 16-byte vector of the row per thread) and
// needs no flag exchange and no fence: the flag travels inside the data.
//   1. every thread reads its 16 bytes of the local partial and stores them into this rank's
//      receive region of every PEER's buffer as four 8-byte words {4 data bytes, epoch} (two
//      16-byte peer stores per peer; an 8-byte word is written atomically, so a word whose epoch
//      matches carries valid data).  Fire and forget;
//   2. the same thread polls the four words it needs of every peer's region of its OWN buffer
//      (local memory) until all carry this call's epoch: the only latency exposed is one NVLink
//      one-way trip.  (A first version raised flags and pulled the partials with peer loads: a flag
//      trip plus a load round trip; a second pushed the data and then a flag with st.release.sys,
//      which waits for the pushes to be acknowledged: 3.8 us per reduction over the norm alone.)
//      Epochs only ever grow, so stale words never match and a replayed CUDA graph needs no
//      reset; the epoch of a row lives in the local header and is advanced by the kernel itself.
//   3. the thread sums the W partials in rank order in fp32 (bit-identical on every rank), adds
//      the residual stream, and the cluster applies the RMS norm.
// Data slots alternate between consecutive reductions.  A peer can run at most one reduction ahead
// of this rank (its next row-parallel GEMV needs the result of the current reduction, hence this
// rank's partial of it), so it writes the other slot while this one is still being read.
//
// Every wait is bounded (default 2 s, settable): when it runs out the CTA records it in the status
// word of the local header and carries on with whatever the slots hold; the host reads the word
// with qfb_comm_read_status.  No multicast, no multimem: plain stores on peer pointers, polls on local memory.
#include <algorithm>
#include <cstdio>
#include <new>

#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxRows = 64;       // batch rows one reduction handles (one CTA each)
constexpr size_t kCommHeaderBytes = 1024;                                         // status word + epochs[kCommMaxRows] + step counter
constexpr int kCommStepWord = 1 + kCommMaxRows;                                   // header word of the step counter
constexpr size_t kCommDataOffset = kCommHeaderBytes;
// a data slot: [own partial, plain fp16: slot_bytes][receive regions, one per source rank: 2 * slot_bytes each]

struct CommArgs {
  char* base[kCommMaxWorld];   // symmetric buffers, by rank (base[rank] is local)
  char* local;                 // = base[rank] (kept apart: the kernel never indexes `base` with a run-time value)
  size_t slot_offset;          // byte offset of the data slot used by this call (its own-partial part)
  size_t recv_offset;          // byte offset of the slot's receive region of source rank 0
  size_t region_bytes;         // bytes between the receive regions of consecutive source ranks
  __half* x;                   // residual stream [rows, d], updated in place (null: no residual)
  const __half* w;             // norm weight [d] (null: no norm)
  __half* out;                 // normed row, or the plain sum when w is null
  int rank, d;
  float eps;
  unsigned long long timeout_ns;
  int pushed;                  // 1: the kernel that wrote the local partial has already sent it to the peers
  int idx;                     // >= 0: step numbering (the epoch is 2^31 | step << 8 | idx, nothing is advanced here)
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// 16 bytes that a peer may have written: read past the L1
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_v4(void* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void comm_cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void comm_st_cluster_f32(const float* local_addr, int cta_rank, float v) {
  const uint32_t la = static_cast<uint32_t>(__cvta_generic_to_shared(local_addr));
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(cta_rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}

// One batch row = one thread-block cluster of C CTAs (grid (C, rows)), each thread one 16-byte vector
// of the row: the peer stores and the polls of a row are spread over C SMs (a single SM moving the
// 2 * 16 KiB * (W - 1) bytes of an 8192-wide row was the long pole at four and eight ranks), and the
// sum of squares of the norm is combined through distributed shared memory with one cluster barrier.
template <int W, int C>
__global__ void __launch_bounds__(256) allreduce_add_rmsnorm_kernel(const CommArgs a) {   // (a CTA has at most 256 vectors)
  grid_launch_dependents();
  // shared memory of another CTA of the cluster may only be written once that CTA runs: every CTA
  // arrives here and waits for the others just before its first remote store (free by then)
  if (C > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  grid_dependency_wait();  // the partial in the local slot was written by the preceding kernel
  const int row = blockIdx.y, tid = threadIdx.x, crank = blockIdx.x;
  unsigned* status = reinterpret_cast<unsigned*>(a.local);
  unsigned* epochs = status + 1;
  __shared__ float red[32];
  __shared__ float css[8];   // sums of squares of the C CTAs of the row (pushed by every CTA into every CTA)
  // (per-row numbering: advanced by one thread once every CTA of the row has read it)
  const unsigned epoch = a.idx >= 0 ? (0x80000000u | (status[kCommStepWord] << 8) | (unsigned)a.idx) : epochs[row] + 1u;

  // ---- push this rank's partial of the row, epoch attached, into every peer's receive region ------
  const int nv = a.d >> 3;
  const int v = crank * blockDim.x + tid;    // this thread's vector of the row
  const bool active = v < nv;
  const size_t own_off = a.slot_offset + (size_t)row * a.d * 2;                                   // plain fp16
  const size_t recv_row = a.recv_offset + (size_t)row * a.d * 4;                                  // {data, epoch} words
  uint4 mine = make_uint4(0, 0, 0, 0);
  if (active) {
    mine = *reinterpret_cast<const uint4*>(a.local + own_off + (size_t)v * 16);   // written by the preceding kernel
    if (!a.pushed) {
      const size_t off = recv_row + (size_t)a.rank * a.region_bytes + (size_t)v * 32;
      const uint4 lo = make_uint4(mine.x, epoch, mine.y, epoch), hi = make_uint4(mine.z, epoch, mine.w, epoch);
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r != a.rank) {
          st_sys_v4(a.base[r] + off, lo);
          st_sys_v4(a.base[r] + off + 16, hi);
        }
    }
  }

  // ---- poll the peers' words of this thread in local memory until they carry the epoch; every pass
  // sums what it sees in rank order, the pass that finds every epoch in place is the one that counts ----
  float acc[8];
  const unsigned long long t0 = global_timer_ns();
  while (true) {
    bool pending = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < W; ++r) {
      uint4 p4 = mine;   // (the own partial: already in registers)
      if (active && r != a.rank) {
        const char* src = a.local + recv_row + (size_t)r * a.region_bytes + (size_t)v * 32;
        const uint4 lo = ld_sys_v4(src), hi = ld_sys_v4(src + 16);
        if (lo.y != epoch || lo.w != epoch || hi.y != epoch || hi.w != epoch) pending = true;
        p4 = make_uint4(lo.x, lo.z, hi.x, hi.z);
      }
      const uint32_t u[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(as_h2(u[j]));
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (!pending) break;
    if (global_timer_ns() - t0 > a.timeout_ns) {  // bounded: record it and go on with what is there
      atomicExch(status, 1u);
      break;
    }
  }

  // the reduced partial is rounded to fp16 (what a collective on fp16 tensors returns), then added
  // to the residual stream with one fp16 addition, as the unfused x + o does
  float ss = 0.f;
  if (active) {
    uint32_t o[4];
    if (a.x) {
      const uint4 xv = *reinterpret_cast<const uint4*>(a.x + (size_t)row * a.d + (size_t)v * 8);
      const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = as_u32(__hadd2(as_h2(xu[j]), __floats2half2_rn(acc[2 * j], acc[2 * j + 1])));
      *reinterpret_cast<uint4*>(a.x + (size_t)row * a.d + (size_t)v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = as_u32(__floats2half2_rn(acc[2 * j], acc[2 * j + 1]));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(as_h2(o[j]));
      acc[2 * j] = f.x;
      acc[2 * j + 1] = f.y;
      ss += f.x * f.x + f.y * f.y;
    }
    if (!a.w && a.out) {  // plain all-reduce (with or without the residual): the sum itself is the output
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = as_u32(__floats2half2_rn(acc[2 * j], acc[2 * j + 1]));
      *reinterpret_cast<uint4*>(a.out + (size_t)row * a.d + (size_t)v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }

  // ---- sum of squares of the row: warps -> CTA -> the C CTAs of the cluster, always in the same order ----
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  if (C > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // pairs with the arrive at the start
  if (tid == 0) {
    float t = 0.f;
    const int nwarps = (blockDim.x + 31) >> 5;
    for (int i = 0; i < nwarps; ++i) t += red[i];
    if (C == 1) css[0] = t;
    else
      for (int c = 0; c < C; ++c) comm_st_cluster_f32(&css[crank], c, t);
  }
  if (C > 1) comm_cluster_barrier();   // every CTA of the row has read the epoch and pushed its sum
  else __syncthreads();
  if (crank == 0 && tid == 0 && a.idx < 0) epochs[row] = epoch;
  if (!a.w || !active) return;
  float tot = 0.f;
#pragma unroll
  for (int c = 0; c < C; ++c) tot += css[c];
  const float rstd = rsqrtf(tot / (float)a.d + a.eps);
  const uint4 g = *reinterpret_cast<const uint4*>(a.w + (size_t)v * 8);
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // the normalised value is rounded to fp16 before the weight multiply, as rmsnorm_kernel does
    const __half2 n = __floats2half2_rn(acc[2 * j] * rstd, acc[2 * j + 1] * rstd);
    o[j] = as_u32(__hmul2(n, as_h2(gw[j])));
  }
  *reinterpret_cast<uint4*>(a.out + (size_t)row * a.d + (size_t)v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

template <int W, int C>
static cudaError_t launch_wc(const CommArgs& a, int rows, int nv, cudaStream_t st) {
  const int block = std::min(256, ((nv + C - 1) / C + 31) / 32 * 32);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C, rows);
  cfg.blockDim = dim3(block);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  int na = 1;
  if (C > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = C;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, allreduce_add_rmsnorm_kernel<W, C>, a);
}

// CTAs per row: enough that a CTA has at most 256 vectors (4 KiB of the row), at most 8
template <int W>
static cudaError_t launch_w(const CommArgs& a, int rows, int nv, cudaStream_t st) {
  if (nv > 1024) return launch_wc<W, 8>(a, rows, nv, st);
  if (nv > 256) return launch_wc<W, 4>(a, rows, nv, st);
  return launch_wc<W, 1>(a, rows, nv, st);
}

}  // namespace qfb

using namespace qfb;

struct qfb_comm {
  int rank, world, device;
  size_t slot_bytes;
  char* base[kCommMaxWorld];
  unsigned long long timeout_ns;
};

// bytes of one data slot: the own partial + a receive region ({data, epoch} words: twice the size) per source rank
static size_t comm_slot_span(size_t slot_bytes) { return slot_bytes * (1 + 2 * (size_t)kCommMaxWorld); }

namespace qfb {
int comm_collect_source(const qfb_comm* c, int slot, int idx, int rows, int d, CollectSource* s) {
  if (!c || !s) return QFB_ERR_NULL_POINTER;
  if (slot < 0 || slot > 1 || idx < 0 || idx > 255 || rows <= 0 || d <= 0 || d % 128 != 0) return QFB_ERR_BAD_SHAPE;
  if (rows > kCommMaxRows || (size_t)rows * d * 2 > c->slot_bytes) return QFB_ERR_TOO_LARGE;
  const size_t slot_offset = kCommDataOffset + (size_t)slot * comm_slot_span(c->slot_bytes);
  s->local = c->base[c->rank];
  s->own_offset = slot_offset;
  s->recv_offset = slot_offset + c->slot_bytes;
  s->region_bytes = 2 * c->slot_bytes;
  s->world = c->world;
  s->rank = c->rank;
  s->step = reinterpret_cast<const unsigned*>(c->base[c->rank]) + kCommStepWord;
  s->idx = (unsigned)idx;
  s->timeout_ns = c->timeout_ns;
  s->status = reinterpret_cast<unsigned*>(c->base[c->rank]);
  return QFB_OK;
}
int comm_push_target(const qfb_comm* c, int slot, int rows, int d, PushTarget* t, void** own_slot) {
  if (!c || !t || !own_slot) return QFB_ERR_NULL_POINTER;
  if (slot < 0 || slot > 1 || rows <= 0 || d <= 0 || d % 128 != 0) return QFB_ERR_BAD_SHAPE;
  if (rows > kCommMaxRows || (size_t)rows * d * 2 > c->slot_bytes) return QFB_ERR_TOO_LARGE;
  const size_t slot_offset = kCommDataOffset + (size_t)slot * comm_slot_span(c->slot_bytes);
  for (int r = 0; r < 8; ++r) t->base[r] = r < c->world ? c->base[r] : nullptr;
  t->world = c->world;
  t->rank = c->rank;
  t->recv_offset = slot_offset + c->slot_bytes + (size_t)c->rank * 2 * c->slot_bytes;
  t->epochs = reinterpret_cast<const unsigned*>(c->base[c->rank]) + 1;
  t->step = reinterpret_cast<const unsigned*>(c->base[c->rank]) + kCommStepWord;
  t->idx = -1;
  *own_slot = c->base[c->rank] + slot_offset;
  return QFB_OK;
}
}  // namespace qfb

static thread_local int tl_comm_cuda_error = 0;
static int comm_check(cudaError_t e) {
  if (e == cudaSuccess) return QFB_OK;
  tl_comm_cuda_error = (int)e;
  (void)cudaGetLastError();
  return QFB_ERR_CUDA;
}

extern "C" {

int qfb_comm_last_cuda_error(void) { return tl_comm_cuda_error; }

size_t qfb_comm_buffer_bytes(size_t slot_bytes) { return kCommDataOffset + 2 * comm_slot_span((slot_bytes + 255) / 256 * 256); }

int qfb_comm_max_rows(void) { return kCommMaxRows; }

int qfb_comm_alloc(size_t slot_bytes, void** base_out, void* ipc_handle_out) {
  if (!base_out || !ipc_handle_out) return QFB_ERR_NULL_POINTER;
  if (slot_bytes == 0) return QFB_ERR_BAD_SHAPE;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
  void* p = nullptr;
  const size_t total = qfb_comm_buffer_bytes(slot_bytes);
  int st = comm_check(cudaMalloc(&p, total));
  if (st != QFB_OK) return st;
  st = comm_check(cudaMemset(p, 0, total));
  if (st == QFB_OK) st = comm_check(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  if (st == QFB_OK) st = comm_check(cudaIpcGetMemHandle(&h, p));
  if (st != QFB_OK) {
    (void)cudaFree(p);
    return st;
  }
  memcpy(ipc_handle_out, &h, sizeof(h));
  *base_out = p;
  return QFB_OK;
}

int qfb_comm_free(void* base) { return base ? comm_check(cudaFree(base)) : QFB_OK; }

int qfb_comm_open(const void* ipc_handle, void** ptr_out) {
  if (!ipc_handle || !ptr_out) return QFB_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  return comm_check(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
}

int qfb_comm_close(void* ptr) { return ptr ? comm_check(cudaIpcCloseMemHandle(ptr)) : QFB_OK; }

int qfb_comm_create(int rank, int world, void* const* bases, size_t slot_bytes, qfb_comm** out) {
  if (!bases || !out) return QFB_ERR_NULL_POINTER;
  if (world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world || slot_bytes == 0) return QFB_ERR_BAD_SHAPE;
  for (int r = 0; r < world; ++r) {
    if (!bases[r]) return QFB_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(bases[r]) & 255u) return QFB_ERR_MISALIGNED;
  }
  qfb_comm* c = new (std::nothrow) qfb_comm();
  if (!c) return QFB_ERR_TOO_LARGE;
  c->rank = rank;
  c->world = world;
  c->device = 0;
  (void)cudaGetDevice(&c->device);
  c->slot_bytes = (slot_bytes + 255) / 256 * 256;
  for (int r = 0; r < kCommMaxWorld; ++r) c->base[r] = r < world ? static_cast<char*>(bases[r]) : nullptr;
  c->timeout_ns = 2000000000ull;
  *out = c;
  return QFB_OK;
}

void qfb_comm_destroy(qfb_comm* c) { delete c; }

void qfb_comm_set_timeout_us(qfb_comm* c, unsigned microseconds) {
  if (c) c->timeout_ns = (unsigned long long)(microseconds ? microseconds : 1u) * 1000ull;
}

void* qfb_comm_slot(const qfb_comm* c, int slot) {  // this rank's own partial of the local slot (plain fp16)
  if (!c || slot < 0 || slot > 1) return nullptr;
  return c->base[c->rank] + kCommDataOffset + (size_t)slot * comm_slot_span(c->slot_bytes);
}

void* qfb_comm_region(const qfb_comm* c, int slot, int source_rank) {  // receive region: {4 data bytes, epoch} words
  if (!c || slot < 0 || slot > 1 || source_rank < 0 || source_rank >= c->world) return nullptr;
  return c->base[c->rank] + kCommDataOffset + (size_t)slot * comm_slot_span(c->slot_bytes) + c->slot_bytes +
         (size_t)source_rank * 2 * c->slot_bytes;
}

static int allreduce_impl(qfb_comm* c, int slot, void* x, const void* w, void* out, int rows, int d, float eps,
                          int pushed, int idx, void* stream);

int qfb_allreduce_add_rmsnorm(qfb_comm* c, int slot, void* x, const void* w, void* out, int rows, int d, float eps,
                              void* stream) {
  return allreduce_impl(c, slot, x, w, out, rows, d, eps, 0, -1, stream);
}

int qfb_allreduce_add_rmsnorm_pushed(qfb_comm* c, int slot, void* x, const void* w, void* out, int rows, int d,
                                     float eps, void* stream) {
  return allreduce_impl(c, slot, x, w, out, rows, d, eps, 1, -1, stream);
}

int qfb_allreduce_add_rmsnorm_step(qfb_comm* c, int slot, int idx, void* x, const void* w, void* out, int rows, int d,
                                   float eps, void* stream) {
  if (idx < 0 || idx > 255) return QFB_ERR_BAD_SHAPE;
  return allreduce_impl(c, slot, x, w, out, rows, d, eps, 1, idx, stream);
}

static __global__ void comm_step_kernel(unsigned* header) { header[kCommStepWord] += 1u; }

int qfb_comm_step_begin(qfb_comm* c, void* stream) {
  if (!c) return QFB_ERR_NULL_POINTER;
  comm_step_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<unsigned*>(c->base[c->rank]));
  return comm_check(cudaGetLastError());
}

static int allreduce_impl(qfb_comm* c, int slot, void* x, const void* w, void* out, int rows, int d, float eps,
                          int pushed, int idx, void* stream) {
  if (!c) return QFB_ERR_NULL_POINTER;
  if (slot < 0 || slot > 1 || rows < 0 || d <= 0 || d % 8 != 0) return QFB_ERR_BAD_SHAPE;
  if (rows == 0) return QFB_OK;
  if (rows > kCommMaxRows || (size_t)rows * d * 2 > c->slot_bytes || d > 8 * 2 * 1024) return QFB_ERR_TOO_LARGE;
  if (w && !out) return QFB_ERR_NULL_POINTER;
  if (!x && !out) return QFB_ERR_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return QFB_ERR_MISALIGNED;
  CommArgs a;
  for (int r = 0; r < kCommMaxWorld; ++r) a.base[r] = c->base[r];
  a.local = c->base[c->rank];
  a.slot_offset = kCommDataOffset + (size_t)slot * comm_slot_span(c->slot_bytes);
  a.recv_offset = a.slot_offset + c->slot_bytes;
  a.region_bytes = 2 * c->slot_bytes;
  a.x = static_cast<__half*>(x);
  a.w = static_cast<const __half*>(w);
  a.out = static_cast<__half*>(out);
  a.rank = c->rank;
  a.d = d;
  a.eps = eps;
  a.timeout_ns = c->timeout_ns;
  a.pushed = pushed;
  a.idx = idx;
  const int nv = d / 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (c->world) {
    case 1: return comm_check(launch_w<1>(a, rows, nv, st));
    case 2: return comm_check(launch_w<2>(a, rows, nv, st));
    case 4: return comm_check(launch_w<4>(a, rows, nv, st));
    case 8: return comm_check(launch_w<8>(a, rows, nv, st));
    default: return QFB_ERR_UNSUPPORTED;
  }
}

int qfb_comm_epoch(qfb_comm* c, int row, void* stream, unsigned* epoch_out) {
  if (!c || !epoch_out) return QFB_ERR_NULL_POINTER;
  if (row < 0 || row >= kCommMaxRows) return QFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned done = 0;
  int s = comm_check(cudaMemcpyAsync(&done, c->base[c->rank] + 4 + 4 * (size_t)row, sizeof(unsigned), cudaMemcpyDeviceToHost, st));
  if (s != QFB_OK) return s;
  s = comm_check(cudaStreamSynchronize(st));
  if (s != QFB_OK) return s;
  *epoch_out = done + 1u;
  return QFB_OK;
}

int qfb_comm_read_status(qfb_comm* c, void* stream, unsigned* status_out) {
  if (!c || !status_out) return QFB_ERR_NULL_POINTER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int s = comm_check(cudaMemcpyAsync(status_out, c->base[c->rank], sizeof(unsigned), cudaMemcpyDeviceToHost, st));
  if (s != QFB_OK) return s;
  s = comm_check(cudaStreamSynchronize(st));
  if (s != QFB_OK) return s;
  if (*status_out) {  // report once, then start clean
    s = comm_check(cudaMemsetAsync(c->base[c->rank], 0, sizeof(unsigned), st));
    if (s != QFB_OK) return s;
    return QFB_ERR_DEVICE_FLAG;
  }
  return QFB_OK;
}

}  // extern "C"
