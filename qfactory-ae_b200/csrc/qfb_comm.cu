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
// peer): a header, a flag table and two data slots.  The row-parallel GEMV writes its fp16 partial
// [rows, d] straight into a data slot of its own buffer.  The reduction kernel then runs one CTA
// per batch row:
//   1. thread p of the CTA stores this call's epoch into the flag (row, my rank) of PEER p's
//      table (st.release.sys), and polls the flag (row, p) of its OWN table (ld.acquire.sys)
//      until it holds that epoch: peer p's partial is complete.  Flags only ever grow, so a
//      replayed CUDA graph needs no reset; the epoch of a row lives in the local header and is
//      advanced by the kernel itself.
//   2. every thread pulls 16 bytes of the row from each rank's slot (plain peer loads, all in
//      flight together), sums them in rank order in fp32 (bit-identical on every rank), adds the
//      residual stream, and the CTA applies the RMS norm of the sum.
// Data slots alternate between consecutive reductions: a rank rewrites a slot only after it
// has passed the entry flags of the NEXT reduction, which every peer raises after it has finished
// reading that slot.
//
// Every wait is bounded (default 5 s, settable): when it runs out the CTA records it in the status
// word of the local header and carries on with whatever the slots hold; the host reads the word
// with qfb_comm_read_status.  No multicast, no multimem: plain loads and stores on peer pointers.
#include <cstdio>
#include <new>

#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxRows = 64;       // batch rows one reduction handles (one CTA each)
constexpr size_t kCommHeaderBytes = 1024;                                         // status word + epochs[kCommMaxRows]
constexpr size_t kCommFlagBytes = (size_t)kCommMaxRows * kCommMaxWorld * 4;       // flags[row][source rank]
constexpr size_t kCommDataOffset = kCommHeaderBytes + kCommFlagBytes;             // 3072: 16-byte aligned

struct CommArgs {
  char* base[kCommMaxWorld];   // symmetric buffers, by rank (base[rank] is local)
  size_t slot_offset;          // byte offset of the data slot used by this call
  __half* x;                   // residual stream [rows, d], updated in place (null: no residual)
  const __half* w;             // norm weight [d] (null: no norm)
  __half* out;                 // normed row, or the plain sum when w is null
  int rank, d;
  float eps;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// 16 bytes of (possibly peer) memory, past the L1 (the line may have been rewritten by its owner)
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// VPT = 16-byte vectors of the row each thread owns (d = 8 * VPT * blockDim.x at most)
template <int W, int VPT>
__global__ void __launch_bounds__(1024) allreduce_add_rmsnorm_kernel(const CommArgs a) {
  grid_launch_dependents();
  grid_dependency_wait();  // the partial in the local slot was written by the preceding kernel
  const int row = blockIdx.x, tid = threadIdx.x;
  unsigned* status = reinterpret_cast<unsigned*>(a.base[a.rank]);
  unsigned* epochs = status + 1;
  unsigned* my_flags = reinterpret_cast<unsigned*>(a.base[a.rank] + kCommHeaderBytes) + row * kCommMaxWorld;
  __shared__ float red[32];

  // ---- entry flags: tell every peer this rank's partial is in place, wait for theirs ----------
  if (tid < W && tid != a.rank) {
    const unsigned epoch = epochs[row] + 1u;
    unsigned* theirs = reinterpret_cast<unsigned*>(a.base[tid] + kCommHeaderBytes) + row * kCommMaxWorld + a.rank;
    st_release_sys(theirs, epoch);
    const unsigned long long t0 = global_timer_ns();
    while ((int)(ld_acquire_sys(my_flags + tid) - epoch) < 0) {
      if (global_timer_ns() - t0 > a.timeout_ns) {  // bounded: record it and go on
        atomicExch(status, 1u);
        break;
      }
    }
  }
  __syncthreads();
  if (tid == 0) epochs[row] += 1u;  // (every reader of epochs[row] is past the barrier)

  // ---- pull the row from every rank, sum in rank order ------------------------------------------
  const int nv = a.d >> 3;
  float acc[VPT][8];
  uint4 part[VPT][W];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
#pragma unroll
    for (int r = 0; r < W; ++r)
      if (v < nv) part[i][r] = ld_peer_v4(a.base[r] + a.slot_offset + ((size_t)row * a.d + (size_t)v * 8) * 2);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
    if (v >= nv) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int r = 0; r < W; ++r) {
      const uint32_t u[4] = {part[i][r].x, part[i][r].y, part[i][r].z, part[i][r].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(as_h2(u[j]));
        acc[i][2 * j] += f.x;
        acc[i][2 * j + 1] += f.y;
      }
    }
    // the reduced partial is rounded to fp16 (what a collective on fp16 tensors returns), then added
    // to the residual stream with one fp16 addition, as the unfused x + o does
    uint32_t o[4];
    if (a.x) {
      const uint4 xv = *reinterpret_cast<const uint4*>(a.x + (size_t)row * a.d + (size_t)v * 8);
      const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = as_u32(__hadd2(as_h2(xu[j]), __floats2half2_rn(acc[i][2 * j], acc[i][2 * j + 1])));
      *reinterpret_cast<uint4*>(a.x + (size_t)row * a.d + (size_t)v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = as_u32(__floats2half2_rn(acc[i][2 * j], acc[i][2 * j + 1]));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(as_h2(o[j]));
      acc[i][2 * j] = f.x;
      acc[i][2 * j + 1] = f.y;
      ss += f.x * f.x + f.y * f.y;
    }
  }
  if (!a.w) {  // plain all-reduce (with or without the residual): the sum itself is the output
    if (a.out) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * blockDim.x;
        if (v < nv) {
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = as_u32(__floats2half2_rn(acc[i][2 * j], acc[i][2 * j + 1]));
          *reinterpret_cast<uint4*>(a.out + (size_t)row * a.d + (size_t)v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
    return;
  }
  // ---- RMS norm of the updated row ---------------------------------------------------------------
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  const int nwarps = (blockDim.x + 31) >> 5;
  for (int i = 0; i < nwarps; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)a.d + a.eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * blockDim.x;
    if (v >= nv) continue;
    const uint4 g = *reinterpret_cast<const uint4*>(a.w + (size_t)v * 8);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // the normalised value is rounded to fp16 before the weight multiply, as rmsnorm_kernel does
      const __half2 n = __floats2half2_rn(acc[i][2 * j] * rstd, acc[i][2 * j + 1] * rstd);
      o[j] = as_u32(__hmul2(n, as_h2(gw[j])));
    }
    *reinterpret_cast<uint4*>(a.out + (size_t)row * a.d + (size_t)v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int W>
static cudaError_t launch_w(const CommArgs& a, int rows, int block, int vpt, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(block);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  switch (vpt) {
    case 1: return cudaLaunchKernelEx(&cfg, allreduce_add_rmsnorm_kernel<W, 1>, a);
    case 2: return cudaLaunchKernelEx(&cfg, allreduce_add_rmsnorm_kernel<W, 2>, a);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace qfb

using namespace qfb;

struct qfb_comm {
  int rank, world, device;
  size_t slot_bytes;
  char* base[kCommMaxWorld];
  unsigned long long timeout_ns;
};

static thread_local int tl_comm_cuda_error = 0;
static int comm_check(cudaError_t e) {
  if (e == cudaSuccess) return QFB_OK;
  tl_comm_cuda_error = (int)e;
  (void)cudaGetLastError();
  return QFB_ERR_CUDA;
}

extern "C" {

int qfb_comm_last_cuda_error(void) { return tl_comm_cuda_error; }

size_t qfb_comm_buffer_bytes(size_t slot_bytes) { return kCommDataOffset + 2 * ((slot_bytes + 255) / 256 * 256); }

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
  c->timeout_ns = 5000000000ull;
  *out = c;
  return QFB_OK;
}

void qfb_comm_destroy(qfb_comm* c) { delete c; }

void qfb_comm_set_timeout_us(qfb_comm* c, unsigned microseconds) {
  if (c) c->timeout_ns = (unsigned long long)(microseconds ? microseconds : 1u) * 1000ull;
}

void* qfb_comm_slot(const qfb_comm* c, int slot) {
  if (!c || slot < 0 || slot > 1) return nullptr;
  return c->base[c->rank] + kCommDataOffset + (size_t)slot * c->slot_bytes;
}

/* byte offset of flag (row, source rank) inside a symmetric buffer (tests pre-raise flags with it) */
size_t qfb_comm_flag_offset(int row, int source_rank) {
  return kCommHeaderBytes + ((size_t)row * kCommMaxWorld + (size_t)source_rank) * 4;
}

int qfb_allreduce_add_rmsnorm(qfb_comm* c, int slot, void* x, const void* w, void* out, int rows, int d, float eps,
                              void* stream) {
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
  a.slot_offset = kCommDataOffset + (size_t)slot * c->slot_bytes;
  a.x = static_cast<__half*>(x);
  a.w = static_cast<const __half*>(w);
  a.out = static_cast<__half*>(out);
  a.rank = c->rank;
  a.d = d;
  a.eps = eps;
  a.timeout_ns = c->timeout_ns;
  const int nv = d / 8;
  const int vpt = nv > 1024 ? 2 : 1;
  const int block = std::min(1024, ((nv + vpt - 1) / vpt + 31) / 32 * 32);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (c->world) {
    case 1: return comm_check(launch_w<1>(a, rows, block, vpt, st));
    case 2: return comm_check(launch_w<2>(a, rows, block, vpt, st));
    case 4: return comm_check(launch_w<4>(a, rows, block, vpt, st));
    case 8: return comm_check(launch_w<8>(a, rows, block, vpt, st));
    default: return QFB_ERR_UNSUPPORTED;
  }
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
