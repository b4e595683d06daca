// Allocation-free entry point for callers that are not allowed to call cudaMalloc.
//
// Some hosts embed this library where device allocation is off the table at call time: a
// serving process whose memory pool was carved up at start-up and is owned by another
// component, code running between the nodes of a pre-planned execution schedule, or a plugin
// sandbox that forbids allocator calls.  Such a caller cannot create the split-K workspace the
// regular entry point wants.  For them the scratch lives in this translation unit as a
// file-scope device array of fixed size; every GPU that loads the library holds its own copy
// until the process exits.
#include <mutex>

#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {
int validate_forward_args(const qfb_layer* layer, const void* x, int m, const void* y);  // qfb_api.cu
}

namespace {

// 8 MiB: enough for the split-K partial sums and counters of every Llama-7B-class layer at up
// to 8 activation rows per pass (largest: 22016 x 4096 needs about 5.7 MiB).
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// Resolves the DEVICE address of the array for the current device.  In host code the name
// `g_static_scratch` is only a handle for the runtime, never a pointer a kernel may use.
int scratch_for_current_device(void** out) {
  int dev = -1;
  const cudaError_t ge = cudaGetDevice(&dev);
  if (ge != cudaSuccess) return qfb::record_cuda_error(ge);
  if (dev < 0 || dev >= kMaxDevices) return QFB_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t se = cudaGetSymbolAddress(&p, g_static_scratch);
    if (se != cudaSuccess) return qfb::record_cuda_error(se);  // (readable through qfb_last_cuda_error)
    if (!p) return QFB_ERR_CUDA;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return QFB_OK;
}

}  // namespace

extern "C" {

size_t qfb_static_scratch_capacity(void) { return kStaticScratchBytes; }

int qfb_gemv_forward_static(const qfb_layer* layer, const void* x, int m, void* y, unsigned flags, void* stream) {
  if (!layer) return QFB_ERR_NULL_POINTER;
  if (m < 0) return QFB_ERR_BAD_SHAPE;
  if (m == 0) return QFB_OK;
  if (layer->layout != QFB_LAYOUT_TILE) return QFB_ERR_UNSUPPORTED;  // the CUDA-core kernel reads the tile layout
  // every argument is checked before the shared array is touched: a rejected call leaves it alone
  const int va = qfb::validate_forward_args(layer, x, m, y);
  if (va != QFB_OK) return va;
  // the split-K kernel handles 8 rows per pass and reuses the scratch between passes
  const size_t need = qfb::gemv_scratch_bytes(m, layer->n, layer->k, layer->bits);
  if (need == 0) return QFB_ERR_BAD_SHAPE;
  if (need > kStaticScratchBytes) return QFB_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int st = scratch_for_current_device(&scratch);
  if (st != QFB_OK) return st;
  // The array keeps whatever the previous call left behind.  The kernel needs its status word
  // and arrival counters to start at zero (the partial sums are always written before they are
  // read), so that prefix, and only it, is cleared on the caller's stream before the launch.
  const int sc = qfb_workspace_init(scratch, qfb::scratch_clear_bytes(layer->n), stream);
  if (sc != QFB_OK) return sc;
  return qfb_linear_forward(layer, x, m, y, scratch, kStaticScratchBytes,
                            (flags & ~QFB_FLAG_FORCE_TENSOR) | QFB_FLAG_FORCE_SIMT, stream);
}

}  // extern "C"
