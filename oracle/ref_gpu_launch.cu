// Same-box GPU comparator: instantiates the REFERENCE project's own kernel template
// (qfactory/include/gptq_gemv.h:14-205 of the reference, included from where it lies; none of it
// is copied here) for the four Llama-7B layer shapes at M = 1, W4 g128 asymmetric, with the
// reference's default design point (qfactory/core/qfunc.py:29-43 of the reference: row-parallel,
// BLOCK_N 1, BLOCK_SIZE 128, eager decode) and NUM_ELM = 8, the largest value with
// NBITS * NUM_ELM <= 32, plus its scheduled point (qfactory/core/qfunc.py:96-103: activations kept
// in L2, quantisation parameters in shared memory).
//
// TEST / MEASUREMENT INFRASTRUCTURE ONLY (built into oracle/_ref/, never linked into the product):
// bench.py times it beside this library's kernel on the same box, and a parity test runs it on the
// reference's own packed layout to pin the CPU oracle against the reference's kernel.
//
// The reference bakes M, N, K into the template, as its JIT does (qfactory/core/qfunc.py:140-181).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gptq_gemv.h"

namespace {

template <int N, int K, bool SCHEDULED>
int launch_shape(half* a, int8_t* b, half* c, half* s, int8_t* z, cudaStream_t st) {
  //                    M  N  K  NBITS GS  SYM   BLOCK_N BLOCK_SIZE NUM_ELM EVICT_A     EVICT_B SMEM_QUANT DEFER  COL
  return gptq_gemv_impl<1, N, K, 4, 128, false, 1, 128, 8, !SCHEDULED, true, SCHEDULED, false, false>(a, b, c, s, z, st);
}

}  // namespace

// shape: 0 (12288,4096), 1 (4096,4096), 2 (22016,4096), 3 (4096,11008); scheduled: 0 default point, 1 scheduled point.
// activation fp16 [1,K]; weight int8 [N, K/2], scale fp16 [N, K/128], zero int8 [N, K/128/2] in the
// reference's packed layout (qfactory/convert.py:49-81 of the reference); output fp16 [1,N].
// Returns the reference launcher's code (0 = launched), or -1 for an unknown shape.
extern "C" int qf_ref_gptq_gemv(int shape, int scheduled, void* activation, void* weight, void* output, void* scale,
                                void* zero, void* stream) {
  half* a = static_cast<half*>(activation);
  int8_t* b = static_cast<int8_t*>(weight);
  half* c = static_cast<half*>(output);
  half* s = static_cast<half*>(scale);
  int8_t* z = static_cast<int8_t*>(zero);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (shape * 2 + (scheduled ? 1 : 0)) {
    case 0: return launch_shape<12288, 4096, false>(a, b, c, s, z, st);
    case 1: return launch_shape<12288, 4096, true>(a, b, c, s, z, st);
    case 2: return launch_shape<4096, 4096, false>(a, b, c, s, z, st);
    case 3: return launch_shape<4096, 4096, true>(a, b, c, s, z, st);
    case 4: return launch_shape<22016, 4096, false>(a, b, c, s, z, st);
    case 5: return launch_shape<22016, 4096, true>(a, b, c, s, z, st);
    case 6: return launch_shape<4096, 11008, false>(a, b, c, s, z, st);
    case 7: return launch_shape<4096, 11008, true>(a, b, c, s, z, st);
    default: return -1;
  }
}

extern "C" int qf_ref_last_cuda_error(void) { return (int)cudaGetLastError(); }
