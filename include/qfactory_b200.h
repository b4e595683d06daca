/*
 * qfactory_b200.h -- C ABI of the B200 (sm_100a) weight-only-quantized linear layer.
 *
 * Computes  y[M,N] = x[M,K] . dequant(W)[N,K]^T  for 2/3/4/8-bit group-quantized
 * weights, fp16 activations, fp32 accumulation and fp16 output.
 *
 * Conventions (the same as the reference's FFI, whose `launch` symbols these replace):
 *   - every pointer is a borrowed DEVICE pointer unless its name ends in `_host`;
 *     the library never allocates or frees device memory in the entry points of this
 *     section and never synchronises the device unless documented;
 *   - work is ordered on the cudaStream_t passed as `stream` (NULL = legacy default);
 *   - every entry point returns a qfb_status (0 = success); nothing is printed.
 *   - re-entrancy: calls on different streams must use different workspaces.
 *
 * Packed layout ("tile-128 interleaved", produced by qfb_pack or by the Python
 * `qfactory.convert.convert_params`):  rows (output features) are padded to a
 * multiple of 128 and grouped in tiles of 128; along K the codes are cut in chunks of
 * 16 bytes per row (128/bits codes; for 3 bits a unit of 128 codes is two 2-bit-plane
 * chunks followed by one 1-bit-plane chunk).
 *   qweight  u8 [Npad/128][K chunks][128 rows][16]      one 128-bit load per row and chunk
 *   scales   f16[Npad/128][K/group ][128 rows]
 *   zeros    u8 [Npad/128][K/group ][128 rows]          effective zero, see below
 * Inside a 32-bit word the 2/4-bit fields are pair-interleaved (even elements in the low
 * half-word, odd ones in the high half-word) so that one LOP3 yields an fp16x2 pair.
 *
 * Second packed layout ("fragment", QFB_LAYOUT_FRAGMENT, layers with K % 128 == 0):
 * the same bytes permuted so that the words of a lane are the A fragments one thread feeds to the
 * warp-level tensor-core instruction (rows g and g+8 of a 16-row block, four k each):
 *   qweight  [Npad/128][2 x 64 rows][K/16 steps of 128*bits bytes][32 lanes][words of 4 row blocks]
 *            (4-bit: one word per row block; 8-bit: two, in two 512-byte chunks per step;
 *             2-bit: one word per pair of row blocks; 3-bit: three words for the four row blocks,
 *             word j of all lanes a 128-byte plane of the step, five 3-bit fields and one spare
 *             bit per half-word, the sixteenth field pair in the spare bits)
 *   scales / zeros  [Npad/128][K/group][128] in fragment row order
 * Batches of at most 16 rows run the mma.sync GEMV on it, larger ones the tcgen05 kernel, which
 * reads the same words; it is the layout of choice whenever the shape allows it.
 *
 * Zero-point semantics follow the reference packer and kernel: the stored, effective
 * zero is min(z + 1, 2^bits - 1) for GPTQ-convention zeros z
 * (reference: qfactory/convert.py:76, qfactory/include/utils.h:53-60); symmetric layers
 * (zeros == NULL) subtract 2^(bits-1) (reference: qfactory/include/gptq_gemv.h:72-73);
 * group-less layers (scales == NULL, group_size == -1) multiply raw unsigned codes
 * (reference: qfactory/include/gemv.h:12-94).
 */
#ifndef QFACTORY_B200_H_
#define QFACTORY_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum qfb_status {
  QFB_OK = 0,
  QFB_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
  QFB_ERR_BAD_SHAPE = 2,      /* M, N, K or group size violate the layout rules */
  QFB_ERR_UNSUPPORTED = 3,    /* bit width / mode / kernel not available */
  QFB_ERR_MISALIGNED = 4,     /* a pointer is not 16-byte aligned */
  QFB_ERR_WORKSPACE = 5,      /* workspace missing or too small */
  QFB_ERR_CUDA = 6,           /* a CUDA runtime call failed; see qfb_last_cuda_error */
  QFB_ERR_TOO_LARGE = 7,      /* request exceeds a fixed capacity */
  QFB_ERR_DEVICE_FLAG = 8     /* a kernel reported a bounded wait that ran out */
} qfb_status;

/* flags for qfb_linear_forward */
#define QFB_FLAG_PDL 1u          /* launch with programmatic stream serialisation: the kernel
                                    prefetches weights before it waits for the preceding kernel */
#define QFB_FLAG_FORCE_SIMT 2u   /* never the tcgen05 kernel: tile-layout layers run the CUDA-core
                                    split-K kernel, fragment-layout layers the mma.sync GEMV (in
                                    passes of 16 rows), whatever the batch size */
#define QFB_FLAG_FORCE_TENSOR 4u /* tile-layout layers: always the tcgen05 kernel (if the shape
                                    allows); fragment-layout layers still run the mma.sync GEMV
                                    up to 16 rows */
#define QFB_FLAG_NO_SYNC 8u      /* qfb_linear_forward_host only: do not synchronise the stream; the
                                    caller queues several layers and synchronises once */

#define QFB_FLAG_TEST_STALLED_WAIT 16u /* test aid for the bounded device-side waits: the kernel's first
                                    bulk-copy barrier is told to expect 16 bytes that never come and every
                                    wait gives up after ~100 us instead of ~1 s.  The copies themselves all
                                    land; the launch returns, the status word of the workspace is set
                                    (qfb_read_status -> QFB_ERR_DEVICE_FLAG).  The mma.sync GEMV still
                                    produces the right output; the tcgen05 kernel abandons the launch
                                    (its output is undefined).  Needs a workspace. */

/* packed layouts */
#define QFB_LAYOUT_TILE 0      /* tile-128 interleaved: every bit width, every batch size */
#define QFB_LAYOUT_FRAGMENT 1  /* tensor-core fragment order: K % 128 == 0, group 64 (not 3-bit) / n*128 / none */

/* One packed layer.  Plain data; the caller owns the device buffers. */
typedef struct qfb_layer {
  const void* qweight;   /* packed codes, 16-byte aligned */
  const void* scales;    /* packed fp16 scales, or NULL for a group-less layer */
  const void* zeros;     /* packed effective zeros, or NULL for symmetric / group-less */
  int32_t n;             /* out_features (unpadded) */
  int32_t k;             /* in_features */
  int32_t bits;          /* 2, 3, 4 or 8 */
  int32_t group_size;    /* multiple of 64 dividing k, or -1 for group-less */
  int32_t layout;        /* QFB_LAYOUT_TILE or QFB_LAYOUT_FRAGMENT */
} qfb_layer;

/* Library / layout version (major*100 + minor). */
int qfb_version(void);
const char* qfb_status_string(int status);
/* cudaError_t of the last failed runtime call seen by this thread (0 if none). */
int qfb_last_cuda_error(void);

/* Sizes of the packed buffers in bytes (0 on invalid arguments). */
size_t qfb_packed_weight_bytes(int n, int k, int bits);
size_t qfb_packed_scale_bytes(int n, int k, int group_size);
size_t qfb_packed_zero_bytes(int n, int k, int group_size);

/* Bytes of workspace qfb_linear_forward needs for up to m_max activation rows.
 * The workspace holds split-K partial sums and per-tile arrival counters. */
size_t qfb_workspace_bytes(int m_max, int n, int k, int bits);
/* Must be called once on a fresh workspace (zeroes the arrival counters, stream-ordered). */
int qfb_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/*
 * The hot path.  Replaces the reference's JIT-emitted
 *   extern "C" void launch(void* activation, void* weight, void* output, void* scale,
 *                          void* zero, void* stream, int& __return_code)
 * (reference: qfactory/core/qfunc.py:140-152, launcher qfactory/include/gptq_gemv.h:156-205)
 * and, with layer->scales == NULL, its group-less variant
 *   extern "C" void launch(int m, void* activation, void* weight, void* output,
 *                          void* stream, int& __return_code)
 * (reference: qfactory/core/qfunc.py:280-292, launcher qfactory/include/gemv.h:96-135).
 * Unlike the reference M is a run-time argument.
 *   x  fp16 [m, k] row-major, 16-byte aligned;  y  fp16 [m, n] row-major.
 */
int qfb_linear_forward(const qfb_layer* layer, const void* x, int m, void* y,
                       void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/*
 * The down projection of a gated MLP with its activation fused in: y = (silu(gate) * up) . dequant(W)^T
 * for gate_up fp16 [m, 2k] = [gate | up] as the fused gate/up linear writes it.  The combination
 * (silu in fp32 rounded to fp16, one fp16 product: the arithmetic of qfb_silu_mul) happens while the
 * GEMV stages its activations, so the separate element-wise launch of the reference's serving stack
 * (third_party/vllm-bitblas/vllm/model_executor/models/llama.py:91-96) and its [m, k] tensor go away.
 * Fragment-layout layers and m <= 16 only (the mma.sync GEMV); otherwise QFB_ERR_UNSUPPORTED and the
 * caller runs qfb_silu_mul + qfb_linear_forward.  Results are bit-identical to that pair.
 */
int qfb_linear_silu_mul_forward(const qfb_layer* layer, const void* gate_up, int m, void* y, void* workspace,
                                size_t workspace_bytes, unsigned flags, void* stream);

/*
 * Same computation for callers that hold HOST buffers: copies x_host (pinned or pageable)
 * into x_staging, runs the layer, copies the result into y_host and synchronises `stream`
 * before returning (unless QFB_FLAG_NO_SYNC is set: then y_host is valid once the caller has
 * synchronised the stream, and the staging buffers must not be reused before that).  x_staging / y_staging are caller-owned device buffers of m*k and m*n
 * fp16 elements.  No counterpart in the reference (its callers hold device tensors).
 */
int qfb_linear_forward_host(const qfb_layer* layer, const void* x_host, int m, void* y_host,
                            void* x_staging, void* y_staging, void* workspace,
                            size_t workspace_bytes, unsigned flags, void* stream);

/*
 * The split-K GEMV for callers that cannot allocate device memory (a process whose device
 * pool is owned elsewhere, code between the steps of a fixed schedule, an allocator-free
 * plugin sandbox).  It has no counterpart in the reference.  Same computation as
 * qfb_linear_forward on the CUDA-core kernel, but the split-K scratch is a fixed device array
 * inside the library (qfb_static_scratch_capacity() bytes, 8 MiB, held by every GPU that loads
 * the library until the process exits) instead of a caller workspace; the caller still passes
 * x and y.  It calls no allocator.  Shapes whose scratch need exceeds the capacity return
 * QFB_ERR_TOO_LARGE.  The first call on each device looks up the array's device address (with
 * that device current); make that first call before any stream capture.  All calls on a device
 * share the one array, which keeps the previous call's contents (the part that must start at
 * zero is cleared on `stream` by each call): calls that overlap on the GPU race and must be
 * serialised by the caller.
 */
int qfb_gemv_forward_static(const qfb_layer* layer, const void* x, int m, void* y, unsigned flags,
                            void* stream);
size_t qfb_static_scratch_capacity(void);

/* Which kernel qfb_linear_forward picks for a tile-layout layer: 1 = SIMT split-K GEMV,
 * 2 = tcgen05 GEMM, 0 = invalid.  Fragment-layout layers run kernel 3 (mma.sync GEMV) up to 16
 * rows and kernel 2 above. */
int qfb_select_kernel(int m, int n, int k, int bits, unsigned flags);

/* Smallest batch that is routed to the tensor-core kernel (default 2).  Process-wide. */
void qfb_set_tensor_min_batch(int min_m);
/* Reads the workspace's status word (synchronises `stream`): returns QFB_ERR_DEVICE_FLAG and
 * *status_out != 0 when a kernel gave up on a bounded wait since qfb_workspace_init. */
int qfb_read_status(const void* workspace, void* stream, unsigned* status_out);

/* Debug / tuning override of the split-K heuristic of the SIMT kernel: split_k <= 0 and
 * k_ways <= 0 restore the built-in choice.  Process-wide, not thread-safe. */
void qfb_set_gemv_tuning(int split_k, int k_ways);
/* Tuning override of the tensor-core kernel's K split (0 = built-in): the split-K factor for batches
 * <= 64; above 64 rows, values 2..4 cut every (row tile, batch tile) unit into that many K ranges. */
void qfb_set_tensor_split(int split_k);
/* Tuning override of the tensor-core kernel's batch tile above 64 rows: 64, 128 or 256 columns
 * (0 = built-in choice). */
void qfb_set_tensor_batch_tile(int columns);
/* Tuning override of the tensor-core kernel's decode groups where it scales in the decode (batches
 * > 32, or groups of 64): 1 = eight decode warps (two CTAs per SM for batch tiles up to 128 columns),
 * 2 = two groups of eight that take alternate stages (one CTA per SM); 0 = built-in choice. */
void qfb_set_tensor_decode_groups(int groups);
/* mma.sync GEMV (fragment layout), how K splits are reduced: 1 (default) lets the cost model
 * choose between a thread-block cluster (distributed shared memory, at most 8 splits) and the
 * workspace; 0 always uses the workspace; 2 uses a cluster whenever there are 2..8 splits. */
void qfb_set_cluster_reduce(int mode);
/* The configuration the last qfb_linear_forward of this thread used (for reports). */
void qfb_get_last_launch(int* kernel, int* grid_x, int* grid_y, int* block, int* smem_bytes);

/*
 * Offline packer on the device.  Replaces qfactory/convert.py:84-97 (convert_params).
 *   codes   i32 [k, n]  values in [0, 2^bits)
 *   scales  f16 [k/group, n]            (NULL for group-less)
 *   zeros   i32 [k/group, n] GPTQ convention (NULL for symmetric / group-less); the packer
 *           stores min(z + 1, 2^bits - 1)
 * Outputs are the three packed buffers described at the top of this file.
 */
int qfb_pack(const int32_t* codes, const void* scales, const int32_t* zeros, int n, int k,
             int bits, int group_size, void* qweight_out, void* scales_out, void* zeros_out,
             void* stream);

/* qfb_pack into the given layout; 1 when the layout can hold the shape, else 0. */
int qfb_pack_layout(const int32_t* codes, const void* scales, const int32_t* zeros, int n, int k,
                    int bits, int group_size, int layout, void* qweight_out, void* scales_out,
                    void* zeros_out, void* stream);
int qfb_layout_supported(int layout, int n, int k, int bits, int group_size);

/*
 * fp16 weight [k, n] -> group-wise asymmetric quantisation, the front end of "construct a layer
 * from an fp16 weight".  Replaces the reference's test helper asymmetric_quant
 * (tests/acc_gptq.py:10-29) bit for bit: per group of group_size rows and per column
 *   scale = (max - min) / (2^bits - 1),  zero = trunc(max(-min / (max - min) * (2^bits - 1) - 1, 0)),
 *   code  = trunc((w - min) / (max - min) * (2^bits - 1)),      every operation rounded to fp16.
 * Outputs: codes i32 [k, n], scales f16 [k/group, n], zeros i32 [k/group, n] (GPTQ "zero - 1"
 * convention): exactly the inputs of qfb_pack.
 */
int qfb_quantize(const void* weight, int k, int n, int bits, int group_size, int32_t* codes_out,
                 void* scales_out, int32_t* zeros_out, void* stream);

/* Inverse of the code packing through the kernels' own bit-extraction path:
 * writes i32 codes [k, n].  Used by the bit-exactness tests. */
int qfb_unpack_codes(const qfb_layer* layer, int32_t* codes_out, void* stream);
/* Dequantised fp16 weight [k, n] = (q - z_eff) * s, through the kernels' decode path. */
int qfb_dequantize(const qfb_layer* layer, void* w_out, void* stream);

/*
 * Element-wise neighbours of the quantized linears in a decoder layer, one launch each.  The
 * reference leaves them to its serving stack
 * (third_party/vllm-bitblas/vllm/model_executor/models/llama.py:60-120, 260-285).
 *   qfb_rmsnorm:  y[r,:] = fp16(x[r,:] * rsqrt(mean(x[r,:]^2) + eps)) * w     x, y fp16 [rows, d], w fp16 [d]
 *   qfb_add_rmsnorm: x[r,:] += residual[r,:] in place (one fp16 addition), then y = the norm of the sum:
 *                 the residual add after O / down and the next norm in one pass
 *   qfb_silu_mul: out[r,j] = silu(gate_up[r,j]) * gate_up[r,half+j]           gate_up fp16 [rows, 2*half]
 *   qfb_rope_cache: rotary embedding (interleaved pairs, fp16 arithmetic) of the query and key heads
 *                 of qkv fp16 [B, T, hq + 2 hkv, hd], in place, at positions pos i64 [T]; the rotated
 *                 keys and the values are also written into k_cache / v_cache fp16
 *                 [B, hkv, max_len, hd] at those positions.  cos, sin fp16 [max_len, hd / 2].
 *                 A position outside [0, max_len) is skipped: no rotation and no cache write for
 *                 that token (qfb_decode_attention clamps the same way), so a graph replayed past
 *                 the cache length never writes out of bounds.
 * d and half are multiples of 8, hd is even; all pointers 16-byte aligned.
 */
int qfb_rope_cache(void* qkv, const void* cos, const void* sin, const void* pos, void* k_cache, void* v_cache,
                   int batch, int tokens, int q_heads, int kv_heads, int head_dim, int max_len, void* stream);
int qfb_rmsnorm(const void* x, const void* w, void* y, int rows, int d, float eps, void* stream);
int qfb_add_rmsnorm(void* x, const void* residual, const void* w, void* y, int rows, int d, float eps, void* stream);
int qfb_silu_mul(const void* gate_up, void* out, int rows, int half, void* stream);
/*
 * Single-query (decode step) attention over the static cache, one launch: for every batch row and
 * query head, softmax(q . K^T / sqrt(hd)) . V over the keys 0 .. pos[0] (pos: one i64 on the
 * device, so a captured graph can be replayed at the next position).
 *   qkv fp16 [B, hq + 2 hkv, hd] (queries already rotated, e.g. by qfb_rope_cache, which also wrote
 *   position pos into the caches); k_cache, v_cache fp16 [B, hkv, max_len, hd]; out fp16 [B, hq * hd].
 * hd = 128, hq / hkv in {1, 2, 4, 8}, max_len <= 16384; otherwise QFB_ERR_UNSUPPORTED.
 */
int qfb_decode_attention(const void* qkv, const void* pos, const void* k_cache, const void* v_cache, void* out,
                         int batch, int q_heads, int kv_heads, int head_dim, int max_len, void* stream);
/*
 * The same with the single-token work of qfb_rope_cache fused in: qkv holds the UN-rotated queries, key
 * and value of the new token; the kernel rotates the queries as it stages them, rotates the new key,
 * attends over the cached keys 0 .. pos[0] - 1 plus the new one, and writes the rotated key and the
 * value into the caches at position pos[0] (one CTA per batch row and key/value head does the write).
 * qkv is not modified.  Same arithmetic, bit for bit, as qfb_rope_cache followed by
 * qfb_decode_attention; one launch less per decoder layer.  cos, sin fp16 [max_len, hd / 2], 8-byte
 * aligned.  A position outside [0, max_len) is not rotated and not written.
 */
int qfb_decode_attention_rope(const void* qkv, const void* cos, const void* sin, const void* pos, void* k_cache,
                              void* v_cache, void* out, int batch, int q_heads, int kv_heads, int head_dim,
                              int max_len, void* stream);

/*
 * One-shot all-reduce over peer memory for the row-parallel linears (O and down projections) of a
 * tensor-parallel decoder, fused with the residual add and the RMS norm that follow it.  Replaces
 * the collective after a row-parallel linear in the reference's serving stack
 * (third_party/vllm-bitblas/vllm/model_executor/layers/linear.py:1100-1124; the one-shot
 * peer-memory kernel that stack prefers for small messages:
 * third_party/vllm-bitblas/csrc/custom_all_reduce.cuh:133-150, 210-226).
 *
 * Set-up (allocates; once per process, not on the hot path): every rank calls qfb_comm_alloc,
 * exchanges the 64-byte handle with its peers by any means (the Python side uses the process
 * group), opens the peers' handles with qfb_comm_open and hands the `world` base pointers, by
 * rank, to qfb_comm_create.  A rank's buffer holds a status word, per-row epochs and two data
 * slots; a slot is this rank's own partial (plain fp16, `slot_bytes`) followed by one receive
 * region per source rank (8-byte words {4 data bytes, epoch}: 2 * `slot_bytes` each).
 *
 * Use: the row-parallel linear writes its fp16 partial [rows, d] into the local slot
 * (qfb_comm_slot); qfb_allreduce_add_rmsnorm stores it, epoch attached, into this rank's receive
 * region of every peer's buffer (peer stores), polls its own receive regions in local memory until
 * every word carries the call's epoch (no flag exchange, no fence: one NVLink one-way latency), and
 * then computes, identically on every rank,
 *     s = fp16(sum over ranks of the partials, in rank order, fp32)
 *     x != NULL:  x[r,:] += s (in place, one fp16 addition);  otherwise the row is s itself
 *     w != NULL:  out[r,:] = fp16(row * rsqrt(mean(row^2) + eps)) * w;   w == NULL: out = row (if out)
 * Consecutive reductions on a communicator MUST alternate between slot 0 and slot 1, and every
 * rank must issue the same sequence of calls (rows, slot): that is what makes a slot safe to
 * rewrite.  rows <= qfb_comm_max_rows(), rows * d * 2 <= slot_bytes, d % 8 == 0, d <= 16384,
 * world in {1, 2, 4, 8}.  Peer memory is written with plain stores; no multicast.
 * qfb_comm_region(comm, slot, r) is the receive region of source rank r inside the local slot and
 * qfb_comm_epoch(comm, row, stream) the epoch the NEXT reduction of a row will use (tests that play
 * a peer's part write its words there; the call synchronises the stream).
 *
 * Every wait is bounded (qfb_comm_set_timeout_us, default 2 s): when it runs out the kernel records
 * it and returns normally with whatever the regions held; qfb_comm_read_status then returns
 * QFB_ERR_DEVICE_FLAG once and clears the word.  CUDA-graph safe: epochs only grow and live in
 * device memory.
 */
typedef struct qfb_comm qfb_comm;
size_t qfb_comm_buffer_bytes(size_t slot_bytes);
int qfb_comm_max_rows(void);
int qfb_comm_alloc(size_t slot_bytes, void** base_out, void* ipc_handle_out /* 64 bytes */);
int qfb_comm_free(void* base);
int qfb_comm_open(const void* ipc_handle, void** ptr_out);
int qfb_comm_close(void* ptr);
int qfb_comm_create(int rank, int world, void* const* bases, size_t slot_bytes, qfb_comm** out);
void qfb_comm_destroy(qfb_comm* comm);
void qfb_comm_set_timeout_us(qfb_comm* comm, unsigned microseconds);
void* qfb_comm_slot(const qfb_comm* comm, int slot);
void* qfb_comm_region(const qfb_comm* comm, int slot, int source_rank);
int qfb_comm_epoch(qfb_comm* comm, int row, void* stream, unsigned* epoch_out);
int qfb_allreduce_add_rmsnorm(qfb_comm* comm, int slot, void* x, const void* w, void* out, int rows, int d,
                              float eps, void* stream);
/*
 * A linear with the residual add and the RMS norm in front of it fused in (reference: separate kernels
 * around the linears, third_party/vllm-bitblas/vllm/model_executor/models/llama.py:260-285):
 *   s = x + residual (one fp16 addition per element; residual may be NULL), written to x_out (may be NULL;
 *   never x or residual themselves: other blocks of the launch still read them);
 *   y = (rmsnorm(s) * norm_weight) . dequant(W)^T.
 * The blocks of the GEMV add, weight and square their K slices while staging them; 1 / rms, a scalar per
 * row, is applied to the result, so the activations are rounded to fp16 once (s * w) instead of twice: y
 * differs from the three-call form by that rounding (within 2e-3 of max|y| in the tests), x_out is
 * bit-identical.  Up to 16 rows of a 4-bit fragment-layout layer with groups of 128 or more;
 * otherwise QFB_ERR_UNSUPPORTED.
 */
int qfb_linear_addnorm_forward(const qfb_layer* layer, const void* x, const void* residual, void* x_out,
                               const void* norm_weight, float eps, int m, void* y, void* workspace,
                               size_t workspace_bytes, unsigned flags, void* stream);

/* The same reduction when the kernel that wrote the partial has already sent it to the peers
 * (qfb_linear_forward_reduce below): the launch only collects, sums, adds and normalises. */
int qfb_allreduce_add_rmsnorm_pushed(qfb_comm* comm, int slot, void* x, const void* w, void* out, int rows, int d,
                                     float eps, void* stream);
/* A row-parallel linear fused with the first half of its reduction (reference: the matmul and the
 * collective call are separate steps, third_party/vllm-bitblas/vllm/model_executor/layers/linear.py:1100-1124):
 * y = x . dequant(W)^T is this rank's partial [m, n] of a sum over the ranks; the kernel writes it into
 * data slot `slot` of the communicator and, as it stores each result, also sends it to every peer (plain
 * peer stores, the reduction's epoch attached to every 4 bytes).  Follow it with
 * qfb_allreduce_add_rmsnorm_pushed on the same slot.  Up to 16 rows of a 4-bit fragment-layout layer
 * (groups of 128 or more, or group-less) whose n is a multiple of 128 and equals the communicator's row
 * width; otherwise QFB_ERR_UNSUPPORTED (use
 * qfb_linear_forward with y = qfb_comm_slot(...) and the plain reduction instead).  The second form takes
 * the fused gate/up tensor of qfb_linear_silu_mul_forward. */
int qfb_linear_forward_reduce(const qfb_layer* layer, const void* x, int m, qfb_comm* comm, int slot,
                              void* workspace, size_t workspace_bytes, unsigned flags, void* stream);
int qfb_linear_silu_mul_forward_reduce(const qfb_layer* layer, const void* gate_up, int m, qfb_comm* comm, int slot,
                                       void* workspace, size_t workspace_bytes, unsigned flags, void* stream);
/*
 * Step numbering: the exchange without a kernel that advances epochs, so that the RECEIVING side can be the
 * GEMV that consumes the sum.  qfb_comm_step_begin (one tiny launch at the start of a decode step; every
 * rank) advances a counter in the local buffer that nothing changes during the step; reduction `idx`
 * (0..255, the same on every rank, slots alternating with it) then uses the epoch 2^31 | step << 8 | idx.
 *   qfb_linear_forward_reduce_step / qfb_linear_silu_mul_forward_reduce_step: the sending GEMV;
 *   qfb_linear_collect_addnorm_forward: qfb_linear_addnorm_forward whose addend is the sum over the ranks
 *     of slot `slot` (own partial + the peers' words, polled while the activations are staged; bounded
 *     waits, qfb_comm_read_status): y = (rmsnorm(x + sum) * norm_weight) . dequant(W)^T, x + sum -> x_out;
 *   qfb_allreduce_add_rmsnorm_step: the collecting reduction kernel for the places where no GEMV follows.
 * Do not mix the two numberings on one slot inside a step.  qfb_linear_addnorm_supported: 1 when the
 * fused-norm GEMV serves the layer for m rows (4-bit fragment layout, a plan without workspace reduction).
 */
int qfb_comm_step_begin(qfb_comm* comm, void* stream);
int qfb_linear_forward_reduce_step(const qfb_layer* layer, const void* x, int m, qfb_comm* comm, int slot, int idx,
                                   void* workspace, size_t workspace_bytes, unsigned flags, void* stream);
int qfb_linear_silu_mul_forward_reduce_step(const qfb_layer* layer, const void* gate_up, int m, qfb_comm* comm, int slot,
                                            int idx, void* workspace, size_t workspace_bytes, unsigned flags,
                                            void* stream);
int qfb_linear_collect_addnorm_forward(const qfb_layer* layer, qfb_comm* comm, int slot, int idx, const void* x,
                                       void* x_out, const void* norm_weight, float eps, int m, void* y,
                                       void* workspace, size_t workspace_bytes, unsigned flags, void* stream);
int qfb_allreduce_add_rmsnorm_step(qfb_comm* comm, int slot, int idx, void* x, const void* w, void* out, int rows,
                                   int d, float eps, void* stream);
int qfb_linear_addnorm_supported(const qfb_layer* layer, int m);
int qfb_comm_read_status(qfb_comm* comm, void* stream, unsigned* status_out);
int qfb_comm_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif /* QFACTORY_B200_H_ */
