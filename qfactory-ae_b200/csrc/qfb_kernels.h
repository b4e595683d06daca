// Internal launch interfaces between the C-ABI layer and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qfb {

struct GemvParams {
  const uint4* qw;
  const __half* qs;      // null: scale 1 (group-less)
  const uint8_t* qz;     // null: zconst
  const __half* x;       // [m, k]
  __half* y;             // [m, n]
  float* partial;        // [S, m, npad] split-K partial sums
  unsigned* counters;    // [tiles] arrival counters, zero between launches
  int m, n, k, npad;
  int units;             // K / unit_k(bits)
  int groups;            // K / group_size (1 when group-less)
  int units_per_group;
  int max_units_per_cta; // ceil(units / S): unit stride between K splits
  int units_per_kway;    // ceil(max_units_per_cta / k-ways): unit stride between the k-ways of a CTA
  uint32_t zconst;
};

cudaError_t launch_gemv(const GemvParams& p, int bits, int mb, dim3 grid, int block, size_t smem, bool pdl,
                        cudaStream_t st);

// exact scratch bytes the split-K GEMV needs for m rows (0 when the shape is invalid)
size_t gemv_scratch_bytes(int m, int n, int k, int bits);
// helpers shared with the allocation-free entry point
int record_cuda_error(cudaError_t e);
size_t scratch_clear_bytes(int n);

// mma.sync split-K kernel over the fragment layout (m <= 16 per launch, 8 for 3-bit layers)
// Row-parallel linears of a tensor-parallel decoder: where the result is one rank's PARTIAL of a sum over
// the ranks, the kernel that stores it also sends it to the peers, in the wire format of the peer-memory
// reduction (qfb_comm.cu): every 4 data bytes followed by the call's epoch, stored into this rank's
// receive region of every peer's symmetric buffer.  world == 0: nothing is sent.
struct PushTarget {
  char* base[8];           // the ranks' symmetric buffers (entries >= world unused)
  int world, rank;
  size_t recv_offset;      // byte offset, inside every buffer, of this rank's receive region of the slot (row 0)
  const unsigned* epochs;  // local header: epoch of the last finished reduction per batch row
  // Step numbering (idx >= 0): the epoch is 2^31 | step << 8 | idx, with `step` a counter in the local header
  // that one small launch advances at the start of a decode step and nothing changes during it, and idx the
  // number of the reduction inside the step.  No kernel has to advance an epoch, so the receiving side can
  // be any kernel: the reduction kernel, or the GEMV that consumes the sum (CollectSource).
  const unsigned* step;
  int idx;
};
// The other half of that exchange inside a GEMV (norm build): the addend of the fused residual add is the sum
// over the ranks of a row-parallel linear's partials, collected from this rank's own buffer while the
// activations are staged: the own partial (plain fp16) and, per peer, the {data, epoch} words it sent.
struct CollectSource {
  const char* local;       // this rank's symmetric buffer (null: no collection; the addend is MmaParams::norm_r)
  size_t own_offset;       // the slot's own partial
  size_t recv_offset;      // the slot's receive region of source rank 0
  size_t region_bytes;     // bytes between the receive regions of consecutive source ranks
  int world, rank;
  const unsigned* step;    // local header: step counter
  unsigned idx;            // number of the reduction inside the step
  unsigned long long timeout_ns;   // bound of every wait; when it runs out `status` is set and the kernel goes on
  unsigned* status;
};
struct MmaParams {
  const uint4* qw;
  const __half* qs;      // null: scale 1 (group-less)
  const uint8_t* qz;     // null: zconst
  const __half* x;       // [m, k]
  __half* y;             // [m, n]
  float* partial;        // [S, m, npad] split-K partial sums
  unsigned* counters;    // [tiles] arrival counters, zero between launches
  int m, n, k, npad;
  int ksteps;            // K / 16
  int groups;            // K / group_size (1 when group-less)
  int chunks_per_group;  // group_size / 64 (K / 64 when group-less)
  int batches;           // K / 128
  int batches_per_cta;   // ceil(batches / S): sizes the staged activation slice
  int batches_div, batches_mod;  // batches / S and batches % S: split s owns batches_div (+1 if s < batches_mod)
  uint32_t zconst;
  int cluster;           // 1: the S splits of a tile are one thread-block cluster and reduce in shared memory
  int recv_offset;       // byte offset of the cluster reduction's receive buffer in dynamic shared memory
  int quads_per_owner;   // cluster reduction: ceil(m * 32 / S) quads (4 rows of one batch column) per CTA of the cluster
  uint32_t qper_magic;   // ceil(2^32 / quads_per_owner): q / quads_per_owner = umulhi(q, qper_magic) for q < 2^9
  unsigned* status;      // may be null; set to 1 when a bounded wait ran out
  int x_stride;          // halfs between activation rows (k, or 2k for a fused gate/up tensor)
  int act;               // 1: activations = silu(x[:, :k]) * x[:, k:2k], combined while they are staged
  int act_offset;        // byte offset of the up-slice staging region in dynamic shared memory (act only)
  int stall_test;        // 1 (QFB_FLAG_TEST_STALLED_WAIT): the activation barrier expects 16 bytes that never
                         // come and gives up after ~100 us, so that the bounded-wait path can be tested
  PushTarget push;       // row-parallel layer of a tensor-parallel decoder: y is also sent to the peers
  // fused residual add + RMS norm in front of the linear (norm_w != null; x is then unused): the activations
  // are rmsnorm(norm_x + norm_r) * norm_w.  The sum norm_x + norm_r is also written to norm_out (may be
  // null; never the same buffer as norm_x or norm_r: other CTAs still read those).
  const __half* norm_x;  // [m, k] residual stream
  const __half* norm_r;  // [m, k] addend, or null
  __half* norm_out;      // [m, k] updated residual stream, or null
  const __half* norm_w;  // [k] norm weight
  float norm_eps;
  CollectSource collect; // norm build: the addend comes from the peers (norm_r is then unused)
};
// CTAs of the mma.sync GEMV of up to this many threads run the 96-register build (five per SM)
constexpr int kMmaSmallBlock = 128;
// rows of a 128-row tile one warp of the mma.sync GEMV owns (64 or 32) for a bit width and number of batch tiles
int mma_rows_per_warp(int bits, int nt);
// clusters of `cluster` CTAs of the mma.sync GEMV the current device holds at once (cached)
int mma_max_active_clusters(int bits, int nt, bool seg64, int block, size_t smem, int cluster);
}  // namespace qfb
struct qfb_comm;
namespace qfb {
// Where a row-parallel GEMV that feeds data slot `slot` of a communicator must send its [rows, d] partial
// (`t`), and the local plain-fp16 copy it must write as its output (`own_slot`).  A status code.
int comm_push_target(const qfb_comm* c, int slot, int rows, int d, PushTarget* t, void** own_slot);
// Where a GEMV that consumes the sum of data slot `slot` finds the partials (reduction `idx` of the step).
int comm_collect_source(const qfb_comm* c, int slot, int idx, int rows, int d, CollectSource* s);
cudaError_t launch_gemv_mma(const MmaParams& p, int bits, int nt, dim3 grid, int block, size_t smem, bool pdl,
                            cudaStream_t st);

struct TcParams {
  const uint4* qw;
  const __half* qs;      // null: group-less (no scaling)
  const uint8_t* qz;     // null: zconst
  __half* y;             // [m, n]
  float* partial;        // [S, m, npad] split-K partial sums
  unsigned* counters;    // [m tiles, n tiles] arrival counters, zero between launches
  unsigned* status;      // set to 1 when a bounded wait ran out
  int m, n, k, npad;
  int groups;
  int kblocks;               // K / 128 pipeline stages
  int steps_per_group;       // group_size / 16 MMA k-steps per quantisation group (K / 16 when group-less)
  int halfstages_per_group;  // group_size / 64
  uint32_t zconst;
  int layout;                // QFB_LAYOUT_TILE or QFB_LAYOUT_FRAGMENT
  // tail-split launches (one-dimensional grid; 0 = the uniform grid (tiles, batch tiles, splits)):
  int tail_split;            // K ranges each unit of the last, partly filled wave is cut into
  int full_units;            // (row tile, batch tile) units that run whole, one CTA each
  int tail_units;            // units that are cut; partial = [tail_split][tail_units][batch tile][128] fp32
  int mtiles;                // batch tiles per row tile (unit = tile * mtiles + batch tile)
  int stall_test;            // 1 (QFB_FLAG_TEST_STALLED_WAIT): the first weight stage's barrier expects 16 bytes
                             // that never come; every wait gives up after ~100 us (bounded-wait path under test)
};
// activations [m, k] fp16 row-major as a 2-D tiled tensor map with boxes of {64, nb}, 128-byte swizzle
cudaError_t launch_gemm_tc(const CUtensorMap& tmap_x, const TcParams& p, int bits, int nb, bool post, int decode_groups,
                           dim3 grid, bool pdl, cudaStream_t st);

// element-wise neighbours of the linears in a decoder layer (qfb_decoder_ops.cu)
cudaError_t launch_rmsnorm(__half* x, const __half* res, const __half* w, __half* y, int rows, int d, float eps,
                           cudaStream_t st);
cudaError_t launch_silu_mul(const __half* gu, __half* out, int rows, int half, cudaStream_t st);
// single-query attention over the static cache (qfb_decode_attention.cu)
bool decode_attention_supported(int hq, int hkv, int hd, int max_len);
// cosv / sinv non-null: the queries and the new key are rotated here and the new key / value are written
// into the caches (the single-token work of launch_rope_cache, fused)
cudaError_t launch_decode_attention(const __half* qkv, __half* k_cache, __half* v_cache, const long long* pos,
                                    __half* out, int B, int hq, int hkv, int max_len, const __half* cosv, const __half* sinv,
                                    cudaStream_t st);
cudaError_t launch_rope_cache(__half* qkv, const __half* cosv, const __half* sinv, const long long* pos, __half* k_cache,
                              __half* v_cache, int B, int T, int hq, int hkv, int hd, int max_len, cudaStream_t st);

struct PackParams {
  const int32_t* codes;   // [k, n]
  const __half* scales;   // [groups, n] or null
  const int32_t* zeros;   // [groups, n] or null
  uint32_t* qw;           // packed words
  __half* qs;
  uint8_t* qz;
  int n, k, bits, group_size, npad, tiles, units, groups;
  int layout;             // QFB_LAYOUT_TILE or QFB_LAYOUT_FRAGMENT
};
cudaError_t launch_pack(const PackParams& p, cudaStream_t st);

cudaError_t launch_quantize(const __half* w, int k, int n, int bits, int group_size, int32_t* codes, __half* scales,
                            int32_t* zeros, cudaStream_t st);

struct UnpackParams {
  const uint4* qw;
  const __half* qs;
  const uint8_t* qz;
  int32_t* codes_out;   // [k, n] or null
  __half* w_out;        // [k, n] or null
  int n, k, bits, npad, tiles, units, groups, units_per_group;
  uint32_t zconst;
  int layout;
};
cudaError_t launch_unpack(const UnpackParams& p, cudaStream_t st);

}  // namespace qfb
