// C-ABI entry points (see include/qfactory_b200.h): argument validation, kernel choice,
// split-K heuristics and launches.  No entry point here allocates device memory.
#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "qfb_common.cuh"
#include "qfb_kernels.h"

namespace qfb {

constexpr int kDefaultSMs = 148;  // B200; used when no device can be asked (size queries on a machine without a GPU)
// multiprocessors of the current device (asked once per device)
static int num_sms() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return kDefaultSMs;
  }
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = kDefaultSMs;
    }
    cached[dev] = n;
  }
  return cached[dev];
}
constexpr size_t kCounterAlign = 256;
constexpr int kMaxSimtRows = 8;  // activation rows one SIMT launch handles
constexpr int kMaxMmaRows = 16;  // activation rows one mma.sync GEMV launch handles
// ... except on 3-bit layers, whose only build has one 8-column batch tile (96 bits per lane and k-step leave
// no registers for a second one): 9..16 rows take two launches
static int mma_pass_rows(int bits) { return bits == 3 ? 8 : kMaxMmaRows; }

static thread_local int tl_last_cuda_error = 0;
static thread_local int tl_last_launch[5] = {0, 0, 0, 0, 0};
static int g_tune_split = 0, g_tune_kways = 0;
static int g_tc_min_m = 2;  // smallest batch routed to the tensor-core kernel
static int g_tc_split = 0;  // tuning override of the tensor-core split-K factor (0 = built-in)
static int g_tc_dg = 0;     // tuning override of the tensor-core kernel's decode groups (0 = built-in)
static int g_tc_nb = 0;     // tuning override of the tensor-core kernel's batch tile above 64 rows (0 = built-in)
static int g_mma_cluster = 1;  // mma.sync GEMV: reduce up to 8 K splits inside a thread-block cluster

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return QFB_OK;
  tl_last_cuda_error = (int)e;
  return QFB_ERR_CUDA;
}

static bool valid_bits(int bits) { return bits == 2 || bits == 3 || bits == 4 || bits == 8; }

static int validate_shape(int n, int k, int bits, int group_size) {
  if (!valid_bits(bits)) return QFB_ERR_UNSUPPORTED;
  if (n <= 0 || k <= 0) return QFB_ERR_BAD_SHAPE;
  if (k % 64 != 0 || k % unit_k(bits) != 0) return QFB_ERR_BAD_SHAPE;
  if (group_size != -1) {
    if (group_size <= 0 || group_size % 64 != 0 || k % group_size != 0 || group_size % unit_k(bits) != 0)
      return QFB_ERR_BAD_SHAPE;
  }
  return QFB_OK;
}

static int validate_layout(int layout, int k, int bits, int group_size) {
  if (layout == QFB_LAYOUT_TILE) return QFB_OK;
  if (layout != QFB_LAYOUT_FRAGMENT) return QFB_ERR_UNSUPPORTED;
  if (bits != 4 && bits != 8 && bits != 2 && bits != 3) return QFB_ERR_UNSUPPORTED;
  if (group_size != -1 && group_size != 64 && group_size % 128 != 0) return QFB_ERR_BAD_SHAPE;
  if (bits == 3 && group_size == 64) return QFB_ERR_BAD_SHAPE;   // (3-bit groups are multiples of 128 in both layouts)
  return k % 128 == 0 ? QFB_OK : QFB_ERR_BAD_SHAPE;
}

static int make_view(const qfb_layer* L, LayerView* v) {
  if (!L || !L->qweight) return QFB_ERR_NULL_POINTER;
  int st = validate_shape(L->n, L->k, L->bits, L->group_size);
  if (st != QFB_OK) return st;
  st = validate_layout(L->layout, L->k, L->bits, L->group_size);
  if (st != QFB_OK) return st;
  v->layout = L->layout;
  if (L->group_size == -1 && (L->scales || L->zeros)) return QFB_ERR_BAD_SHAPE;
  if (L->group_size != -1 && !L->scales) return QFB_ERR_NULL_POINTER;
  if (!aligned16(L->qweight) || !aligned16(L->scales) || !aligned16(L->zeros)) return QFB_ERR_MISALIGNED;
  v->qw = static_cast<const uint4*>(L->qweight);
  v->qs = static_cast<const __half*>(L->scales);
  v->qz = static_cast<const uint8_t*>(L->zeros);
  v->n = L->n;
  v->k = L->k;
  v->bits = L->bits;
  v->group_size = L->group_size;
  v->npad = padded_rows(L->n);
  v->tiles = v->npad / kTileRows;
  v->units = L->k / unit_k(L->bits);
  v->groups = L->group_size == -1 ? 1 : L->k / L->group_size;
  v->units_per_group = v->units / v->groups;
  // symmetric layers subtract 2^(bits-1); group-less layers use the raw codes
  v->zconst = (L->group_size == -1) ? 0u : (1u << (L->bits - 1));
  return QFB_OK;
}

// Upper bound of the split-K factor for a shape; sizes the workspace.
static int split_cap(int tiles, int units) {
  int cap = (num_sms() * 16 + tiles - 1) / tiles;
  return std::max(1, std::min(cap, units));
}

// Workspace layout: [0, 256) status words (word 0: a kernel's bounded wait ran out);
// [256, 256 + counters) arrival counters; then the fp32 split-K partial sums.
constexpr size_t kHeaderBytes = 256;
static size_t counters_bytes(int tiles) {
  const size_t n = (size_t)std::max(tiles, 2048);
  return (n * sizeof(unsigned) + kCounterAlign - 1) / kCounterAlign * kCounterAlign;
}
static size_t partial_offset(int tiles) { return kHeaderBytes + counters_bytes(tiles); }

// ---- tensor-core path planning --------------------------------------------------------
struct TcPlan { int nb, mtiles, split, dg; bool post; int tail_split, full_units, tail_units; };

static bool tc_supported(const LayerView& v) { return v.k % 128 == 0; }

static TcPlan plan_tc(const LayerView& v, int m) {
  TcPlan pl;
  pl.split = 1;
  pl.tail_split = 0;
  pl.full_units = pl.tail_units = 0;
  // per-stage accumulators need quantisation groups made of whole 128-k stages
  const bool post_ok = v.group_size == -1 || v.group_size % 128 == 0;
  pl.dg = 1;
  if (m <= 64) {
    // HBM-bound regime: split K until the SMs are covered
    pl.post = post_ok && m <= 32;
    pl.nb = !pl.post ? 64 : m <= 16 ? 16 : 32;
    pl.mtiles = 1;
    const int kblocks = v.k / 128;
    const int target = num_sms() * ((pl.post && pl.nb <= 32 && pl.dg == 1) ? 2 : 1);
    int split = std::max(1, target / v.tiles);
    split = std::min(split, std::max(1, kblocks / 4));
    split = std::min(split, 32);
    // measured: the wider the batch tile, the dearer a split (partials, reduce, per-CTA fill);
    // beyond 8 rows it only pays while the tiles alone leave most SMs idle or K is very long
    if (pl.nb == 16 && m > 8 && v.tiles >= 90) split = 1;
    if (pl.nb == 32) {  // two CTAs per SM: few tiles want a power-of-two split, many tiles none (measured)
      if (v.tiles >= 90) split = 1;
      else while (split & (split - 1)) split &= split - 1;
    }
    if (pl.nb == 64 && kblocks < 160) split = 1;
    if (g_tc_split > 0) split = std::min(g_tc_split, std::max(1, kblocks));
    if (v.tiles > 512) split = 1;  // the counter array holds 512 tiles x 4 row quarters
    pl.split = split;
  } else {
    // tensor-bound regime: scale in the decode, one accumulator over all of K;
    // pick the widest batch tile that still yields at least one CTA per SM
    pl.post = false;
    pl.nb = 64;
    for (int nb : {256, 128}) {
      if (m >= nb && (long long)v.tiles * ((m + nb - 1) / nb) >= num_sms()) { pl.nb = nb; break; }
    }
    if (pl.nb == 64 && (long long)v.tiles * ((m + 127) / 128) >= num_sms() / 2) pl.nb = 128;
    if (g_tc_nb == 64 || g_tc_nb == 128 || g_tc_nb == 256) pl.nb = g_tc_nb;
    pl.mtiles = (m + pl.nb - 1) / pl.nb;
    const int kblocks = v.k / 128;
    if (g_tc_split > 1) {  // tuning override: every unit is cut
      pl.tail_split = std::min(g_tc_split, 4);
    } else if (g_tc_split == 0 && g_tc_nb == 0 && m >= 96 && m <= 512 && kblocks >= 64) {
      // Few row tiles (N small against the SM count): narrow batch tiles would decode every weight
      // tile once per batch tile.  Better (measured: (8192,28672) at 128 rows 123 -> 78 us): the
      // widest tile the batch fills, every unit cut into 2..4 K ranges of one CTA each, fp32
      // partials summed in range order by the last CTA to arrive.
      const int nbw = m > 128 ? 256 : 128;
      const int units = v.tiles * ((m + nbw - 1) / nbw);
      const int s = std::min(std::min(4, kblocks / 16), num_sms() / std::max(1, units));
      if (nbw > pl.nb && s >= 2) {
        pl.nb = nbw;
        pl.mtiles = (m + nbw - 1) / nbw;
        pl.tail_split = s;
      }
    }
    if (pl.tail_split > 1) {
      pl.full_units = 0;
      pl.tail_units = v.tiles * pl.mtiles;
    }
  }
  // scale-in-the-decode mode: two decode groups on alternate stages in one CTA per SM (the latency
  // of one stage's decode, not its throughput, bounds the pipeline there: measured +10-15 % at
  // 128..512 rows), or, for batch tiles up to 128 columns on layers with more row tiles than SMs, one
  // decode group and two CTAs per SM (two independent pipelines: measured +5-12 % at 64..128 rows)
  if (!pl.post) {
    const bool two_per_sm = pl.nb <= 128 && pl.tail_split <= 1 && (long long)v.tiles * pl.mtiles >= num_sms() * 6 / 5 &&
                            m <= 128;
    pl.dg = g_tc_dg > 0 ? std::min(g_tc_dg, 2) : (two_per_sm ? 1 : 2);
  }
  return pl;
}

static size_t tc_tail_partial_bytes(const TcPlan& pl) {
  return (size_t)pl.tail_split * pl.tail_units * pl.nb * kTileRows * sizeof(float);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  }
  return fn;
}

static int run_tc(const LayerView& v, const __half* x, int m, __half* y, void* workspace, size_t ws_bytes,
                  unsigned flags, cudaStream_t st) {
  const TcPlan pl = plan_tc(v, m);
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return QFB_ERR_UNSUPPORTED;
  CUtensorMap tm;
  const cuuint64_t gdim[2] = {(cuuint64_t)v.k, (cuuint64_t)m};
  const cuuint64_t gstr[1] = {(cuuint64_t)v.k * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)pl.nb};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), gdim, gstr, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return QFB_ERR_CUDA;
  TcParams p = {};
  p.qw = v.qw;
  p.qs = v.qs;
  p.qz = v.qz;
  p.y = y;
  p.m = m;
  p.n = v.n;
  p.k = v.k;
  p.npad = v.npad;
  p.groups = v.groups;
  p.kblocks = v.k / 128;
  const int gs = v.group_size == -1 ? v.k : v.group_size;
  p.steps_per_group = gs / 16;
  p.halfstages_per_group = gs / 64;
  p.zconst = v.zconst;
  p.layout = v.layout;
  p.partial = nullptr;
  p.counters = nullptr;
  p.status = nullptr;
  if (workspace && ws_bytes >= kHeaderBytes) p.status = static_cast<unsigned*>(workspace);
  p.tail_split = 0;
  p.full_units = p.tail_units = 0;
  p.mtiles = pl.mtiles;
  p.stall_test = (flags & QFB_FLAG_TEST_STALLED_WAIT) ? 1 : 0;
  if (pl.split > 1) {
    const size_t off = partial_offset(v.tiles);
    const size_t need = off + (size_t)pl.split * m * v.npad * sizeof(float);
    if (!workspace || ws_bytes < need) return QFB_ERR_WORKSPACE;
    p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kHeaderBytes);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + off);
  }
  dim3 grid(v.tiles, pl.mtiles, pl.split);
  if (pl.tail_split > 1) {
    // the tail split is an optimisation: a workspace too small for its partial sums means the
    // plain grid, not an error (the counters of tail units sit in the first 2048 slots)
    const size_t off = partial_offset(v.tiles);
    const size_t need = off + tc_tail_partial_bytes(pl);
    if (workspace && ws_bytes >= need && pl.tail_units * 4 <= 2048) {
      p.tail_split = pl.tail_split;
      p.full_units = pl.full_units;
      p.tail_units = pl.tail_units;
      p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kHeaderBytes);
      p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + off);
      grid = dim3(pl.full_units + pl.tail_units * pl.tail_split, 1, 1);
    }
  }
  tl_last_launch[0] = 2;
  tl_last_launch[1] = grid.x * grid.y;
  tl_last_launch[2] = p.tail_split > 1 ? p.tail_split : grid.z;
  tl_last_launch[3] = 256 + 256 * pl.dg;
  tl_last_launch[4] = pl.nb;
  return check_cuda(launch_gemm_tc(tm, p, v.bits, pl.nb, pl.post, pl.dg, grid, (flags & QFB_FLAG_PDL) != 0, st));
}

static int choose_kernel(const LayerView& v, int m, unsigned flags) {
  if (flags & QFB_FLAG_FORCE_SIMT) return 1;
  if (!tc_supported(v)) return 1;
  if (flags & QFB_FLAG_FORCE_TENSOR) return 2;
  if (m >= g_tc_min_m) return 2;
  // a single activation row: the CUDA-core kernel wins while the packed weight is small
  // (measured cross-over near 64 MB); above that the tensor-core pipeline is ahead
  const double wbytes = (double)v.npad * v.k * v.bits / 8.0;
  return wbytes >= 64.0 * 1024 * 1024 ? 2 : 1;
}

struct GemvPlan { int split, kways, mb; size_t smem; };

static GemvPlan plan_gemv(const LayerView& v, int m_rows) {
  GemvPlan pl;
  pl.mb = m_rows <= 1 ? 1 : m_rows <= 2 ? 2 : m_rows <= 4 ? 4 : 8;
  const int uk = unit_k(v.bits);
  int kways = g_tune_kways > 0 ? g_tune_kways : 2;
  kways = std::max(1, std::min(kways, 2));  // the kernel is built for at most 256 threads
  // one register batch of units per thread: 8 vectors of 16 bytes in flight
  const int batch = v.bits == 3 ? 2 : v.bits == 2 ? 4 : 8;
  int split = g_tune_split > 0 ? g_tune_split : (v.units + batch * kways - 1) / (batch * kways);
  // keep the staged activation slice of a CTA below 96 KiB
  const size_t xrow_bytes = (size_t)v.k * 2;
  const int split_min = (int)((xrow_bytes * pl.mb + 96 * 1024 - 1) / (96 * 1024));
  split = std::max(split, split_min);
  split = std::max(1, std::min(split, split_cap(v.tiles, v.units)));
  while (kways > 1 && v.units / split < kways) --kways;
  pl.split = split;
  pl.kways = kways;
  const int max_units = (v.units + split - 1) / split;
  const size_t xbytes = (size_t)pl.mb * max_units * uk * 2;
  const size_t rbytes = (size_t)(kways - 1) * pl.mb * kTileRows * sizeof(float);
  pl.smem = std::max<size_t>(std::max(xbytes, rbytes), 16);
  return pl;
}

static int run_gemv(const LayerView& v, const __half* x, int m, __half* y, void* workspace, size_t ws_bytes,
                    unsigned flags, cudaStream_t st) {
  for (int m0 = 0; m0 < m; m0 += kMaxSimtRows) {
    const int rows = std::min(kMaxSimtRows, m - m0);
    const GemvPlan pl = plan_gemv(v, rows);
    GemvParams p = {};
    p.qw = v.qw;
    p.qs = v.qs;
    p.qz = v.qz;
    p.x = x + (size_t)m0 * v.k;
    p.y = y + (size_t)m0 * v.n;
    p.m = rows;
    p.n = v.n;
    p.k = v.k;
    p.npad = v.npad;
    p.units = v.units;
    p.groups = v.groups;
    p.units_per_group = v.units_per_group;
    p.max_units_per_cta = (v.units + pl.split - 1) / pl.split;
    p.units_per_kway = (p.max_units_per_cta + pl.kways - 1) / pl.kways;
    p.zconst = v.zconst;
    p.partial = nullptr;
    p.counters = nullptr;
    if (pl.split > 1) {
      const size_t off = partial_offset(v.tiles);
      const size_t need = off + (size_t)pl.split * rows * v.npad * sizeof(float);
      if (!workspace || ws_bytes < need) return QFB_ERR_WORKSPACE;
      p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kHeaderBytes);
      p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + off);
    }
    const dim3 grid(pl.split, v.tiles);
    const int block = kTileRows * pl.kways;
    tl_last_launch[0] = 1;
    tl_last_launch[1] = grid.x;
    tl_last_launch[2] = grid.y;
    tl_last_launch[3] = block;
    tl_last_launch[4] = (int)pl.smem;
    int stt = check_cuda(launch_gemv(p, v.bits, pl.mb, grid, block, pl.smem, (flags & QFB_FLAG_PDL) != 0, st));
    if (stt != QFB_OK) return stt;
  }
  return QFB_OK;
}

// ---- mma.sync GEMV over the fragment layout ---------------------------------------------
// warps of the mma.sync GEMV an SM holds: 16 at 128 registers per thread, 20 at 96 (CTAs of up to
// kMmaSmallBlock threads)
static int mma_warps_per_sm(int block) { return block <= kMmaSmallBlock ? 20 : 16; }
struct MmaPlan { int nt, split, kways, cluster, recv_offset; size_t smem; };

// most splits through the workspace (its size follows from this bound)
static int mma_split_cap(int tiles, int batches) {
  return std::max(1, std::min(batches, (num_sms() * 4 + tiles - 1) / tiles));
}
// most splits inside a cluster: enough CTAs of the smallest block to fill every slot of the device once
static int mma_cluster_split_cap(int tiles, int batches, int min_block) {
  const int slots = num_sms() * (mma_warps_per_sm(min_block) * 32 / min_block);
  return std::max(1, std::min(std::min(batches, 8), (slots + tiles - 1) / tiles));
}

// bytes of the staged activation slice and its per-segment sums; a second slice follows them when
// gate and up slices are combined while they are staged
static size_t mma_stage_bytes(int rows, int nt, int bpc) {
  return (size_t)rows * (bpc * 128 + 16) * 2 + (size_t)bpc * 2 * 8 * nt * sizeof(float);
}
static size_t mma_smem(int rows, int nt, int bpc, int kways, bool act = false) {
  const size_t stage = mma_stage_bytes(rows, nt, bpc) + (act ? (size_t)rows * (bpc * 128 + 16) * 2 : 0);
  const size_t red = (size_t)kways * rows * 132 * sizeof(float);  // k-way reduction lines
  return (std::max(stage, red) + 15) / 16 * 16;
}
// the receive buffer of the in-cluster split-K reduction follows the region above
static int mma_quads_per_owner(int rows, int split) { return (rows * 32 + split - 1) / split; }
static size_t mma_recv_bytes(int rows, int split) {
  return (size_t)split * mma_quads_per_owner(rows, split) * 4 * sizeof(float);
}

// Split-K factor, k-ways and reduction mode of the mma.sync GEMV.  Cost model fitted to sweeps
// on B200, in units of one 128-k batch of one warp (~0.25 us): the CTAs of a launch should be
// resident at once (a second wave costs a full CTA time); a CTA costs its longest k-way plus a
// fixed part worth ~1.5 batches; reducing the splits inside a thread-block cluster costs a small
// part that grows with rows x splits, reducing them through the workspace a fixed fence /
// atomic / re-read chain.  How many clusters fit at once is asked from the occupancy API (clusters must sit
// inside one GPC, so a grid that fits by CTA count may still need a second wave).
static MmaPlan plan_mma_search(int tiles, int k, int rows, bool seg64, int bits, bool act, bool no_ws) {
  MmaPlan pl;
  pl.nt = rows <= 8 ? 1 : 2;
  const int batches = k / 128;
  // warps per k-way: 2 x 64 rows (m <= 8; 2-, 3- and 4-bit) or 4 x 32 rows; at most 256 threads
  const int wpk = kTileRows / mma_rows_per_warp(bits, pl.nt);
  const int kways_max = 8 / wpk;
  const int cap_ws = mma_split_cap(tiles, batches);
  const int cap = std::max(cap_ws, g_mma_cluster ? mma_cluster_split_cap(tiles, batches, 32 * wpk) : 1);
  const size_t smem_max = 100 * 1024;
  int best_s = cap_ws, best_kw = 1, best_cl = 0;
  double best_cost = 1e30;
  for (int kw = kways_max; kw >= 1; kw >>= 1) {
    if (g_tune_kways > 0 && kw != std::min(g_tune_kways, kways_max)) continue;
    const int block = 32 * wpk * kw;
    for (int s = 1; s <= cap; ++s) {
      if (g_tune_split > 0 && s != std::min(g_tune_split, cap)) continue;
      const int bpc = (batches + s - 1) / s;
      const size_t smem = mma_smem(rows, pl.nt, bpc, kw, act);
      if (smem > smem_max && s < cap) continue;
      const int per_kway = (bpc + kw - 1) / kw;
      const double base = 0.05 * s + 0.01 * (kways_max - kw);
      // through the workspace: the registers (16 or 20 warps per SM) and the shared memory bound the residency
      if (s <= cap_ws && !(g_mma_cluster == 2 && s > 1 && s <= 8) && (!no_ws || s == 1)) {
        const int resident = std::max(1, std::min(mma_warps_per_sm(block) / (wpk * kw), (int)((200 * 1024) / (smem + 1024))));
        const int waves = (tiles * s + num_sms() * resident - 1) / (num_sms() * resident);
        const double cost = (double)waves * (per_kway + 1.5) + base + (s > 1 ? 3.0 + 0.02 * rows * s : 0.0);
        if (cost < best_cost) { best_cost = cost; best_s = s; best_kw = kw; best_cl = 0; }
      }
      if (s > 1 && s <= 8 && g_mma_cluster) {
        const int fit = mma_max_active_clusters(bits, pl.nt, seg64, block, smem + mma_recv_bytes(rows, s), s);
        if (fit > 0) {
          const int waves = (tiles + fit - 1) / fit;
          const double cost = (double)waves * (per_kway + 1.5) + base + 0.02 * rows * s;
          if (cost < best_cost) { best_cost = cost; best_s = s; best_kw = kw; best_cl = 1; }
        }
      }
    }
  }
  pl.split = best_s;
  pl.cluster = best_cl;
  const int bpc = (batches + best_s - 1) / best_s;
  // a power of two (the kernel splits a CTA's range among the k-ways with a shift), no more than the batches of a CTA
  pl.kways = best_kw;
  while (pl.kways > 1 && pl.kways > batches / best_s) pl.kways >>= 1;
  pl.smem = std::max<size_t>(mma_smem(rows, pl.nt, bpc, pl.kways, act), 16);
  pl.recv_offset = (int)pl.smem;
  if (pl.cluster) pl.smem += mma_recv_bytes(rows, pl.split);
  return pl;
}

// The search above asks the occupancy API and walks a few hundred candidates: its result is kept
// per (device, shape, rows, group mode, bit width, tuning overrides), so a repeated call costs a
// map lookup on the host.
// `no_ws`: only plans that reduce the K splits inside a cluster, or do not split (the fused norm needs them)
static MmaPlan plan_mma(int tiles, int k, int rows, bool seg64, int bits, bool act, bool no_ws = false) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, int, int, int, int, int, int, int>, MmaPlan> cache;
  int dev = 0;
  (void)cudaGetDevice(&dev);
  const auto key = std::make_tuple(dev, tiles, k, rows, (int)seg64 + 2 * (int)act + 4 * (int)no_ws, bits, g_tune_split, g_tune_kways,
                                   g_mma_cluster);
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  const MmaPlan pl = plan_mma_search(tiles, k, rows, seg64, bits, act, no_ws);
  std::lock_guard<std::mutex> lock(mu);
  cache[key] = pl;
  return pl;
}

// `act`: x is a fused gate/up tensor [m, 2k] and the layer's input is silu(gate) * up
// residual add + RMS norm fused in front of the linear (MmaParams::norm_*)
struct NormArgs {
  const __half* x;
  const __half* r;
  __half* out;
  const __half* w;
  float eps;
  const CollectSource* collect;   // non-null: the addend is collected from the peers (r unused)
};

static int run_mma(const LayerView& v, const __half* x, int m, __half* y, void* workspace, size_t ws_bytes,
                   unsigned flags, cudaStream_t st, bool act = false, const PushTarget* push = nullptr,
                   const NormArgs* norm = nullptr) {
  const int x_stride = act ? 2 * v.k : v.k;
  const int pass_rows = mma_pass_rows(v.bits);
  for (int m0 = 0; m0 < m; m0 += pass_rows) {
    const int rows = std::min(pass_rows, m - m0);
    const MmaPlan pl = plan_mma(v.tiles, v.k, rows, v.group_size == 64, v.bits, act, norm != nullptr);
    if (pl.smem > 200 * 1024) return QFB_ERR_TOO_LARGE;
    if (norm && pl.split > 1 && !pl.cluster) return QFB_ERR_UNSUPPORTED;   // (no cluster plan fits this device)
    MmaParams p = {};
    p.qw = v.qw;
    p.qs = v.qs;
    p.qz = v.qz;
    p.x = x + (size_t)m0 * x_stride;
    p.x_stride = x_stride;
    p.act = act ? 1 : 0;
    p.y = y + (size_t)m0 * v.n;
    p.m = rows;
    p.n = v.n;
    p.k = v.k;
    p.npad = v.npad;
    p.ksteps = v.k / 16;
    p.groups = v.groups;
    p.chunks_per_group = (v.group_size == -1 ? v.k : v.group_size) / 64;
    p.batches = v.k / 128;
    p.batches_per_cta = (p.batches + pl.split - 1) / pl.split;
    p.act_offset = (int)mma_stage_bytes(rows, pl.nt, p.batches_per_cta);
    p.stall_test = (flags & QFB_FLAG_TEST_STALLED_WAIT) ? 1 : 0;
    if (push) p.push = *push;   // (callers pass it for single-pass launches only)
    if (norm) {
      p.norm_x = norm->x;
      p.norm_r = norm->r;
      p.norm_out = norm->out;
      p.norm_w = norm->w;
      p.norm_eps = norm->eps;
      if (norm->collect) p.collect = *norm->collect;
    }
    p.batches_div = p.batches / pl.split;
    p.batches_mod = p.batches % pl.split;
    p.zconst = v.zconst;
    p.partial = nullptr;
    p.counters = nullptr;
    // up to 8 splits reduce inside a thread-block cluster; more go through the workspace
    p.cluster = pl.cluster;
    p.recv_offset = pl.recv_offset;
    p.quads_per_owner = mma_quads_per_owner(rows, pl.split);  // >= 4 (32 quads per row, at most 8 splits in a cluster)
    p.qper_magic = (uint32_t)(((1ull << 32) + p.quads_per_owner - 1) / p.quads_per_owner);
    p.status = (workspace && ws_bytes >= kHeaderBytes) ? static_cast<unsigned*>(workspace) : nullptr;
    if (pl.split > 1 && !p.cluster) {
      const size_t off = partial_offset(v.tiles);
      const size_t need = off + (size_t)pl.split * rows * v.npad * sizeof(float);
      if (!workspace || ws_bytes < need) return QFB_ERR_WORKSPACE;
      p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kHeaderBytes);
      p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + off);
    }
    const dim3 grid(pl.split, v.tiles);
    const int block = 32 * (kTileRows / mma_rows_per_warp(v.bits, pl.nt)) * pl.kways;
    tl_last_launch[0] = 3;
    tl_last_launch[1] = grid.x;
    tl_last_launch[2] = grid.y;
    tl_last_launch[3] = block;
    tl_last_launch[4] = (int)pl.smem;
    cudaError_t ce = launch_gemv_mma(p, v.bits, pl.nt, grid, block, pl.smem, (flags & QFB_FLAG_PDL) != 0, st);
    if (ce != cudaSuccess && p.cluster) {
      // a cluster launch the device refuses (e.g. a partitioned GPU): same split through the workspace
      (void)cudaGetLastError();
      const size_t off = partial_offset(v.tiles);
      const size_t need = off + (size_t)pl.split * rows * v.npad * sizeof(float);
      if (workspace && ws_bytes >= need) {
        p.cluster = 0;
        p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kHeaderBytes);
        p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + off);
        ce = launch_gemv_mma(p, v.bits, pl.nt, grid, block, pl.smem, (flags & QFB_FLAG_PDL) != 0, st);
      }
    }
    const int stt = check_cuda(ce);
    if (stt != QFB_OK) return stt;
  }
  return QFB_OK;
}

// Shared with the allocation-free entry point (qfb_static_scratch.cu): the argument checks of
// qfb_linear_forward without a launch, the recording of a CUDA error for qfb_last_cuda_error, and the
// bytes at the start of a scratch area that must be zero before a launch (status word + counters).
int validate_forward_args(const qfb_layer* layer, const void* x, int m, const void* y) {
  LayerView v;
  const int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  if (m < 0) return QFB_ERR_BAD_SHAPE;
  if (m > 0 && (!x || !y)) return QFB_ERR_NULL_POINTER;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 1u)) return QFB_ERR_MISALIGNED;
  return QFB_OK;
}
int record_cuda_error(cudaError_t e) {
  if (e != cudaSuccess) (void)cudaGetLastError();  // clear the runtime's pending error as well
  return check_cuda(e);
}
size_t scratch_clear_bytes(int n) { return partial_offset(padded_rows(n) / kTileRows); }

// Exact scratch need of the CUDA-core split-K kernel for `m` rows under the built-in plan
// (0 for invalid shapes); used by the allocation-free entry point.
size_t gemv_scratch_bytes(int m, int n, int k, int bits) {
  if (m <= 0 || validate_shape(n, k, bits, -1) != QFB_OK) return 0;
  LayerView v = {};
  v.n = n;
  v.k = k;
  v.bits = bits;
  v.npad = padded_rows(n);
  v.tiles = v.npad / kTileRows;
  v.units = k / unit_k(bits);
  const int rows = std::min(m, kMaxSimtRows);
  const GemvPlan pl = plan_gemv(v, rows);
  return partial_offset(v.tiles) + (size_t)pl.split * rows * v.npad * sizeof(float);
}

}  // namespace qfb

using namespace qfb;

extern "C" {

int qfb_version(void) { return 100; }

const char* qfb_status_string(int s) {
  switch (s) {
    case QFB_OK: return "ok";
    case QFB_ERR_NULL_POINTER: return "null pointer";
    case QFB_ERR_BAD_SHAPE: return "bad shape";
    case QFB_ERR_UNSUPPORTED: return "unsupported";
    case QFB_ERR_MISALIGNED: return "misaligned pointer";
    case QFB_ERR_WORKSPACE: return "workspace missing or too small";
    case QFB_ERR_CUDA: return "cuda runtime error";
    case QFB_ERR_TOO_LARGE: return "request too large";
    case QFB_ERR_DEVICE_FLAG: return "device-side bounded wait ran out";
    default: return "unknown status";
  }
}

int qfb_last_cuda_error(void) { return tl_last_cuda_error; }

size_t qfb_packed_weight_bytes(int n, int k, int bits) {
  if (validate_shape(n, k, bits, -1) != QFB_OK) return 0;
  return (size_t)padded_rows(n) * (k / unit_k(bits)) * unit_vecs(bits) * 16;
}

size_t qfb_packed_scale_bytes(int n, int k, int group_size) {
  if (n <= 0 || k <= 0 || group_size <= 0 || k % group_size) return 0;
  return (size_t)padded_rows(n) * (k / group_size) * 2;
}

size_t qfb_packed_zero_bytes(int n, int k, int group_size) {
  if (n <= 0 || k <= 0 || group_size <= 0 || k % group_size) return 0;
  return (size_t)padded_rows(n) * (k / group_size);
}

size_t qfb_workspace_bytes(int m_max, int n, int k, int bits) {
  if (m_max <= 0 || validate_shape(n, k, bits, -1) != QFB_OK) return 0;
  const int npad = padded_rows(n);
  const int tiles = npad / kTileRows;
  const int rows = std::min(m_max, kMaxSimtRows);
  size_t partial = (size_t)split_cap(tiles, k / unit_k(bits)) * rows * npad * sizeof(float);
  if (k % 128 == 0) {
    LayerView v = {};
    v.n = n; v.k = k; v.bits = bits; v.npad = npad; v.tiles = tiles;
    const int probes[] = {16, 32, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 4096, m_max};
    for (int gs : {64, 128}) {  // the group size selects between the two accumulation modes
      v.group_size = gs;
      for (int m : probes) {
        if (m > m_max) continue;
        const TcPlan pl = plan_tc(v, m);
        if (pl.split > 1) partial = std::max(partial, (size_t)pl.split * m * npad * sizeof(float));
        if (pl.tail_split > 1) partial = std::max(partial, tc_tail_partial_bytes(pl));
      }
    }
  }
  if (k % 128 == 0) {  // fragment-layout layers: the mma.sync GEMV's split bound
    const size_t rows_mma = (size_t)std::min(m_max, kMaxMmaRows);
    partial = std::max(partial, (size_t)mma_split_cap(tiles, k / 128) * rows_mma * npad * sizeof(float));
  }
  return partial_offset(tiles) + partial;
}

int qfb_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return QFB_ERR_NULL_POINTER;
  if (!aligned16(workspace)) return QFB_ERR_MISALIGNED;
  const size_t nb = std::min(workspace_bytes, (size_t)1 << 20);
  return check_cuda(cudaMemsetAsync(workspace, 0, nb, static_cast<cudaStream_t>(stream)));
}

int qfb_select_kernel(int m, int n, int k, int bits, unsigned flags) {
  if (m <= 0 || validate_shape(n, k, bits, -1) != QFB_OK) return 0;
  LayerView v = {};
  v.bits = bits;
  v.k = k;
  v.npad = padded_rows(n);
  return choose_kernel(v, m, flags);
}

void qfb_set_tensor_min_batch(int min_m) { g_tc_min_m = min_m > 0 ? min_m : 2; }

int qfb_read_status(const void* workspace, void* stream, unsigned* status_out) {
  if (!workspace || !status_out) return QFB_ERR_NULL_POINTER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int s = check_cuda(cudaMemcpyAsync(status_out, workspace, sizeof(unsigned), cudaMemcpyDeviceToHost, st));
  if (s != QFB_OK) return s;
  s = check_cuda(cudaStreamSynchronize(st));
  if (s != QFB_OK) return s;
  return *status_out ? QFB_ERR_DEVICE_FLAG : QFB_OK;
}

void qfb_set_gemv_tuning(int split_k, int k_ways) {
  g_tune_split = split_k;
  g_tune_kways = k_ways;
}

void qfb_set_tensor_split(int split_k) { g_tc_split = split_k > 0 ? split_k : 0; }
void qfb_set_tensor_decode_groups(int groups) { g_tc_dg = groups > 0 ? groups : 0; }
void qfb_set_tensor_batch_tile(int columns) { g_tc_nb = columns > 0 ? columns : 0; }

void qfb_set_cluster_reduce(int mode) { g_mma_cluster = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }

void qfb_get_last_launch(int* kernel, int* grid_x, int* grid_y, int* block, int* smem_bytes) {
  if (kernel) *kernel = tl_last_launch[0];
  if (grid_x) *grid_x = tl_last_launch[1];
  if (grid_y) *grid_y = tl_last_launch[2];
  if (block) *block = tl_last_launch[3];
  if (smem_bytes) *smem_bytes = tl_last_launch[4];
}

int qfb_linear_forward(const qfb_layer* layer, const void* x, int m, void* y, void* workspace,
                       size_t workspace_bytes, unsigned flags, void* stream) {
  LayerView v;
  int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  if (m < 0) return QFB_ERR_BAD_SHAPE;
  if (m == 0) return QFB_OK;
  if (!x || !y) return QFB_ERR_NULL_POINTER;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 1u) || !aligned16(workspace)) return QFB_ERR_MISALIGNED;
  // fragment-layout layers: the mma.sync GEMV up to 16 rows, the tcgen05 kernel (which reads the
  // same fragment words) above
  if (v.layout == QFB_LAYOUT_FRAGMENT && (m <= kMaxMmaRows || (flags & QFB_FLAG_FORCE_SIMT)))
    return run_mma(v, static_cast<const __half*>(x), m, static_cast<__half*>(y), workspace, workspace_bytes, flags,
                   static_cast<cudaStream_t>(stream));
  if (v.layout == QFB_LAYOUT_FRAGMENT || choose_kernel(v, m, flags) == 2)
    return run_tc(v, static_cast<const __half*>(x), m, static_cast<__half*>(y), workspace, workspace_bytes, flags,
                  static_cast<cudaStream_t>(stream));
  return run_gemv(v, static_cast<const __half*>(x), m, static_cast<__half*>(y), workspace, workspace_bytes, flags,
                  static_cast<cudaStream_t>(stream));
}

int qfb_linear_silu_mul_forward(const qfb_layer* layer, const void* gate_up, int m, void* y, void* workspace,
                                size_t workspace_bytes, unsigned flags, void* stream) {
  LayerView v;
  int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  if (m < 0) return QFB_ERR_BAD_SHAPE;
  if (m == 0) return QFB_OK;
  if (!gate_up || !y) return QFB_ERR_NULL_POINTER;
  if (!aligned16(gate_up) || (reinterpret_cast<uintptr_t>(y) & 1u) || !aligned16(workspace)) return QFB_ERR_MISALIGNED;
  // served by the mma.sync GEMV only, whose activation staging does the combination
  if (v.layout != QFB_LAYOUT_FRAGMENT || m > mma_pass_rows(v.bits)) return QFB_ERR_UNSUPPORTED;
  return run_mma(v, static_cast<const __half*>(gate_up), m, static_cast<__half*>(y), workspace, workspace_bytes, flags,
                 static_cast<cudaStream_t>(stream), true);
}

// The row-parallel linears of a tensor-parallel decoder: the partial goes into the communicator's data slot
// AND, in the wire format of the reduction, into this rank's receive region of every peer.
static int forward_reduce(const qfb_layer* layer, const void* x, int m, qfb_comm* comm, int slot, int idx, void* workspace,
                          size_t workspace_bytes, unsigned flags, void* stream, bool act) {
  LayerView v;
  int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  if (!comm || !x) return QFB_ERR_NULL_POINTER;
  if (m <= 0) return m == 0 ? QFB_OK : QFB_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(workspace)) return QFB_ERR_MISALIGNED;
  // served by the mma.sync GEMV in one pass, on layers whose output rows are whole aligned quads
  if (v.layout != QFB_LAYOUT_FRAGMENT || m > kMaxMmaRows || v.n % 128 != 0) return QFB_ERR_UNSUPPORTED;
  if (v.bits != 4 || v.group_size == 64) return QFB_ERR_UNSUPPORTED;   // (the sending build exists for these only)
  PushTarget t;
  void* own = nullptr;
  st = comm_push_target(comm, slot, m, v.n, &t, &own);
  if (st != QFB_OK) return st;
  if (idx > 255) return QFB_ERR_BAD_SHAPE;
  t.idx = idx;   // (< 0: per-row epochs, advanced by the reduction kernel)
  return run_mma(v, static_cast<const __half*>(x), m, static_cast<__half*>(own), workspace, workspace_bytes, flags,
                 static_cast<cudaStream_t>(stream), act, &t);
}

int qfb_linear_addnorm_forward(const qfb_layer* layer, const void* x, const void* residual, void* x_out,
                               const void* norm_weight, float eps, int m, void* y, void* workspace,
                               size_t workspace_bytes, unsigned flags, void* stream) {
  LayerView v;
  int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  if (m < 0) return QFB_ERR_BAD_SHAPE;
  if (m == 0) return QFB_OK;
  if (!x || !norm_weight || !y) return QFB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(residual) || !aligned16(x_out) || !aligned16(norm_weight) || !aligned16(workspace) ||
      (reinterpret_cast<uintptr_t>(y) & 1u))
    return QFB_ERR_MISALIGNED;
  if (x_out && (x_out == x || x_out == residual)) return QFB_ERR_BAD_SHAPE;   // other CTAs still read the inputs
  // served by one launch of the mma.sync GEMV's norm build (4-bit, groups of 128 and more)
  if (v.layout != QFB_LAYOUT_FRAGMENT || m > kMaxMmaRows || v.bits != 4 || v.group_size == 64) return QFB_ERR_UNSUPPORTED;
  const NormArgs na = {static_cast<const __half*>(x), static_cast<const __half*>(residual), static_cast<__half*>(x_out),
                       static_cast<const __half*>(norm_weight), eps, nullptr};
  return run_mma(v, static_cast<const __half*>(x), m, static_cast<__half*>(y), workspace, workspace_bytes, flags,
                 static_cast<cudaStream_t>(stream), false, nullptr, &na);
}

int qfb_linear_addnorm_supported(const qfb_layer* layer, int m) {
  LayerView v;
  if (make_view(layer, &v) != QFB_OK || m <= 0) return 0;
  if (v.layout != QFB_LAYOUT_FRAGMENT || m > kMaxMmaRows || v.bits != 4 || v.group_size == 64) return 0;
  const MmaPlan pl = plan_mma(v.tiles, v.k, m, false, v.bits, false, true);
  return (pl.smem <= 200 * 1024 && (pl.split == 1 || pl.cluster)) ? 1 : 0;
}

int qfb_linear_collect_addnorm_forward(const qfb_layer* layer, qfb_comm* comm, int slot, int idx, const void* x,
                                       void* x_out, const void* norm_weight, float eps, int m, void* y,
                                       void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
  LayerView v;
  int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  if (m < 0) return QFB_ERR_BAD_SHAPE;
  if (m == 0) return QFB_OK;
  if (!comm || !x || !norm_weight || !y) return QFB_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(x_out) || !aligned16(norm_weight) || !aligned16(workspace) ||
      (reinterpret_cast<uintptr_t>(y) & 1u))
    return QFB_ERR_MISALIGNED;
  if (x_out && x_out == x) return QFB_ERR_BAD_SHAPE;
  if (v.layout != QFB_LAYOUT_FRAGMENT || m > kMaxMmaRows || v.bits != 4 || v.group_size == 64) return QFB_ERR_UNSUPPORTED;
  CollectSource cs;
  st = comm_collect_source(comm, slot, idx, m, v.k, &cs);
  if (st != QFB_OK) return st;
  const NormArgs na = {static_cast<const __half*>(x), nullptr, static_cast<__half*>(x_out),
                       static_cast<const __half*>(norm_weight), eps, &cs};
  return run_mma(v, static_cast<const __half*>(x), m, static_cast<__half*>(y), workspace, workspace_bytes, flags,
                 static_cast<cudaStream_t>(stream), false, nullptr, &na);
}

int qfb_linear_forward_reduce(const qfb_layer* layer, const void* x, int m, qfb_comm* comm, int slot, void* workspace,
                              size_t workspace_bytes, unsigned flags, void* stream) {
  return forward_reduce(layer, x, m, comm, slot, -1, workspace, workspace_bytes, flags, stream, false);
}

int qfb_linear_forward_reduce_step(const qfb_layer* layer, const void* x, int m, qfb_comm* comm, int slot, int idx,
                                   void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
  if (idx < 0) return QFB_ERR_BAD_SHAPE;
  return forward_reduce(layer, x, m, comm, slot, idx, workspace, workspace_bytes, flags, stream, false);
}

int qfb_linear_silu_mul_forward_reduce_step(const qfb_layer* layer, const void* gate_up, int m, qfb_comm* comm, int slot,
                                            int idx, void* workspace, size_t workspace_bytes, unsigned flags,
                                            void* stream) {
  if (idx < 0) return QFB_ERR_BAD_SHAPE;
  return forward_reduce(layer, gate_up, m, comm, slot, idx, workspace, workspace_bytes, flags, stream, true);
}

int qfb_linear_silu_mul_forward_reduce(const qfb_layer* layer, const void* gate_up, int m, qfb_comm* comm, int slot,
                                       void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
  return forward_reduce(layer, gate_up, m, comm, slot, -1, workspace, workspace_bytes, flags, stream, true);
}

int qfb_linear_forward_host(const qfb_layer* layer, const void* x_host, int m, void* y_host, void* x_staging,
                            void* y_staging, void* workspace, size_t workspace_bytes, unsigned flags,
                            void* stream) {
  if (!layer || !x_host || !y_host || !x_staging || !y_staging) return QFB_ERR_NULL_POINTER;
  if (m <= 0) return m == 0 ? QFB_OK : QFB_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int s = check_cuda(cudaMemcpyAsync(x_staging, x_host, (size_t)m * layer->k * 2, cudaMemcpyHostToDevice, st));
  if (s != QFB_OK) return s;
  s = qfb_linear_forward(layer, x_staging, m, y_staging, workspace, workspace_bytes, flags, stream);
  if (s != QFB_OK) return s;
  s = check_cuda(cudaMemcpyAsync(y_host, y_staging, (size_t)m * layer->n * 2, cudaMemcpyDeviceToHost, st));
  if (s != QFB_OK) return s;
  if (flags & QFB_FLAG_NO_SYNC) return QFB_OK;
  return check_cuda(cudaStreamSynchronize(st));
}

int qfb_layout_supported(int layout, int n, int k, int bits, int group_size) {
  return validate_shape(n, k, bits, group_size) == QFB_OK && validate_layout(layout, k, bits, group_size) == QFB_OK;
}

int qfb_pack(const int32_t* codes, const void* scales, const int32_t* zeros, int n, int k, int bits,
             int group_size, void* qweight_out, void* scales_out, void* zeros_out, void* stream) {
  return qfb_pack_layout(codes, scales, zeros, n, k, bits, group_size, QFB_LAYOUT_TILE, qweight_out, scales_out,
                         zeros_out, stream);
}

int qfb_pack_layout(const int32_t* codes, const void* scales, const int32_t* zeros, int n, int k, int bits,
                    int group_size, int layout, void* qweight_out, void* scales_out, void* zeros_out,
                    void* stream) {
  int st = validate_shape(n, k, bits, group_size);
  if (st != QFB_OK) return st;
  st = validate_layout(layout, k, bits, group_size);
  if (st != QFB_OK) return st;
  if (!codes || !qweight_out) return QFB_ERR_NULL_POINTER;
  if (group_size != -1 && (!scales || !scales_out)) return QFB_ERR_NULL_POINTER;
  if (group_size == -1 && (scales || zeros)) return QFB_ERR_BAD_SHAPE;
  if (zeros && !zeros_out) return QFB_ERR_NULL_POINTER;
  if (!aligned16(qweight_out) || !aligned16(scales_out) || !aligned16(zeros_out)) return QFB_ERR_MISALIGNED;
  PackParams p;
  p.codes = codes;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = zeros;
  p.qw = static_cast<uint32_t*>(qweight_out);
  p.qs = group_size == -1 ? nullptr : static_cast<__half*>(scales_out);
  p.qz = zeros ? static_cast<uint8_t*>(zeros_out) : nullptr;
  p.n = n;
  p.k = k;
  p.bits = bits;
  p.group_size = group_size;
  p.npad = padded_rows(n);
  p.tiles = p.npad / kTileRows;
  p.units = k / unit_k(bits);
  p.groups = group_size == -1 ? 1 : k / group_size;
  p.layout = layout;
  return check_cuda(launch_pack(p, static_cast<cudaStream_t>(stream)));
}

int qfb_quantize(const void* weight, int k, int n, int bits, int group_size, int32_t* codes_out, void* scales_out,
                 int32_t* zeros_out, void* stream) {
  if (!weight || !codes_out || !scales_out || !zeros_out) return QFB_ERR_NULL_POINTER;
  if (!valid_bits(bits)) return QFB_ERR_UNSUPPORTED;
  if (k <= 0 || n <= 0 || group_size <= 0 || k % group_size != 0) return QFB_ERR_BAD_SHAPE;
  return check_cuda(launch_quantize(static_cast<const __half*>(weight), k, n, bits, group_size, codes_out,
                                    static_cast<__half*>(scales_out), zeros_out, static_cast<cudaStream_t>(stream)));
}

static int run_unpack(const qfb_layer* layer, int32_t* codes_out, void* w_out, void* stream) {
  LayerView v;
  int st = make_view(layer, &v);
  if (st != QFB_OK) return st;
  UnpackParams p;
  p.qw = v.qw;
  p.qs = v.qs;
  p.qz = v.qz;
  p.codes_out = codes_out;
  p.w_out = static_cast<__half*>(w_out);
  p.n = v.n;
  p.k = v.k;
  p.bits = v.bits;
  p.npad = v.npad;
  p.tiles = v.tiles;
  p.units = v.units;
  p.groups = v.groups;
  p.units_per_group = v.units_per_group;
  p.zconst = v.zconst;
  p.layout = v.layout;
  return check_cuda(launch_unpack(p, static_cast<cudaStream_t>(stream)));
}

int qfb_rope_cache(void* qkv, const void* cosv, const void* sinv, const void* pos, void* k_cache, void* v_cache,
                   int batch, int tokens, int q_heads, int kv_heads, int head_dim, int max_len, void* stream) {
  if (!qkv || !cosv || !sinv || !pos || !k_cache || !v_cache) return QFB_ERR_NULL_POINTER;
  if (batch < 0 || tokens < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim % 2 != 0 || max_len <= 0)
    return QFB_ERR_BAD_SHAPE;
  if (batch == 0 || tokens == 0) return QFB_OK;
  return check_cuda(launch_rope_cache(static_cast<__half*>(qkv), static_cast<const __half*>(cosv),
                                      static_cast<const __half*>(sinv), static_cast<const long long*>(pos),
                                      static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), batch, tokens,
                                      q_heads, kv_heads, head_dim, max_len, static_cast<cudaStream_t>(stream)));
}

int qfb_decode_attention(const void* qkv, const void* pos, const void* k_cache, const void* v_cache, void* out, int batch,
                         int q_heads, int kv_heads, int head_dim, int max_len, void* stream) {
  if (!qkv || !pos || !k_cache || !v_cache || !out) return QFB_ERR_NULL_POINTER;
  if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_len <= 0) return QFB_ERR_BAD_SHAPE;
  if (!decode_attention_supported(q_heads, kv_heads, head_dim, max_len)) return QFB_ERR_UNSUPPORTED;
  if (!aligned16(qkv) || !aligned16(k_cache) || !aligned16(v_cache) || (reinterpret_cast<uintptr_t>(out) & 1u))
    return QFB_ERR_MISALIGNED;
  if (batch == 0) return QFB_OK;
  return check_cuda(launch_decode_attention(static_cast<const __half*>(qkv),
                                            const_cast<__half*>(static_cast<const __half*>(k_cache)),
                                            const_cast<__half*>(static_cast<const __half*>(v_cache)),
                                            static_cast<const long long*>(pos), static_cast<__half*>(out), batch, q_heads,
                                            kv_heads, max_len, nullptr, nullptr, static_cast<cudaStream_t>(stream)));
}

int qfb_decode_attention_rope(const void* qkv, const void* cosv, const void* sinv, const void* pos, void* k_cache,
                              void* v_cache, void* out, int batch, int q_heads, int kv_heads, int head_dim, int max_len,
                              void* stream) {
  if (!qkv || !cosv || !sinv || !pos || !k_cache || !v_cache || !out) return QFB_ERR_NULL_POINTER;
  if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_len <= 0) return QFB_ERR_BAD_SHAPE;
  if (!decode_attention_supported(q_heads, kv_heads, head_dim, max_len)) return QFB_ERR_UNSUPPORTED;
  if (!aligned16(qkv) || !aligned16(k_cache) || !aligned16(v_cache) || (reinterpret_cast<uintptr_t>(out) & 1u) ||
      (reinterpret_cast<uintptr_t>(cosv) & 7u) || (reinterpret_cast<uintptr_t>(sinv) & 7u))
    return QFB_ERR_MISALIGNED;
  if (batch == 0) return QFB_OK;
  return check_cuda(launch_decode_attention(static_cast<const __half*>(qkv), static_cast<__half*>(k_cache),
                                            static_cast<__half*>(v_cache), static_cast<const long long*>(pos),
                                            static_cast<__half*>(out), batch, q_heads, kv_heads, max_len,
                                            static_cast<const __half*>(cosv), static_cast<const __half*>(sinv),
                                            static_cast<cudaStream_t>(stream)));
}

int qfb_rmsnorm(const void* x, const void* w, void* y, int rows, int d, float eps, void* stream) {
  if (!x || !w || !y) return QFB_ERR_NULL_POINTER;
  if (rows < 0 || d <= 0 || d % 8 != 0) return QFB_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return QFB_ERR_MISALIGNED;
  if (rows == 0) return QFB_OK;
  return check_cuda(launch_rmsnorm(const_cast<__half*>(static_cast<const __half*>(x)), nullptr,
                                   static_cast<const __half*>(w), static_cast<__half*>(y), rows, d, eps,
                                   static_cast<cudaStream_t>(stream)));
}

int qfb_add_rmsnorm(void* x, const void* residual, const void* w, void* y, int rows, int d, float eps, void* stream) {
  if (!x || !residual || !w || !y) return QFB_ERR_NULL_POINTER;
  if (rows < 0 || d <= 0 || d % 8 != 0) return QFB_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(residual) || !aligned16(w) || !aligned16(y)) return QFB_ERR_MISALIGNED;
  if (rows == 0) return QFB_OK;
  return check_cuda(launch_rmsnorm(static_cast<__half*>(x), static_cast<const __half*>(residual),
                                   static_cast<const __half*>(w), static_cast<__half*>(y), rows, d, eps,
                                   static_cast<cudaStream_t>(stream)));
}

int qfb_silu_mul(const void* gate_up, void* out, int rows, int half, void* stream) {
  if (!gate_up || !out) return QFB_ERR_NULL_POINTER;
  if (rows < 0 || half <= 0 || half % 8 != 0) return QFB_ERR_BAD_SHAPE;
  if (!aligned16(gate_up) || !aligned16(out)) return QFB_ERR_MISALIGNED;
  if (rows == 0) return QFB_OK;
  return check_cuda(launch_silu_mul(static_cast<const __half*>(gate_up), static_cast<__half*>(out), rows, half,
                                    static_cast<cudaStream_t>(stream)));
}

int qfb_unpack_codes(const qfb_layer* layer, int32_t* codes_out, void* stream) {
  if (!codes_out) return QFB_ERR_NULL_POINTER;
  return run_unpack(layer, codes_out, nullptr, stream);
}

int qfb_dequantize(const qfb_layer* layer, void* w_out, void* stream) {
  if (!w_out) return QFB_ERR_NULL_POINTER;
  return run_unpack(layer, nullptr, w_out, stream);
}

}  // extern "C"
