// Host side of the tcgen05 GEMM engine: tensor-map construction, tile-plan selection and the
// launchers that every fused-epilogue entry point shares.
#pragma once
#include <cudaTypedefs.h>
#include <mutex>
#include "common.cuh"
#include "gemm2_sm100.cuh"

namespace pomh {
using namespace pomk;

// ---------------------------------------------------------------- tensor maps
// cuTensorMapEncodeTiled is fetched through the runtime so the library has no
// link-time dependency on the driver (it must load on machines without one).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor of `rank` <= 4 dims (innermost first), zero fill out of bounds.  elem_bytes 2 = bf16, 4 = fp32.
inline int make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_elems,
             const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, int elem_bytes = 2) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return POM_ERR_CUDA;
  if (!aligned16(base)) return POM_ERR_BAD_ALIGN;
  if (rank < 2 || rank > 4) return POM_ERR_BAD_SHAPE;
  cuuint64_t gdim[4];
  cuuint64_t gstr[3];
  cuuint32_t bx[4];
  cuuint32_t es[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    if (dims[i] == 0) return POM_ERR_BAD_SHAPE;
    gdim[i] = dims[i];
    bx[i] = box[i];
    if (box[i] == 0 || box[i] > 256) return POM_ERR_BAD_SHAPE;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    uint64_t bytes = strides_elems[i] * static_cast<uint64_t>(elem_bytes);
    if (bytes % 16 != 0) return POM_ERR_BAD_STRIDE;
    if (bytes >= (1ull << 40)) return POM_ERR_TOO_LARGE;
    gstr[i] = bytes;
  }
  CUresult r = fn(m, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? POM_OK : POM_ERR_CUDA;
}

// Epilogue tensor: bf16 (batches, rows, cols) with row stride ld, moved in 32 x 32 blocks (64-byte swizzle).
// batch_stride (elements) 0 = rows * ld.
inline int make_io_map(CUtensorMap* m, const void* base, int64_t cols, int64_t rows, int64_t batches, int64_t ld,
                int64_t batch_stride = 0) {
  if (ld % 8 || ld < cols) return POM_ERR_BAD_STRIDE;
  uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(batches)};
  uint64_t str[2] = {static_cast<uint64_t>(ld),
                     batch_stride ? static_cast<uint64_t>(batch_stride)
                                  : static_cast<uint64_t>(ld) * static_cast<uint64_t>(rows)};
  uint32_t box[3] = {32, 32, 1};
  return make_map(m, base, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

// Epilogue tensor of a GEMM with rotary column pairing: the P columns are `nq` runs of `q` channels
// (1-D rotary: [first | partner]; 2-D: [row first | row partner | col first | col partner]) addressed as
// (channel in run, run, row in batch, batch) and moved in 32-row x 16-channel blocks (32-byte swizzle), so a
// block that hangs over the end of its run is clipped there.
inline int make_io_map_paired(CUtensorMap* m, const void* base, int64_t q, int64_t nq, int64_t rows, int64_t batches,
                       int64_t ld, int64_t batch_stride = 0) {
  if (ld % 8 || ld < q * nq || q % 8) return POM_ERR_BAD_STRIDE;
  uint64_t dims[4] = {static_cast<uint64_t>(q), static_cast<uint64_t>(nq), static_cast<uint64_t>(rows),
                      static_cast<uint64_t>(batches)};
  uint64_t str[3] = {static_cast<uint64_t>(q), static_cast<uint64_t>(ld),
                     batch_stride ? static_cast<uint64_t>(batch_stride)
                                  : static_cast<uint64_t>(ld) * static_cast<uint64_t>(rows)};
  uint32_t box[4] = {16, 1, 32, 1};
  return make_map(m, base, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_32B);
}

// The first 32 rows of a (len, q) fp32 rotary table, moved in 32-row x 16-column blocks (64-byte swizzle).
inline int make_lane_table_map(CUtensorMap* m, const float* table, int64_t q, int64_t len) {
  if (q % 4) return POM_ERR_BAD_STRIDE;
  uint64_t dims[2] = {static_cast<uint64_t>(q), static_cast<uint64_t>(len < 32 ? len : 32)};
  uint64_t str[1] = {static_cast<uint64_t>(q)};
  uint32_t box[2] = {16, 32};
  return make_map(m, table, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_64B, 4);
}

struct Operands {
  const void* A;
  const void* Bm;
  int64_t M, N, K;  // per batch rows, columns, reduction
  int64_t lda, ldb;
  int batches;
  bool a_mn, b_mn;
  const float* tile_weight = nullptr;  // optional per (batch, 128-row tile) weights: 0 skips the tile
  // strided batches: element offsets between consecutive batches (0 = the matrices follow one another);
  // b_batched: the B operand has one matrix per batch too
  int64_t a_batch_stride = 0, b_batch_stride = 0;
  bool b_batched = false;
  // rotary column pairing (K-major B only): the N columns are `pair_sections` sections of 2 * pair_q channels,
  // first channels followed by their partners; every tile holds first channels in its left half and their
  // partners in its right half
  int pair_q = 0;
  int pair_sections = 1;
};

// `b_rows`: rows of the B tile one CTA loads per stage (K-major B only; MN-major B uses 64-wide boxes).
inline int build_maps(const Operands& o, int b_rows, CUtensorMap* tmA, CUtensorMap* tmB) {
  int rc;
  const uint64_t nb_a = static_cast<uint64_t>(o.batches);
  const uint64_t nb_b = o.b_batched ? static_cast<uint64_t>(o.batches) : 1;
  if (!o.a_mn) {
    uint64_t dims[3] = {static_cast<uint64_t>(o.K), static_cast<uint64_t>(o.M), nb_a};
    uint64_t str[2] = {static_cast<uint64_t>(o.lda),
                       static_cast<uint64_t>(o.a_batch_stride ? o.a_batch_stride : o.lda * o.M)};
    uint32_t box[3] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(kBM), 1};
    rc = make_map(tmA, o.A, 3, dims, str, box);
  } else {
    uint64_t dims[3] = {static_cast<uint64_t>(o.M), static_cast<uint64_t>(o.K), nb_a};
    uint64_t str[2] = {static_cast<uint64_t>(o.lda),
                       static_cast<uint64_t>(o.a_batch_stride ? o.a_batch_stride : o.lda * o.K)};
    uint32_t box[3] = {64, static_cast<uint32_t>(kBK), 1};
    rc = make_map(tmA, o.A, 3, dims, str, box);
  }
  if (rc) return rc;
  if (!o.b_mn) {
    uint64_t dims[3] = {static_cast<uint64_t>(o.K), static_cast<uint64_t>(o.N), nb_b};
    uint64_t str[2] = {static_cast<uint64_t>(o.ldb),
                       static_cast<uint64_t>(o.b_batch_stride ? o.b_batch_stride : o.ldb * o.N)};
    uint32_t box[3] = {static_cast<uint32_t>(kBK), static_cast<uint32_t>(b_rows), 1};
    rc = make_map(tmB, o.Bm, 3, dims, str, box);
  } else {
    uint64_t dims[3] = {static_cast<uint64_t>(o.N), static_cast<uint64_t>(o.K), nb_b};
    uint64_t str[2] = {static_cast<uint64_t>(o.ldb),
                       static_cast<uint64_t>(o.b_batch_stride ? o.b_batch_stride : o.ldb * o.K)};
    uint32_t box[3] = {64, static_cast<uint32_t>(kBK), 1};
    rc = make_map(tmB, o.Bm, 3, dims, str, box);
  }
  return rc;
}

// Diagnostic knob (pom_set_gemm_mode).  Units digit: 0 automatic choice, 1 always the one-CTA kernel, 2 always the
// two-CTA (pair) kernel; tens digit: 1 / 2 / 3 forces 128 / 192 / 256 columns per tile; hundreds digit 1: the
// paired epilogues never get the column-stationary grid.
extern std::atomic<int> g_gemm_mode;

// Rows per B-operand box of a paired tile: the whole half tile, or, with two sections, the largest piece that never
// reaches over the border between them.
inline int paired_box_rows(const Operands& o, int bn) {
  if (!o.pair_q) return bn;
  int a = o.pair_q, b = bn / 2;
  if (o.pair_sections == 1) return b;
  while (b) {
    const int r = a % b;
    a = b, b = r;
  }
  return a;
}

inline GemmGeom make_geom(const Operands& o, int bn, int split_k) {
  GemmGeom g;
  g.batches = o.batches;
  g.rows_per_batch = static_cast<int>(o.M);
  g.m_tiles_per_batch = static_cast<int>(ceil_div(o.M, kBM));
  g.pair_q = o.pair_q;
  g.pair_total = o.pair_q * o.pair_sections;
  g.b_box_rows = paired_box_rows(o, bn);
  g.n_tiles = static_cast<int>(o.pair_q ? ceil_div(g.pair_total, bn / 2) : ceil_div(o.N, bn));
  g.n_cols = static_cast<int>(o.N);
  g.k_blocks = static_cast<int>(ceil_div(o.K, kBK));
  if (split_k < 1) split_k = 1;
  if (split_k > g.k_blocks) split_k = g.k_blocks;
  g.kb_per_split = static_cast<int>(ceil_div(g.k_blocks, split_k));
  g.split_k = static_cast<int>(ceil_div(g.k_blocks, g.kb_per_split));
  g.group_m = 8;
  g.tile_weight = o.tile_weight;
  g.b_batched = o.b_batched ? 1 : 0;
  return g;
}

inline int check_operands(const Operands& o) {
  if (!o.A || !o.Bm) return POM_ERR_NULL;
  if (o.M <= 0 || o.N <= 0 || o.K <= 0 || o.batches <= 0) return POM_ERR_BAD_SHAPE;
  if (o.M > INT32_MAX || o.N > INT32_MAX || o.K > INT32_MAX) return POM_ERR_TOO_LARGE;
  if (o.lda % 8 || o.ldb % 8) return POM_ERR_BAD_STRIDE;
  if ((!o.a_mn && o.lda < o.K) || (o.a_mn && o.lda < o.M)) return POM_ERR_BAD_STRIDE;
  if ((!o.b_mn && o.ldb < o.K) || (o.b_mn && o.ldb < o.N)) return POM_ERR_BAD_STRIDE;
  return POM_OK;
}

template <class Kern>
int set_smem_once(Kern kern, int smem, std::atomic<uint64_t>* done) {
  return once_per_device(*done, [&] {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      (void)cudaGetLastError();
      return static_cast<int>(POM_ERR_CUDA);
    }
    return static_cast<int>(POM_OK);
  });
}

// Epilogues whose constants depend on the tile's columns (Epi::kStager: lane tables, coefficients, bias) run
// column-stationary when that costs little: a grid of rows x n_tiles CTAs (or clusters) walking bands of `rows`
// m-tiles gives every CTA the same columns in all of its tiles, so those constants are loaded once per CTA.
// Returns the rows per band, or 0 to keep the default schedule (more than 1/16 of the SMs would idle, or the
// problem has no second wave).
inline int stationary_rows(long long units, int n_tiles, int slots) {
  if (g_gemm_mode.load(std::memory_order_relaxed) / 100 == 1) return 0;  // diagnostic: default schedule
  if (n_tiles > slots || units <= slots) return 0;
  const int rows = slots / n_tiles;
  return (slots - rows * n_tiles) * 16 <= slots ? rows : 0;
}

// Launch with programmatic stream serialization: the kernel may become resident while its predecessor drains; it
// calls griddepcontrol.wait before it reads anything the predecessor wrote.
template <class Kern, class... Args>
int launch_overlapped(Kern kern, int grid, int smem, cudaStream_t st, Args... args) {
  if (launch_pdl(kern, dim3(static_cast<unsigned>(grid)), dim3(kGemmThreads), static_cast<size_t>(smem), st, args...) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  count_launch();
  return check_launch();
}

// One CTA per 128 x BN tile.
template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
int launch(const Operands& o, int split_k, const EpiMaps& maps, const typename Epi::Params& ep, int* status,
           cudaStream_t st) {
  CUtensorMap tmA, tmB;
  int rc = build_maps(o, paired_box_rows(o, BN), &tmA, &tmB);
  if (rc) return rc;
  GemmGeom g = make_geom(o, BN, split_k);
  constexpr int smem = gemm_smem_bytes<BN, STAGES, Epi>();
  auto kern = gemm_tcgen05_kernel<BN, STAGES, A_MN, B_MN, Epi>;
  static std::atomic<uint64_t> attr_set{0};
  if ((rc = set_smem_once(kern, smem, &attr_set))) return rc;
  const long long units = 1ll * g.batches * g.m_tiles_per_batch * g.n_tiles * g.split_k;
  if (units > INT32_MAX) return POM_ERR_TOO_LARGE;
  int grid = static_cast<int>(units < sm_count() ? units : sm_count());
  if constexpr (Epi::kStager) {
    const int rows = g.split_k == 1 ? stationary_rows(units, g.n_tiles, sm_count()) : 0;
    if (rows) grid = rows * g.n_tiles, g.group_m = rows;
  }
  return launch_overlapped(kern, grid, smem, st, tmA, tmB, maps, g, ep, status);
}

// Two CTAs (one cluster) per 256 x BN tile; each CTA loads BN/2 rows of the B tile.
template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
int launch_pair(const Operands& o, int split_k, const EpiMaps& maps, const typename Epi::Params& ep, int* status,
                cudaStream_t st) {
  CUtensorMap tmA, tmB;
  int rc = build_maps(o, o.pair_q ? paired_box_rows(o, BN) : BN / 2, &tmA, &tmB);
  if (rc) return rc;
  GemmGeom g = make_geom(o, BN, split_k);
  constexpr int smem = gemm2_smem_bytes<BN, STAGES, Epi>();
  auto kern = gemm_tcgen05_2cta_kernel<BN, STAGES, A_MN, B_MN, Epi>;
  static std::atomic<uint64_t> attr_set{0};
  if ((rc = set_smem_once(kern, smem, &attr_set))) return rc;
  const long long units = 1ll * g.batches * ((g.m_tiles_per_batch + 1) / 2) * g.n_tiles * g.split_k;
  if (units > INT32_MAX) return POM_ERR_TOO_LARGE;
  int clusters = static_cast<int>(units < sm_count() / 2 ? units : sm_count() / 2);
  if constexpr (Epi::kStager) {
    const int rows = g.split_k == 1 ? stationary_rows(units, g.n_tiles, sm_count() / 2) : 0;
    if (rows) clusters = rows * g.n_tiles, g.group_m = 2 * rows;  // group_m counts m-tiles: two per pair
  }
  return launch_overlapped(kern, 2 * clusters, smem, st, tmA, tmB, maps, g, ep, status);
}

struct TilePlan {
  bool pair;
  int bn;
};

// Tile plan by estimated time: (waves of work units over the SMs, or SM pairs) x (columns per tile) x a factor
// per kernel flavour and width.  The factors are measured time per (wave x column) relative to the pair kernel at
// 256 columns (32768..8192 x 1152 x 2304 and x 4608 products on B200): narrower tiles re-read the A operand more
// often and pay more per column, but they divide a small problem into more units, which wins when the wide plan
// would leave most SMs idle in its last wave (8192-row problems: 160 pair tiles = 2.2 waves of 74 clusters).
inline double plan_factor(bool pair, int bn) {
  if (pair) return bn == 256 ? 1.00 : bn == 192 ? 1.21 : 1.71;
  return bn == 256 ? 1.02 : bn == 192 ? 1.17 : 1.53;
}

inline TilePlan pick_plan(const Operands& o, bool allow_192, bool splittable = false) {
  // diagnostic override (pom_set_gemm_mode): units digit 1 / 2 forces the one-CTA / pair kernel, tens digit
  // 1 / 2 / 3 forces 128 / 192 / 256 columns per tile where that width exists for the operands
  const int knob = g_gemm_mode.load(std::memory_order_relaxed) % 100;
  const int mode = knob % 10;
  const int force_bn = knob / 10 == 1 ? 128 : knob / 10 == 2 ? 192 : knob / 10 == 3 ? 256 : 0;
  const long long m_tiles = 1ll * o.batches * ceil_div(o.M, kBM);
  TilePlan best{false, 128};
  double best_cost = -1.0;
  for (int pair = 1; pair >= 0; --pair) {
    if (mode == 1 && pair) continue;
    if (mode == 2 && !pair) continue;
    const int cands[3] = {256, 192, 128};
    for (int bn : cands) {
      const bool has_192 = allow_192 && !(pair && o.b_mn);
      if (bn == 192 && !has_192) continue;
      if (o.N <= 128 && bn != 128) continue;
      if (force_bn && bn != force_bn && !(force_bn == 192 && !has_192)) continue;
      const long long n_tiles = o.pair_q ? ceil_div(1ll * o.pair_sections * o.pair_q, bn / 2) : ceil_div(o.N, bn);
      const long long units = (pair ? (m_tiles + 1) / 2 : m_tiles) * n_tiles;
      const int slots = pair ? sm_count() / 2 : sm_count();
      // split-K products fill the last wave with K slices (pick_split): their cost is the work itself (an odd row
      // of tiles that leaves half a pair empty is not charged either: the split spreads it)
      const double waves = splittable ? (pair ? 0.5 : 1.0) * static_cast<double>(m_tiles * n_tiles) / slots
                                      : static_cast<double>(ceil_div(units, slots));
      const double cost = waves * bn * plan_factor(pair != 0, bn);
      if (best_cost < 0 || cost < best_cost - 1e-9) {
        best_cost = cost;
        best = TilePlan{pair != 0, bn};
      }
    }
  }
  return best;
}

// Split of the reduction dimension for accumulate-mode GEMMs: the smallest split whose work
// units fill the last wave to at least 93 %, keeping at least 8 k-blocks per split.
inline int pick_split(long long units, long long kblocks, int slots) {
  long long cap = kblocks / 8 > 0 ? kblocks / 8 : 1;
  if (cap > 32) cap = 32;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= cap; ++s) {
    const long long u = units * s;
    const double eff = static_cast<double>(u) / static_cast<double>(ceil_div(u, slots) * slots);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = s;
    }
    if (eff >= 0.93) return s;
  }
  return best;
}

inline long long plan_units(const Operands& o, const TilePlan& p) {
  const long long mt = ceil_div(o.M, kBM);
  const long long nt = o.pair_q ? ceil_div(1ll * o.pair_sections * o.pair_q, p.bn / 2) : ceil_div(o.N, p.bn);
  return 1ll * o.batches * (p.pair ? (mt + 1) / 2 : mt) * nt;
}

// Pipeline depth: as many stages as fit beside the epilogue staging area and scratch in the
// 227 KiB of shared memory one CTA may use (at most 8).
template <int STAGE_BYTES, class Epi, int BN>
constexpr int stages_for() {
  constexpr int kMaxSmem = 232448;
  constexpr int n = (kMaxSmem - SmemPlan<1>::bytes(0, Epi::template smem_bytes<BN>(), Epi::kStageBytes)) / STAGE_BYTES;
  return n > 8 ? 8 : (n < 1 ? 1 : n);  // (a width that does not fit at all is never launched: see run_plan)
}

// Dispatch over kernel flavour and tile width for a fixed operand order and epilogue.
template <bool A_MN, bool B_MN, class Epi>
int run_plan(const TilePlan& p, const Operands& o, int split, const EpiMaps& maps, const typename Epi::Params& ep,
             int* status, cudaStream_t st) {
  if (p.pair) {
    // an epilogue whose staging leaves fewer than three pipeline stages beside a 256-column tile takes the next width
    constexpr bool k256_fits = stages_for<Gemm2Smem<256>::kStageBytes, Epi, 256>() >= 3;
    if (p.bn == 256 && (k256_fits || B_MN))
      return launch_pair<256, stages_for<Gemm2Smem<256>::kStageBytes, Epi, 256>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
    if constexpr (!B_MN) {
      if (p.bn == 192 || p.bn == 256)
        return launch_pair<192, stages_for<Gemm2Smem<192>::kStageBytes, Epi, 192>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
    }
    return launch_pair<128, stages_for<Gemm2Smem<128>::kStageBytes, Epi, 128>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
  }
  constexpr bool k256_one_fits = stages_for<GemmSmem<256>::kStageBytes, Epi, 256>() >= 2;
  if (p.bn == 256 && k256_one_fits)
    return launch<256, stages_for<GemmSmem<256>::kStageBytes, Epi, 256>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
  if (p.bn == 192 || p.bn == 256)
    return launch<192, stages_for<GemmSmem<192>::kStageBytes, Epi, 192>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
  return launch<128, stages_for<GemmSmem<128>::kStageBytes, Epi, 128>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
}

template <class Epi>
int run_plan_any_major(const TilePlan& p, const Operands& o, int split, const EpiMaps& maps,
                       const typename Epi::Params& ep, int* status, cudaStream_t st) {
  if (!o.a_mn && !o.b_mn) return run_plan<false, false, Epi>(p, o, split, maps, ep, status, st);
  if (!o.a_mn && o.b_mn) return run_plan<false, true, Epi>(p, o, split, maps, ep, status, st);
  if (o.a_mn && !o.b_mn) return run_plan<true, false, Epi>(p, o, split, maps, ep, status, st);
  return run_plan<true, true, Epi>(p, o, split, maps, ep, status, st);
}


}  // namespace pomh
