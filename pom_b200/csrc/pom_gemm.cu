// Host launchers for the tcgen05 GEMM engine and its fused PoM epilogues, plus
// the fp32 SIMT GEMM of the high-precision mode.
#include <cudaTypedefs.h>
#include <mutex>
#include "common.cuh"
#include "epilogues.cuh"
#include "gemm2_sm100.cuh"

using namespace pomk;
using namespace pomh;

namespace pomh {
std::atomic<long long> g_launches{0};
}

namespace {

// ---------------------------------------------------------------- tensor maps
// cuTensorMapEncodeTiled is fetched through the runtime so the library has no
// link-time dependency on the driver (it must load on machines without one).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// bf16 tensor of `rank` dims (innermost first), 128-byte swizzle, zero fill out of bounds.
int make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_elems,
             const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return POM_ERR_CUDA;
  if (!aligned16(base)) return POM_ERR_BAD_ALIGN;
  cuuint64_t gdim[3];
  cuuint64_t gstr[2];
  cuuint32_t bx[3];
  cuuint32_t es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    if (dims[i] == 0) return POM_ERR_BAD_SHAPE;
    gdim[i] = dims[i];
    bx[i] = box[i];
    if (box[i] == 0 || box[i] > 256) return POM_ERR_BAD_SHAPE;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    uint64_t bytes = strides_elems[i] * 2ull;
    if (bytes % 16 != 0) return POM_ERR_BAD_STRIDE;
    if (bytes >= (1ull << 40)) return POM_ERR_TOO_LARGE;
    gstr[i] = bytes;
  }
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim,
                  gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? POM_OK : POM_ERR_CUDA;
}

// Epilogue tensor: bf16 (batches, rows, cols) with row stride ld, moved in 32 x 32 blocks (64-byte swizzle).
// batch_stride (elements) 0 = rows * ld.
int make_io_map(CUtensorMap* m, const void* base, int64_t cols, int64_t rows, int64_t batches, int64_t ld,
                int64_t batch_stride = 0) {
  if (ld % 8 || ld < cols) return POM_ERR_BAD_STRIDE;
  uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(batches)};
  uint64_t str[2] = {static_cast<uint64_t>(ld),
                     batch_stride ? static_cast<uint64_t>(batch_stride)
                                  : static_cast<uint64_t>(ld) * static_cast<uint64_t>(rows)};
  uint32_t box[3] = {32, 32, 1};
  return make_map(m, base, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_64B);
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
};

// `b_rows`: rows of the B tile one CTA loads per stage (K-major B only; MN-major B uses 64-wide boxes).
int build_maps(const Operands& o, int b_rows, CUtensorMap* tmA, CUtensorMap* tmB) {
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

GemmGeom make_geom(const Operands& o, int bn, int split_k) {
  GemmGeom g;
  g.batches = o.batches;
  g.rows_per_batch = static_cast<int>(o.M);
  g.m_tiles_per_batch = static_cast<int>(ceil_div(o.M, kBM));
  g.n_tiles = static_cast<int>(ceil_div(o.N, bn));
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

int check_operands(const Operands& o) {
  if (!o.A || !o.Bm) return POM_ERR_NULL;
  if (o.M <= 0 || o.N <= 0 || o.K <= 0 || o.batches <= 0) return POM_ERR_BAD_SHAPE;
  if (o.M > INT32_MAX || o.N > INT32_MAX || o.K > INT32_MAX) return POM_ERR_TOO_LARGE;
  if (o.lda % 8 || o.ldb % 8) return POM_ERR_BAD_STRIDE;
  if ((!o.a_mn && o.lda < o.K) || (o.a_mn && o.lda < o.M)) return POM_ERR_BAD_STRIDE;
  if ((!o.b_mn && o.ldb < o.K) || (o.b_mn && o.ldb < o.N)) return POM_ERR_BAD_STRIDE;
  return POM_OK;
}

// 0: automatic choice, 1: always the one-CTA kernel, 2: always the two-CTA (pair) kernel.
std::atomic<int> g_gemm_mode{0};

template <class Kern>
int set_smem_once(Kern kern, int smem, bool* done) {
  if (*done) return POM_OK;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  *done = true;
  return POM_OK;
}

// One CTA per 128 x BN tile.
template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
int launch(const Operands& o, int split_k, const EpiMaps& maps, const typename Epi::Params& ep, int* status,
           cudaStream_t st) {
  CUtensorMap tmA, tmB;
  int rc = build_maps(o, BN, &tmA, &tmB);
  if (rc) return rc;
  GemmGeom g = make_geom(o, BN, split_k);
  constexpr int smem = gemm_smem_bytes<BN, STAGES, Epi::kSmemBytes>();
  auto kern = gemm_tcgen05_kernel<BN, STAGES, A_MN, B_MN, Epi>;
  static bool attr_set = false;
  if ((rc = set_smem_once(kern, smem, &attr_set))) return rc;
  const long long units = 1ll * g.batches * g.m_tiles_per_batch * g.n_tiles * g.split_k;
  if (units > INT32_MAX) return POM_ERR_TOO_LARGE;
  const int grid = static_cast<int>(units < sm_count() ? units : sm_count());
  kern<<<grid, kGemmThreads, smem, st>>>(tmA, tmB, maps, g, ep, status);
  count_launch();
  return check_launch();
}

// Two CTAs (one cluster) per 256 x BN tile; each CTA loads BN/2 rows of the B tile.
template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
int launch_pair(const Operands& o, int split_k, const EpiMaps& maps, const typename Epi::Params& ep, int* status,
                cudaStream_t st) {
  CUtensorMap tmA, tmB;
  int rc = build_maps(o, BN / 2, &tmA, &tmB);
  if (rc) return rc;
  GemmGeom g = make_geom(o, BN, split_k);
  constexpr int smem = gemm2_smem_bytes<BN, STAGES, Epi::kSmemBytes>();
  auto kern = gemm_tcgen05_2cta_kernel<BN, STAGES, A_MN, B_MN, Epi>;
  static bool attr_set = false;
  if ((rc = set_smem_once(kern, smem, &attr_set))) return rc;
  const long long units = 1ll * g.batches * ((g.m_tiles_per_batch + 1) / 2) * g.n_tiles * g.split_k;
  if (units > INT32_MAX) return POM_ERR_TOO_LARGE;
  const int clusters = static_cast<int>(units < sm_count() / 2 ? units : sm_count() / 2);
  kern<<<2 * clusters, kGemmThreads, smem, st>>>(tmA, tmB, maps, g, ep, status);
  count_launch();
  return check_launch();
}

struct TilePlan {
  bool pair;
  int bn;
};

// Operand bytes pulled from L2 per output element are proportional to (rowsA + rowsB) / (128 * BN)
// with rowsB = BN (one CTA) or BN/2 (pair); weigh that by the padded width and take the cheapest.
TilePlan pick_plan(const Operands& o, bool allow_192, bool splittable = false) {
  const int mode = g_gemm_mode.load(std::memory_order_relaxed);
  const long long m_tiles = 1ll * o.batches * ceil_div(o.M, kBM);
  TilePlan best{false, 128};
  double best_cost = -1.0;
  for (int pair = 0; pair < 2; ++pair) {
    if (mode == 1 && pair) continue;
    if (mode == 2 && !pair) continue;
    if (mode == 0 && pair && m_tiles * ceil_div(o.N, 256) < sm_count()) continue;  // too little work to pair up
    const int cands[3] = {256, 192, 128};
    for (int bn : cands) {
      if (bn == 192 && (!allow_192 || (pair && o.b_mn))) continue;
      if (o.N <= 128 && bn != 128) continue;
      const double padded = static_cast<double>(ceil_div(o.N, bn) * bn);
      double cost = padded * (128.0 + (pair ? bn / 2 : bn)) / bn;
      // fewer work units than SMs (or SM pairs): the idle ones are paid for too (split-K GEMMs fill them)
      const long long units = (pair ? (m_tiles + 1) / 2 : m_tiles) * ceil_div(o.N, bn);
      const int slots = pair ? sm_count() / 2 : sm_count();
      if (!splittable && units < slots) cost *= static_cast<double>(slots) / static_cast<double>(units);
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
int pick_split(long long units, long long kblocks, int slots) {
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

long long plan_units(const Operands& o, const TilePlan& p) {
  const long long mt = ceil_div(o.M, kBM);
  return 1ll * o.batches * (p.pair ? (mt + 1) / 2 : mt) * ceil_div(o.N, p.bn);
}

// Pipeline depth: as many stages as fit beside the epilogue staging area and scratch in the
// 227 KiB of shared memory one CTA may use (at most 8).
template <int STAGE_BYTES, class Epi>
constexpr int stages_for() {
  constexpr int kMaxSmem = 232448;
  constexpr int n = (kMaxSmem - SmemPlan<1>::bytes(0, Epi::kSmemBytes)) / STAGE_BYTES;
  return n > 8 ? 8 : n;
}

// Dispatch over kernel flavour and tile width for a fixed operand order and epilogue.
template <bool A_MN, bool B_MN, class Epi>
int run_plan(const TilePlan& p, const Operands& o, int split, const EpiMaps& maps, const typename Epi::Params& ep,
             int* status, cudaStream_t st) {
  if (p.pair) {
    if (p.bn == 256)
      return launch_pair<256, stages_for<Gemm2Smem<256>::kStageBytes, Epi>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
    if constexpr (!B_MN) {
      if (p.bn == 192)
        return launch_pair<192, stages_for<Gemm2Smem<192>::kStageBytes, Epi>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
    }
    return launch_pair<128, stages_for<Gemm2Smem<128>::kStageBytes, Epi>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
  }
  if (p.bn == 256)
    return launch<256, stages_for<GemmSmem<256>::kStageBytes, Epi>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
  if (p.bn == 192)
    return launch<192, stages_for<GemmSmem<192>::kStageBytes, Epi>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
  return launch<128, stages_for<GemmSmem<128>::kStageBytes, Epi>(), A_MN, B_MN, Epi>(o, split, maps, ep, status, st);
}

template <class Epi>
int run_plan_any_major(const TilePlan& p, const Operands& o, int split, const EpiMaps& maps,
                       const typename Epi::Params& ep, int* status, cudaStream_t st) {
  if (!o.a_mn && !o.b_mn) return run_plan<false, false, Epi>(p, o, split, maps, ep, status, st);
  if (!o.a_mn && o.b_mn) return run_plan<false, true, Epi>(p, o, split, maps, ep, status, st);
  if (o.a_mn && !o.b_mn) return run_plan<true, false, Epi>(p, o, split, maps, ep, status, st);
  return run_plan<true, true, Epi>(p, o, split, maps, ep, status, st);
}

// ---------------------------------------------------------------- fp32 SIMT GEMM
// 64x64 tile, 16-deep k step, 256 threads with 4x4 outputs each.  Strided operand
// access covers both storage orders.  Accuracy, not speed, is the purpose.
__global__ void __launch_bounds__(256)
sgemm_kernel(const float* __restrict__ A, const float* __restrict__ Bm, float* __restrict__ C, int M, int N, int K,
             long long sam, long long sak, long long sbn, long long sbk, long long ldc, float alpha, int accumulate) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      // choose the faster-varying index to follow the contiguous dimension
      int mm, kk;
      if (sak == 1) {
        kk = i & 15;
        mm = i >> 4;
      } else {
        mm = i & 63;
        kk = i >> 6;
      }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? A[gm * sam + gk * sak] : 0.f;
    }
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int nn, kk;
      if (sbk == 1) {
        kk = i & 15;
        nn = i >> 4;
      } else {
        nn = i & 63;
        kk = i >> 6;
      }
      const int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < N && gk < K) ? Bm[gn * sbn + gk * sbk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* c = C + static_cast<long long>(gm) * ldc + gn;
      const float v = alpha * acc[i][j];
      *c = accumulate ? (*c + v) : v;
    }
  }
}

}  // namespace

// =========================================================================== C ABI
extern "C" {

int pom_gemm_bf16(const pom_gemm_args* a, int* status, void* stream) {
  if (!a || !a->C) return POM_ERR_NULL;
  Operands o{a->A, a->Bm, a->M, a->N, a->K, a->lda, a->ldb, a->batches, a->a_mn_major != 0, a->b_mn_major != 0};
  o.a_batch_stride = a->a_batch_stride;
  o.b_batch_stride = a->b_batch_stride;
  o.b_batched = a->b_batched != 0;
  if (a->a_batch_stride % 8 || a->b_batch_stride % 8 || a->a_batch_stride < 0 || a->b_batch_stride < 0 ||
      a->c_batch_stride < 0)
    return POM_ERR_BAD_STRIDE;
  int rc = check_operands(o);
  if (rc) return rc;
  if (a->out_mode < 0 || a->out_mode > 2) return POM_ERR_UNSUPPORTED;
  if (a->ldc < a->N) return POM_ERR_BAD_STRIDE;
  if (a->out_mode == POM_OUT_BF16 && (a->ldc % 8 || !aligned16(a->C))) return POM_ERR_BAD_ALIGN;
  int split = a->split_k;
  if (a->out_mode != POM_OUT_F32_ACCUM) {
    if (split > 1) return POM_ERR_UNSUPPORTED;
    split = 1;
  }
  const TilePlan plan = pick_plan(o, true, a->out_mode == POM_OUT_F32_ACCUM && a->split_k == 0);
  if (split == 0) split = pick_split(plan_units(o, plan), ceil_div(a->K, kBK), plan.pair ? sm_count() / 2 : sm_count());
  EpiStore::Params ep;
  ep.C = a->C;
  ep.ldc = a->ldc;
  ep.batch_stride = a->c_batch_stride ? a->c_batch_stride : a->M * a->ldc;
  if (a->out_mode == POM_OUT_BF16 && a->c_batch_stride % 8) return POM_ERR_BAD_STRIDE;
  if (a->residual && a->c_batch_stride) return POM_ERR_UNSUPPORTED;
  ep.mode = a->out_mode;
  ep.alpha = a->alpha;
  ep.act = a->act;
  ep.residual = static_cast<const __nv_bfloat16*>(a->residual);
  ep.ldr = a->ldr;
  if ((a->act || a->residual) && a->out_mode != POM_OUT_BF16) return POM_ERR_UNSUPPORTED;
  if (a->act < 0 || a->act > 1 || (a->residual && a->ldr < a->N)) return POM_ERR_UNSUPPORTED;
  EpiMaps maps{};
  if (a->out_mode == POM_OUT_BF16 &&
      (rc = make_io_map(&maps.out0, a->C, a->N, a->M, a->batches, a->ldc, a->c_batch_stride)))
    return rc;
  return run_plan_any_major<EpiStore>(plan, o, split, maps, ep, status, static_cast<cudaStream_t>(stream));
}

int pom_set_gemm_mode(int mode) {
  if (mode < 0 || mode > 2) return POM_ERR_UNSUPPORTED;
  g_gemm_mode.store(mode);
  return POM_OK;
}

int pom_gemm_f32(const pom_gemm_args* a, void* stream) {
  if (!a || !a->A || !a->Bm || !a->C) return POM_ERR_NULL;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batches <= 0) return POM_ERR_BAD_SHAPE;
  if (a->out_mode != POM_OUT_F32 && a->out_mode != POM_OUT_F32_ACCUM) return POM_ERR_UNSUPPORTED;
  if (a->a_mn_major && a->batches != 1) return POM_ERR_UNSUPPORTED;
  const long long Mtot = a->M * a->batches;
  if (Mtot > INT32_MAX || a->N > INT32_MAX || a->K > INT32_MAX) return POM_ERR_TOO_LARGE;
  const long long sam = a->a_mn_major ? 1 : a->lda, sak = a->a_mn_major ? a->lda : 1;
  const long long sbn = a->b_mn_major ? 1 : a->ldb, sbk = a->b_mn_major ? a->ldb : 1;
  dim3 grid(static_cast<unsigned>(ceil_div(a->N, 64)), static_cast<unsigned>(ceil_div(Mtot, 64)));
  if (grid.y > 65535) return POM_ERR_TOO_LARGE;
  sgemm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(a->A), static_cast<const float*>(a->Bm), static_cast<float*>(a->C),
      static_cast<int>(Mtot), static_cast<int>(a->N), static_cast<int>(a->K), sam, sak, sbn, sbk, a->ldc, a->alpha,
      a->out_mode == POM_OUT_F32_ACCUM);
  count_launch();
  return check_launch();
}

int pom_ctx_gemm(const pom_ctx_args* a, int* status, void* stream) {
  if (!a || !a->coeff || !a->partial) return POM_ERR_NULL;
  if (a->K < 1) return POM_ERR_BAD_SHAPE;
  Operands o{a->X, a->Wpo, a->N, a->P, a->D, a->ldx, a->ldw, a->B, false, false};
  o.tile_weight = a->row_weight ? a->tile_weight : nullptr;
  int rc = check_operands(o);
  if (rc) return rc;
  if (a->hp_out && (a->ld_hp % 8 || a->ld_hp < a->P || !aligned16(a->hp_out))) return POM_ERR_BAD_ALIGN;
  EpiCtx::Params ep;
  ep.coeff = a->coeff;
  ep.K = a->K;
  ep.row_weight = a->row_weight;
  ep.save_hp = a->hp_out != nullptr;
  ep.partial = a->partial;
  ep.P = a->P;
  EpiMaps maps{};
  if (a->hp_out && (rc = make_io_map(&maps.out0, a->hp_out, a->P, a->N, a->B, a->ld_hp))) return rc;
  return run_plan<false, false, EpiCtx>(pick_plan(o, false), o, 1, maps, ep, status,
                                        static_cast<cudaStream_t>(stream));
}

int pom_gate_gemm(const pom_gate_args* a, int* status, void* stream) {
  if (!a || !a->bias || !a->H || !a->sh_out) return POM_ERR_NULL;
  Operands o{a->X, a->Wse, a->T, a->P, a->D, a->ldx, a->ldw, a->B, false, false};
  int rc = check_operands(o);
  if (rc) return rc;
  if (a->h_row_stride != 0) return POM_ERR_UNSUPPORTED;
  if (a->ld_sh % 8 || a->ld_sh < a->P || !aligned16(a->sh_out)) return POM_ERR_BAD_ALIGN;
  if (a->z_out && (a->ld_z % 8 || a->ld_z < a->P || !aligned16(a->z_out))) return POM_ERR_BAD_ALIGN;
  EpiGate::Params ep;
  ep.bias = a->bias;
  ep.H = a->H;
  ep.h_batch_stride = a->h_batch_stride;
  ep.save_z = a->z_out != nullptr;
  EpiMaps maps{};
  if (a->z_out && (rc = make_io_map(&maps.out0, a->z_out, a->P, a->T, a->B, a->ld_z))) return rc;
  if ((rc = make_io_map(&maps.out1, a->sh_out, a->P, a->T, a->B, a->ld_sh))) return rc;
  return run_plan<false, false, EpiGate>(pick_plan(o, false), o, 1, maps, ep, status,
                                         static_cast<cudaStream_t>(stream));
}

int pom_gate_bwd_gemm(const pom_gate_bwd_args* a, int* status, void* stream) {
  if (!a || !a->bias || !a->H || !a->z || !a->g_out || !a->dh_partial || !a->db_partial) return POM_ERR_NULL;
  // dSH[t, p] = sum_d dY[t, d] * Wo[d, p]: the B operand is Wo stored (K = D rows, N = P columns).
  Operands o{a->dY, a->Wo, a->T, a->P, a->D, a->ld_dy, a->ldw, a->B, false, true};
  int rc = check_operands(o);
  if (rc) return rc;
  if (a->ld_g % 8 || !aligned16(a->g_out) || a->ld_z % 8 || !aligned16(a->z)) return POM_ERR_BAD_ALIGN;
  EpiGateBwd::Params ep;
  ep.bias = a->bias;
  ep.H = a->H;
  ep.h_batch_stride = a->h_batch_stride;
  ep.dh_partial = a->dh_partial;
  ep.db_partial = a->db_partial;
  ep.P = a->P;
  EpiMaps maps{};
  if ((rc = make_io_map(&maps.in0, a->z, a->P, a->T, a->B, a->ld_z))) return rc;
  if ((rc = make_io_map(&maps.out0, a->g_out, a->P, a->T, a->B, a->ld_g))) return rc;
  return run_plan<false, true, EpiGateBwd>(pick_plan(o, false), o, 1, maps, ep, status,
                                           static_cast<cudaStream_t>(stream));
}

}  // extern "C"
