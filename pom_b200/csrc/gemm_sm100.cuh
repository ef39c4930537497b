// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA-fed tcgen05.mma with
// fp32 accumulators in tensor memory and a pluggable epilogue.
//
//   C[m, n] = sum_k A[m, k] * B[n, k]
//
// Either operand may be K-major (rows of K contiguous in memory) or MN-major
// (the matrix is stored transposed: rows indexed by k, M or N contiguous), so
// the same kernel covers the projections (X·Wᵀ), the data-gradient products
// (G·W) and the weight-gradient products (Gᵀ·X) of the PoM layer without any
// transposed copy.
//
// CTA layout (352 threads, one CTA per SM):
//   warp 0      : TMA producer   (one lane issues the tile loads)
//   warp 1      : MMA issuer     (one lane issues tcgen05.mma / commit); owns TMEM alloc
//   warps 2..9  : epilogue       (two warps per 32-lane quarter of the accumulator, interleaving
//                                 the 32-column chunks of the tile)
//   warp 10     : stager         (epilogues with Epi::kStager: fills the constants of the next tile)
// The accumulator is double-buffered in tensor memory (2 x BN fp32 columns), so
// the epilogue of tile i overlaps the main loop of tile i+1.
//
// M tiles never straddle a batch: the A operand is addressed as (k, row, batch)
// and rows past the end of a batch are zero-filled by TMA, which lets epilogues
// reduce over the tokens of one sample without segmenting.
#pragma once
#include "ptx_sm100.cuh"
#include "pom_math.cuh"

namespace pomk {

constexpr int kBM = 128;          // rows per tile (= TMEM lanes)
constexpr int kBK = 64;           // K elements per pipeline stage (= one 128-byte swizzle row)
constexpr int kEpiColSplit = 2;     // epilogue warps per 32-lane quarter; they interleave the 32-column chunks
constexpr int kEpiThreads = 128 * kEpiColSplit;
// warp 0: TMA producer, warp 1: MMA issuer, warps 2..9: epilogue, warp 10: stager (fills the constants of the
// epilogue's next tile while the epilogue warps work on the current one; idle for epilogues that have none)
constexpr int kStagerWarp = 2 + 4 * kEpiColSplit;
constexpr int kGemmThreads = 32 * (kStagerWarp + 1);
constexpr int kEpiBarrier = 1;

enum GemmStatus : int {
  kStatusOk = 0,
  kStatusProducerTimeout = 101,
  kStatusMmaTimeout = 102,
  kStatusEpilogueTimeout = 103,
};

struct GemmGeom {
  int batches;            // independent row blocks of A / C (1 for a flat GEMM)
  int rows_per_batch;     // rows of A / C inside one batch
  int m_tiles_per_batch;  // ceil(rows_per_batch / 128)
  int n_tiles;            // ceil(n_cols / BN)
  int n_cols;             // columns of C
  int k_blocks;           // ceil(K / 64)
  int kb_per_split;       // k blocks handled by one split (== k_blocks when split_k == 1)
  int split_k;            // number of K splits (each split has at least one k block)
  int group_m;            // rasterisation: m tiles per band
  // Optional (batches * m_tiles_per_batch) fp32: a tile whose entry is 0 is not computed (no loads, no MMAs; its
  // epilogue sees t.live == false).  Used by the context phase to skip 128-token tiles that a mask empties.
  const float* tile_weight;
  int b_batched;          // 1: the B operand has one matrix per batch (third tensor-map coordinate = batch)
  // Rotary column pairing (0 = off): the N columns are one or two sections of 2 * pair_q channels, pair_q first
  // channels followed by their pair_q rotation partners.  The pairs of all sections, laid end to end, are cut into
  // tiles of BN/2 pairs: a tile holds the first channels of its pairs in its left half and their partners in its
  // right half.  A tile may reach over the border between the two sections; a 16-pair sub-unit and a B box of
  // `b_box_rows` rows never do (two sections: pair_q is a multiple of 16 and of b_box_rows).
  int pair_q;
  int pair_total;  // pair_q x sections
  int b_box_rows;  // rows per B-operand box (paired, K-major B): BN/2, or gcd(pair_q, BN/2) with two sections
};

struct TileCtx {
  int b;           // batch
  int mt;          // m tile inside the batch
  int row0;        // first row inside the batch
  int rows_valid;  // valid rows of this tile (1..128)
  int col0;        // first column of C (paired: global column of the tile's first first-channel)
  int col1;        // paired: global column of the partner of col0 (= col0 + pair_q)
  int u0;          // paired: index of col0 inside its section's run of first channels
  int sec;         // paired: section of the tile's first pair
  int gp0;         // paired: index of the tile's first pair among the pairs of all sections laid end to end
  int split;       // K split index
  bool live;       // false: the main loop is skipped for this tile (see GemmGeom::tile_weight)
};

// Where pair j of a paired tile sits: its section, its index inside the section's run of first channels, the global
// column of its first channel (the partner is pair_q columns further), and whether it exists at all.
struct PairPos {
  int sec, u, col;
  bool ok;
};
__device__ __forceinline__ PairPos pair_pos(const GemmGeom& g, const TileCtx& t, int j) {
  PairPos p;
  const int gp = t.gp0 + j;
  p.sec = gp >= g.pair_q && g.pair_total > g.pair_q ? 1 : 0;  // at most two sections
  p.u = gp - (p.sec ? g.pair_q : 0);
  p.col = p.sec * 2 * g.pair_q + p.u;
  p.ok = gp < g.pair_total;
  return p;
}

__device__ __forceinline__ void set_tile_cols(const GemmGeom& g, TileCtx& t, int n, int bn) {
  if (g.pair_q) {
    t.gp0 = n * (bn >> 1);
    const PairPos p = pair_pos(g, t, 0);
    t.sec = p.sec;
    t.u0 = p.u;
    t.col0 = p.col;
    t.col1 = t.col0 + g.pair_q;
  } else {
    t.col0 = n * bn;
    t.col1 = t.col0;
    t.u0 = t.col0;
    t.sec = 0;
    t.gp0 = 0;
  }
}

// Paired tiles, K-major B: loads the BN/2 rows of one half of the B tile (partner == 0: the first channels of the
// tile's pairs, 1: their partners) as boxes of g.b_box_rows rows; rows of pairs that do not exist are zero-filled
// (a box starting past the last row of B).
template <int BN, class Load>
__device__ __forceinline__ void load_paired_b_half(const GemmGeom& g, const TileCtx& t, int partner, uint8_t* dst,
                                                   Load load) {
  for (int j = 0; j < BN / 2; j += g.b_box_rows) {
    const PairPos p = pair_pos(g, t, j);
    load(dst + j * (kBK * 2), p.ok ? p.col + partner * g.pair_q : g.n_cols);
  }
}

__device__ __forceinline__ TileCtx decode_tile(const GemmGeom& g, int unit, int bn) {
  TileCtx t;
  const int tiles_m = g.batches * g.m_tiles_per_batch;
  const int per_split = tiles_m * g.n_tiles;
  t.split = unit / per_split;
  int u = unit - t.split * per_split;
  // Bands of group_m m-tiles; inside a band consecutive units walk m first so
  // concurrently running CTAs share B tiles through L2 and reuse A tiles.
  const int band_sz = g.group_m * g.n_tiles;
  const int band = u / band_sz;
  const int in_band = u - band * band_sz;
  const int m_lo = band * g.group_m;
  const int band_rows = min(g.group_m, tiles_m - m_lo);
  const int n = in_band / band_rows;
  const int m = m_lo + (in_band - n * band_rows);
  t.b = m / g.m_tiles_per_batch;
  t.mt = m - t.b * g.m_tiles_per_batch;
  t.row0 = t.mt * kBM;
  t.rows_valid = min(kBM, g.rows_per_batch - t.row0);
  set_tile_cols(g, t, n, bn);
  t.live = !g.tile_weight || __ldg(g.tile_weight + m) != 0.f;
  return t;
}

template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;  // 16 KiB
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
};

// ---------------------------------------------------------------------------
// Epilogue I/O through the TMA engine
// ---------------------------------------------------------------------------
// Tensor maps of the epilogue: up to two bf16 outputs and one bf16 input, each addressed
// as (column, row-in-batch, batch) with a 32 x 32 box and 64-byte swizzle.
struct alignas(64) EpiMaps {
  CUtensorMap out0;
  CUtensorMap out1;
  CUtensorMap in0;
  CUtensorMap in1;
  // rotary epilogues: rows 0..31 of the {cos, sin} table of section 0 and of section 1 (fp32, 32 x 16 boxes)
  CUtensorMap lane[4];
};

// Per-warp staging: two 2 KiB chunk buffers (1 KiB aligned) and one mbarrier for bulk loads.
struct EpiIO {
  uint8_t* buf0;
  uint8_t* buf1;
  uint64_t* bar;
  uint32_t load_phase;  // parity of the next bulk load to complete on `bar`
  volatile int* abort_flag;
  int* status;
  int* tail_count;  // [2] per tile parity: epilogue warps that have finished their share of a tile (stager epilogues)
};

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

constexpr int kEpiWarps = 4 * kEpiColSplit;
constexpr int kEpiStageBytes = 4096;  // default per epilogue warp: two 2 KiB blocks for bulk stores / loads

// Carves the dynamic shared memory of both GEMM kernels:
//   [pipeline tiles][epilogue staging 8 x 4 KiB][barriers, TMEM holder, abort flag: 512 B][epilogue scratch]
constexpr int kBarrierBytes = 512;
template <int STAGES>
struct SmemPlan {
  uint8_t* tiles;
  uint8_t* staging;
  uint64_t* full_bar;    // [STAGES]  TMA -> MMA
  uint64_t* empty_bar;   // [STAGES]  MMA -> TMA
  uint64_t* tfull_bar;   // [2]       MMA -> epilogue
  uint64_t* tempty_bar;  // [2]       epilogue -> MMA
  uint64_t* wload_bar;   // [8]       per epilogue warp: bulk loads into its staging block
  uint64_t* sfull_bar;   // [2]       stager -> epilogue: the constants of a tile are in their slot
  uint64_t* sempty_bar;  // [2]       epilogue -> stager: every epilogue warp has finished with the slot
  uint32_t* tmem_holder;
  volatile int* abort_flag;
  int* tail_count;
  float* epi_scratch;
  __device__ __forceinline__ SmemPlan(uint8_t* raw, int stage_bytes, int epi_stage_bytes = kEpiStageBytes) {
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    tiles = base;
    staging = base + STAGES * stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpiWarps * epi_stage_bytes);
    full_bar = bars;
    empty_bar = bars + STAGES;
    tfull_bar = bars + 2 * STAGES;
    tempty_bar = bars + 2 * STAGES + 2;
    wload_bar = bars + 2 * STAGES + 4;
    sfull_bar = bars + 2 * STAGES + 4 + kEpiWarps;
    sempty_bar = bars + 2 * STAGES + 6 + kEpiWarps;
    tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 8 + kEpiWarps);
    abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    tail_count = reinterpret_cast<int*>(tmem_holder + 2);
    static_assert((2 * STAGES + 10 + kEpiWarps) * 8 <= kBarrierBytes, "barrier area too small");
    epi_scratch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + kBarrierBytes);
  }
  static constexpr int bytes(int stage_bytes, int epi_smem, int epi_stage_bytes = kEpiStageBytes) {
    return STAGES * stage_bytes + kEpiWarps * epi_stage_bytes + kBarrierBytes + epi_smem + 1024;  // + alignment slack
  }
};

template <class Epi>
constexpr int epi_stage_bytes() {
  return Epi::kStageBytes;
}

template <int BN, int STAGES, class Epi>
constexpr int gemm_smem_bytes() {
  return SmemPlan<STAGES>::bytes(GemmSmem<BN>::kStageBytes, Epi::template smem_bytes<BN>(), Epi::kStageBytes);
}

// ---------------------------------------------------------------------------
// The kernel.  `Epi` supplies:
//   struct Params;                      trivially copyable, passed by value
//   static constexpr int kSmemBytes;    scratch shared by the epilogue warps
//   template<int BN> static __device__ void prologue(const Params&, const EpiMaps&, const GemmGeom&,
//        const TileCtx&, int warp_in_epi, int epi_tid, float* scratch, EpiIO&, int tile_iter);
//        runs before the accumulator is ready: stages per-column constants, starts bulk loads
//   template<int BN> static __device__ void run(const Params&, const EpiMaps&, const GemmGeom&, const TileCtx&,
//        uint32_t tmem_acc, int quarter, int lane, int half, int epi_tid, float* scratch, EpiIO&, int tile_iter);
//   static constexpr bool kStager;      true: the constants of a tile are filled by the stager warp, one tile ahead,
//        into slot (tile_iter & 1) of the scratch; the epilogue warps then never meet at a named barrier: prologue()
//        only starts per-warp loads, run() finds its constants in place.  Such an epilogue also supplies
//   template<int BN> static __device__ uint32_t stage_cols(const Params&, const EpiMaps&, const GemmGeom&,
//        const TileCtx&, int lane, float* scratch, uint64_t* bar);
//        constants that depend on the tile's columns only (kept while consecutive tiles of the CTA share their
//        columns); returns the bytes of the bulk loads it started on `bar`
//   template<int BN> static __device__ void stage_tile(const Params&, const EpiMaps&, const GemmGeom&,
//        const TileCtx&, int lane, float* scratch, int slot);
//        constants of this tile's rows and batch
// ---------------------------------------------------------------------------

// The stager warp's loop over the tiles of its CTA.  `decode(unit)` yields the TileCtx of a unit.
template <int BN, class Epi, class Decode>
__device__ __forceinline__ void stager_loop(const typename Epi::Params& ep, const EpiMaps& maps, const GemmGeom& geom,
                                            int first_unit, int unit_stride, int total_units, Decode decode, int lane,
                                            float* scratch, uint64_t* sfull, uint64_t* sempty,
                                            volatile int* abort_flag, int* status) {
  int cur_sec = -1, cur_u0 = -1, iter = 0;
  for (int unit = first_unit; unit < total_units; unit += unit_stride, ++iter) {
    const TileCtx t = decode(unit);
    const int slot = iter & 1;
    // the slot is free once every epilogue warp has released the tile before the previous one
    bool ok = mbar_wait(&sempty[slot], ((iter >> 1) & 1u) ^ 1u, abort_flag, status, kStatusEpilogueTimeout);
    const bool new_cols = t.sec != cur_sec || t.u0 != cur_u0;
    // the column constants are shared by both slots: they change only after the previous tile has been released
    if (ok && new_cols && iter >= 1)
      ok = mbar_wait(&sempty[slot ^ 1], ((iter - 1) >> 1) & 1u, abort_flag, status, kStatusEpilogueTimeout);
    if (!__all_sync(0xffffffffu, ok)) break;
    uint32_t tx = 0;
    if (new_cols) {
      tx = Epi::template stage_cols<BN>(ep, maps, geom, t, lane, scratch, &sfull[slot]);
      cur_sec = t.sec, cur_u0 = t.u0;
    }
    Epi::template stage_tile<BN>(ep, maps, geom, t, lane, scratch, slot);
    __syncwarp();
    if (lane == 0) {
      if (tx) mbar_expect_tx(&sfull[slot], tx);  // arrives and adds the bytes of the bulk loads in flight
      else mbar_arrive(&sfull[slot]);
    }
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ EpiMaps maps, const GemmGeom geom, const typename Epi::Params ep,
                    int* __restrict__ status) {
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN must be 64..256 in steps of 64");
  constexpr int kABytes = GemmSmem<BN>::kABytes;
  constexpr int kBBytes = GemmSmem<BN>::kBBytes;
  constexpr int kStageBytes = GemmSmem<BN>::kStageBytes;
  constexpr uint32_t kTmemCols = (2 * BN <= 128) ? 128u : (2 * BN <= 256) ? 256u : 512u;
  constexpr uint32_t kIdesc = make_idesc_bf16(BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  const SmemPlan<STAGES> sm(smem_raw, kStageBytes, Epi::kStageBytes);
  uint8_t* tiles = sm.tiles;
  uint64_t* full_bar = sm.full_bar;
  uint64_t* empty_bar = sm.empty_bar;
  uint64_t* tfull_bar = sm.tfull_bar;
  uint64_t* tempty_bar = sm.tempty_bar;
  uint32_t* tmem_holder = sm.tmem_holder;
  volatile int* abort_flag = sm.abort_flag;
  float* epi_scratch = sm.epi_scratch;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], kEpiWarps);
    }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&sm.wload_bar[w], 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm.sfull_bar[a], 1);
      mbar_init(&sm.sempty_bar[a], kEpiWarps);
      sm.tail_count[a] = 0;
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // everything above overlapped the tail of the previous kernel of the stream; its results are read from here on
  griddep_wait();
  griddep_launch();

  const int total_units = geom.batches * geom.m_tiles_per_batch * geom.n_tiles * geom.split_k;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int unit = blockIdx.x; unit < total_units && alive; unit += gridDim.x) {
        const TileCtx t = decode_tile(geom, unit, BN);
        const int kb0 = t.split * geom.kb_per_split;
        const int kb1 = t.live ? min(geom.k_blocks, kb0 + geom.kb_per_split) : kb0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) {
            alive = false;
            break;
          }
          uint8_t* sa = tiles + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          const int bz = geom.b_batched ? t.b : 0;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          if constexpr (!A_MN) {
            tma_load_3d(sa, &tmA, &full_bar[stage], kb * kBK, t.row0, t.b);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_3d(sa + j * (kBK * 128), &tmA, &full_bar[stage], t.row0 + j * 64, kb * kBK, t.b);
          }
          if constexpr (!B_MN) {
            if (geom.pair_q) {  // first channels, then their rotation partners
              auto load = [&](uint8_t* dst, int row) { tma_load_3d(dst, &tmB, &full_bar[stage], kb * kBK, row, bz); };
              load_paired_b_half<BN>(geom, t, 0, sb, load);
              load_paired_b_half<BN>(geom, t, 1, sb + (BN / 2) * kBK * 2, load);
            } else {
              tma_load_3d(sb, &tmB, &full_bar[stage], kb * kBK, t.col0, bz);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (kBK * 128), &tmB, &full_bar[stage], t.col0 + j * 64, kb * kBK, bz);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!alive) {
        // Give loads already in flight time to land before the CTA retires.
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool alive = true;
      for (int unit = blockIdx.x; unit < total_units && alive; unit += gridDim.x, ++iter) {
        const TileCtx t = decode_tile(geom, unit, BN);
        const int kb0 = t.split * geom.kb_per_split;
        const int kb1 = t.live ? min(geom.k_blocks, kb0 + geom.kb_per_split) : kb0;
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1u;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, status, kStatusMmaTimeout)) {
          alive = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, kStatusMmaTimeout)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k16 = 0; k16 < kBK / 16; ++k16) {
            // K-major: step 16 elements (32 B) inside the swizzled 128 B row.
            // MN-major: step 16 k-rows = two 8-row atoms (2048 B).
            const uint64_t da = A_MN ? make_smem_desc(sa + k16 * 2048, kBK * 128, 1024)
                                     : make_smem_desc(sa + k16 * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k16 * 2048, kBK * 128, 1024)
                                     : make_smem_desc(sb + k16 * 32, 16, 1024);
            umma_bf16(tmem_d, da, db, kIdesc, (kb > kb0 || k16 > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (alive) umma_commit(&tfull_bar[acc]);  // accumulator complete
      }
      if (!alive) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
      }
    }
  } else if (warp < kStagerWarp) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are readable by this warp
    const int half = (warp - 2) >> 2;  // which of the interleaved column chunks this warp takes
    const int epi_tid = (warp - 2) * 32 + lane;
    EpiIO io;
    io.buf0 = sm.staging + (warp - 2) * Epi::kStageBytes;
    io.buf1 = io.buf0 + Epi::kStageBytes / 2;
    io.bar = &sm.wload_bar[warp - 2];
    io.load_phase = 0;
    io.abort_flag = abort_flag;
    io.status = status;
    io.tail_count = sm.tail_count;
    int iter = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, ++iter) {
      const TileCtx t = decode_tile(geom, unit, BN);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      // Stage the per-column constants of this tile (or start this warp's loads) while its main loop is running.
      Epi::template prologue<BN>(ep, maps, geom, t, warp - 2, epi_tid, epi_scratch, io, iter);
      // All 32 lanes poll so the warp stays converged for the .aligned TMEM loads.
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, status, kStatusEpilogueTimeout);
      if constexpr (Epi::kStager) {
        if (ok) ok = mbar_wait(&sm.sfull_bar[acc], acc_phase, abort_flag, status, kStatusEpilogueTimeout);
        if (!__all_sync(0xffffffffu, ok)) break;  // no named barriers in this epilogue: every warp leaves alone
      } else {
        // The epilogue warps decide together whether to go on, so none of them can be left
        // waiting at a named barrier that another one will never reach.
        if (named_bar_any(kEpiBarrier, kEpiThreads, !ok)) break;
      }
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quarter * 32) << 16);
      Epi::template run<BN>(ep, maps, geom, t, tmem_acc, quarter, lane, half, epi_tid, epi_scratch, io, iter);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[acc]);
        if constexpr (Epi::kStager) mbar_arrive(&sm.sempty_bar[acc]);
      }
    }
    if (lane == 0) bulk_wait_all();  // bulk stores still reading this warp's staging block
  } else {
    // ------------------------------------------------------------ stager
    if constexpr (Epi::kStager) {
      stager_loop<BN, Epi>(ep, maps, geom, blockIdx.x, gridDim.x, total_units,
                           [&](int unit) { return decode_tile(geom, unit, BN); }, lane, epi_scratch, sm.sfull_bar,
                           sm.sempty_bar, abort_flag, status);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace pomk
