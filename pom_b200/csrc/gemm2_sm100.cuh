// Two-SM variant of the GEMM engine: a cluster of two CTAs computes one 256 x BN
// output tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A
// and only HALF of the B tile (BN/2 rows), so the bytes pulled from L2 per flop drop
// by a third against the one-CTA kernel, whose 128 x 256 tiles are L2-bandwidth bound.
// Every CTA issues its own plain TMA loads; nothing is broadcast between CTAs.
//
//   CTA rank 0 (leader): TMA producer, MMA issuer for the pair, epilogue of rows 0..127
//   CTA rank 1 (peer)  : TMA producer,                           epilogue of rows 128..255
//
// Synchronisation (all waits bounded):
//   full[s]   leader only.  The leader arms it with the byte count of BOTH CTAs; the peer's
//             loads signal it remotely (cta_group::2 load form, barrier address mapped to rank 0).
//   empty[s]  in both CTAs, released by two tcgen05.commit (one local, one to the peer's address).
//   tfull[a]  in both CTAs, same mechanism, after the last k-block of a tile.
//   tempty[a] leader only; the epilogue warps of both CTAs arrive on it (the peer remotely).
#pragma once
#include "gemm_sm100.cuh"

namespace pomk {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory object in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                             int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                             int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at `cluster_addr` (this CTA's or the peer's) once every MMA issued so far
// by this thread has finished.
__device__ __forceinline__ void umma2_commit(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

__host__ __device__ constexpr uint32_t make_idesc_bf16_m256(int bn, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(bn >> 3) << 17) |
         (static_cast<uint32_t>(256 >> 4) << 24);
}

// Work unit -> the tile of THIS CTA (rank r takes the r-th 128-row half of the 256-row pair tile).
// A pair may hang over the end of a batch: then rows_valid is 0 and the tile contributes nothing.
__device__ __forceinline__ TileCtx decode_pair_tile(const GemmGeom& g, int unit, int bn, int rank) {
  const int pairs_per_batch = (g.m_tiles_per_batch + 1) >> 1;
  const int pairs_m = g.batches * pairs_per_batch;
  const int per_split = pairs_m * g.n_tiles;
  TileCtx t;
  t.split = unit / per_split;
  const int u = unit - t.split * per_split;
  const int gm = max(1, g.group_m >> 1);
  const int band_sz = gm * g.n_tiles;
  const int band = u / band_sz;
  const int in_band = u - band * band_sz;
  const int m_lo = band * gm;
  const int band_rows = min(gm, pairs_m - m_lo);
  const int n = in_band / band_rows;
  const int mp = m_lo + (in_band - n * band_rows);
  t.b = mp / pairs_per_batch;
  t.mt = 2 * (mp - t.b * pairs_per_batch) + rank;
  t.row0 = t.mt * kBM;
  t.rows_valid = max(0, min(kBM, g.rows_per_batch - t.row0));
  set_tile_cols(g, t, n, bn);
  // the two halves of a pair share one main loop: it is skipped only when both are empty
  t.live = true;
  if (g.tile_weight) {
    const int m0 = t.b * g.m_tiles_per_batch + 2 * (mp - t.b * pairs_per_batch);
    const bool second = 2 * (mp - t.b * pairs_per_batch) + 1 < g.m_tiles_per_batch;
    t.live = __ldg(g.tile_weight + m0) != 0.f || (second && __ldg(g.tile_weight + m0 + 1) != 0.f);
  }
  return t;
}

template <int BN>
struct Gemm2Smem {
  static constexpr int kABytes = kBM * kBK * 2;        // this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * kBK * 2;   // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
};

template <int BN, int STAGES, class Epi>
constexpr int gemm2_smem_bytes() {
  return SmemPlan<STAGES>::bytes(Gemm2Smem<BN>::kStageBytes, Epi::template smem_bytes<BN>(), Epi::kStageBytes);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ EpiMaps maps, const GemmGeom geom, const typename Epi::Params ep,
                         int* __restrict__ status) {
  static_assert(BN == 128 || BN == 256 || (BN == 192 && !B_MN), "unsupported pair-tile width");
  constexpr int kABytes = Gemm2Smem<BN>::kABytes;
  constexpr int kStageBytes = Gemm2Smem<BN>::kStageBytes;
  constexpr int kHalfN = BN / 2;
  constexpr uint32_t kTmemCols = (2 * BN <= 256) ? 256u : 512u;
  constexpr uint32_t kIdesc = make_idesc_bf16_m256(BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  const SmemPlan<STAGES> sm(smem_raw, kStageBytes, Epi::kStageBytes);
  uint8_t* tiles = sm.tiles;
  uint64_t* full_bar = sm.full_bar;      // used in the leader
  uint64_t* empty_bar = sm.empty_bar;    // both CTAs
  uint64_t* tfull_bar = sm.tfull_bar;    // both CTAs
  uint64_t* tempty_bar = sm.tempty_bar;  // used in the leader
  uint32_t* tmem_holder = sm.tmem_holder;
  volatile int* abort_flag = sm.abort_flag;
  float* epi_scratch = sm.epi_scratch;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * kEpiWarps);
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
    tmem_alloc2(tmem_holder, kTmemCols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any remote arrive or remote load completion
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // everything above overlapped the tail of the previous kernel of the stream; its results are read from here on
  griddep_wait();
  griddep_launch();

  const int pairs_per_batch = (geom.m_tiles_per_batch + 1) >> 1;
  const int total_units = geom.batches * pairs_per_batch * geom.n_tiles * geom.split_k;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      // paired columns: the leader's half of the B tile holds the first channels, the peer's their partners
      auto b_col = [&](const TileCtx& tt) {
        return geom.pair_q ? (rank == 0 ? tt.col0 : tt.col1) : tt.col0 + static_cast<int>(rank) * kHalfN;
      };
      for (int unit = cluster_id; unit < total_units && alive; unit += n_clusters) {
        const TileCtx t = decode_pair_tile(geom, unit, BN, rank);
        const int kb0 = t.split * geom.kb_per_split;
        const int kb1 = t.live ? min(geom.k_blocks, kb0 + geom.kb_per_split) : kb0;
        const int bcol0 = b_col(t);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, status, kStatusProducerTimeout)) {
            alive = false;
            break;
          }
          uint8_t* sa = tiles + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          const uint32_t full0 = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int bz = geom.b_batched ? t.b : 0;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kStageBytes);
          if constexpr (!A_MN) {
            tma2_load_3d(sa, &tmA, full0, kb * kBK, t.row0, t.b);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma2_load_3d(sa + j * (kBK * 128), &tmA, full0, t.row0 + j * 64, kb * kBK, t.b);
          }
          if constexpr (!B_MN) {
            if (geom.pair_q) {  // the leader's half of the B tile: first channels; the peer's: their partners
              load_paired_b_half<BN>(geom, t, static_cast<int>(rank), sb,
                                     [&](uint8_t* dst, int row) { tma2_load_3d(dst, &tmB, full0, kb * kBK, row, bz); });
            } else {
              tma2_load_3d(sb, &tmB, full0, kb * kBK, bcol0, bz);
            }
          } else {
#pragma unroll
            for (int j = 0; j < kHalfN / 64; ++j)
              tma2_load_3d(sb + j * (kBK * 128), &tmB, full0, bcol0 + j * 64, kb * kBK, bz);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!alive) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool alive = true;
      for (int unit = cluster_id; unit < total_units && alive; unit += n_clusters, ++iter) {
        const TileCtx t = decode_pair_tile(geom, unit, BN, 0);
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
            const uint64_t da = A_MN ? make_smem_desc(sa + k16 * 2048, kBK * 128, 1024)
                                     : make_smem_desc(sa + k16 * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k16 * 2048, kBK * 128, 1024)
                                     : make_smem_desc(sb + k16 * 32, 16, 1024);
            umma2_bf16(tmem_d, da, db, kIdesc, (kb > kb0 || k16 > 0) ? 1u : 0u);
          }
          // release the stage in both CTAs once these MMAs have read it
          const uint32_t e_local = smem_u32(&empty_bar[stage]);
          umma2_commit(e_local);
          umma2_commit(map_to_cta(e_local, 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (alive) {
          const uint32_t f_local = smem_u32(&tfull_bar[acc]);
          umma2_commit(f_local);
          umma2_commit(map_to_cta(f_local, 1));
        }
      }
      if (!alive) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
      }
    }
  } else if (warp < kStagerWarp) {
    // ------------------------------------------------------------ epilogue (both CTAs, own rows)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int epi_tid = (warp - 2) * 32 + lane;
    EpiIO io;
    io.buf0 = sm.staging + (warp - 2) * Epi::kStageBytes;
    io.buf1 = io.buf0 + Epi::kStageBytes / 2;
    io.bar = &sm.wload_bar[warp - 2];
    io.load_phase = 0;
    io.abort_flag = abort_flag;
    io.status = status;
    io.tail_count = sm.tail_count;
    const uint32_t tempty_leader[2] = {map_to_cta(smem_u32(&tempty_bar[0]), 0), map_to_cta(smem_u32(&tempty_bar[1]), 0)};
    int iter = 0;
    for (int unit = cluster_id; unit < total_units; unit += n_clusters, ++iter) {
      const TileCtx t = decode_pair_tile(geom, unit, BN, rank);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      Epi::template prologue<BN>(ep, maps, geom, t, warp - 2, epi_tid, epi_scratch, io, iter);
      bool ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, status, kStatusEpilogueTimeout);
      if constexpr (Epi::kStager) {
        if (ok) ok = mbar_wait(&sm.sfull_bar[acc], acc_phase, abort_flag, status, kStatusEpilogueTimeout);
        if (!__all_sync(0xffffffffu, ok)) break;
      } else {
        if (named_bar_any(kEpiBarrier, kEpiThreads, !ok)) break;
      }
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(quarter * 32) << 16);
      Epi::template run<BN>(ep, maps, geom, t, tmem_acc, quarter, lane, half, epi_tid, epi_scratch, io, iter);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(tempty_leader[acc]);
        if constexpr (Epi::kStager) mbar_arrive(&sm.sempty_bar[acc]);
      }
    }
    if (lane == 0) bulk_wait_all();
  } else {
    // ------------------------------------------------------------ stager (both CTAs, own rows)
    if constexpr (Epi::kStager) {
      stager_loop<BN, Epi>(ep, maps, geom, cluster_id, n_clusters, total_units,
                           [&](int unit) { return decode_pair_tile(geom, unit, BN, rank); }, lane, epi_scratch,
                           sm.sfull_bar, sm.sempty_bar, abort_flag, status);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the leader's MMAs read the peer's shared memory: nobody leaves early
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

}  // namespace pomk
