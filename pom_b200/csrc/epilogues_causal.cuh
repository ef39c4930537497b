// Token-causal forms of the paired epilogues (reference pom/pom.py:92-95, pom_triton_causal.py:68-344 and
// the rotary variants pom_triton_rope.py:483-873): the prefix mean over tokens
//     H[n] = (1 / (n + 1)) * sum_{m <= n} R_m·poly(act(hp[m]))
// never exists as a separate pass over the (tokens x channels) features.
//
//   context epilogue   per 32-token group (one epilogue warp = one TMEM lane quarter) and 16-pair sub-unit: the
//                      rotated polynomial features are summed down the 32 rows (inclusive running sum) and leave
//                      as bf16 `pre` (tokens x channels) plus one fp32 total per (group, channel).
//   group scan         a tiny kernel turns the group totals into exclusive carries (+ the carry of earlier ranks).
//   gate epilogue      re-reads its `pre` block, adds the group's carry, divides by the global token index + 1 and
//                      gates: SH = R·hardsigmoid(z + b) ⊙ H[n].
//   gate backward      the same H[n] for dz; the gradient of the prefix means, dSH ⊙ R·s / (n + 1), is summed UP
//                      the rows (suffix) and leaves as bf16 `suf` plus group totals; after the reverse group scan the
//                      streamed aggregation backward reads hp and suf once.
//
// The running sums use a transposed pass through shared memory: every lane writes its row of the 32 x 32 block,
// then owns one column and walks the 32 rows.  That costs about as many instructions as the butterfly column sum it
// replaces, and the column total falls out of it.
//
// Rotation is optional (RopeEpi::rotate == 0: cos = 1, sin = 0); the column pairing of the tile is kept either
// way, so plain token-causal layers run through the same kernels.
#pragma once
#include "epilogues_rope.cuh"

namespace pomk {

// Transposition scratch of one warp: 32 rows x 32 fp32 with the 16-byte pieces of a row XOR-swizzled by the row,
// so that row writes (one lane per row) and column reads (one lane per column) are both free of bank conflicts.
__device__ __forceinline__ void tr_write_row(uint8_t* scr, int lane, const float (&v)[32]) {
#pragma unroll
  for (int k = 0; k < 8; ++k)
    *reinterpret_cast<float4*>(scr + lane * 128 + ((k ^ (lane & 7)) << 4)) =
        make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
}
__device__ __forceinline__ float tr_read(const uint8_t* scr, int row, int col) {
  return *reinterpret_cast<const float*>(scr + row * 128 + (((col >> 2) ^ (row & 7)) << 4) + ((col & 3) << 2));
}
// Byte offset of element (row, c) of a 32 x 16 bf16 block stored with the 32-byte swizzle.
__device__ __forceinline__ uint32_t blk16_off(int row, int c) {
  return row * 32 + ((((c >> 3) ^ ((row >> 2) & 1))) << 4) + ((c & 7) << 1);
}

// Lane `lane` owns column `lane` of the block in `scr` (columns 0..15: first channels -> blk, 16..31: partners ->
// blk + 1024): inclusive running sums down the rows (REVERSE: up the rows) written as bf16; returns the column total.
template <bool REVERSE>
__device__ __forceinline__ float scan_column(const uint8_t* scr, uint8_t* blk, int lane) {
  uint8_t* dst = blk + (lane >> 4) * 1024;
  const int c = lane & 15;
  float run = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int r = REVERSE ? 31 - i : i;
    run += tr_read(scr, r, lane);
    *reinterpret_cast<__nv_bfloat16*>(dst + blk16_off(r, c)) = __float2bfloat16_rn(run);
  }
  return run;
}

// Four bf16 values (columns i .. i+3, i a multiple of 4) of row `lane` of a 32 x 16 block.
__device__ __forceinline__ void read_block16_4(const uint8_t* buf, int lane, int i, float (&o)[4]) {
  const uint2 q = *reinterpret_cast<const uint2*>(buf + swz32(lane, i >> 3) + ((i & 7) << 1));
  o[0] = __uint_as_float(q.x << 16), o[1] = __uint_as_float(q.x & 0xffff0000u);
  o[2] = __uint_as_float(q.y << 16), o[3] = __uint_as_float(q.y & 0xffff0000u);
}

struct CausalEpi {
  float* group_sums;        // (B, groups, P) fp32: totals written by the context / gate-backward epilogue
  const float* carry;       // (B, groups, P) fp32: exclusive carries read by the gate / gate-backward epilogue
  int groups;               // ceil(rows per batch / 32)
  long long token_offset;   // global index of token 0 of this call
  int P;
};

// Stager warp: carry[quarter][c] of the tile's four 32-token groups for the tile's (paired) columns, four columns
// per load (P, pair_q and the tile's first pair are multiples of 4).
template <int BN>
__device__ __forceinline__ void stage_carry(float* dst, const CausalEpi& ce, const GemmGeom& g, const TileCtx& t,
                                            int lane) {
  constexpr int kVec = BN / 4;  // float4 per row group
#pragma unroll
  for (int k = 0; k < 4 * kVec / 32; ++k) {
    const int idx = lane + 32 * k;
    const int quarter = idx / kVec, c = (idx - quarter * kVec) * 4;
    bool ok;
    const int col = paired_col<BN>(g, t, c, &ok);
    const int grp = (t.row0 >> 5) + quarter;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok && grp < ce.groups && t.rows_valid > 0)
      v = __ldg(reinterpret_cast<const float4*>(ce.carry + (static_cast<long long>(t.b) * ce.groups + grp) * ce.P + col));
    *reinterpret_cast<float4*>(dst + 4 * idx) = v;
  }
}

// --------------------------------------------------------------- context phase, token-causal
struct EpiCtxCausal {
  struct Params {
    const float* coeff;
    int K;
    int save_hp;
    RopeEpi rope;
    CausalEpi causal;
  };
  static constexpr int kMaxK = 4;
  // per warp: {hp first, hp partner, pre first, pre partner} 1 KiB output blocks, then the 4 KiB transposition block
  static constexpr int kStageBytes = 8192;
  static constexpr int kSmemBytes = 0;
  static constexpr bool kStager = true;
  template <int BN>
  using Scratch = PairScratch<BN, kMaxK, 0, 0>;  // columns: coefficients [degree][BN]
  template <int BN>
  static constexpr int smem_bytes() {
    return Scratch<BN>::kBytes;
  }

  template <int BN>
  static __device__ __forceinline__ uint32_t stage_cols(const Params& p, const EpiMaps& maps, const GemmGeom& g,
                                                        const TileCtx& t, int lane, float* scratch, uint64_t* bar) {
    const Scratch<BN> sc(scratch);
    const uint32_t tx = rope_stage_lane<BN>(p.rope, maps, g, t, lane, sc.lane(), bar);
    float* cst = sc.cols();
    const int K = p.K;
    for (int idx = lane; idx < BN * K; idx += 32) {
      const int c = idx / K, i = idx - c * K;
      bool ok;
      const int col = paired_col<BN>(g, t, c, &ok);
      cst[i * BN + c] = ok ? __ldg(p.coeff + static_cast<long long>(col) * K + i) : 0.f;
    }
    return tx;
  }
  template <int BN>
  static __device__ __forceinline__ void stage_tile(const Params& p, const EpiMaps&, const GemmGeom& g,
                                                    const TileCtx& t, int lane, float* scratch, int slot) {
    const Scratch<BN> sc(scratch);
    rope_stage_base<BN>(p.rope, g, t, lane, sc.base_cos(slot), sc.base_sin(slot));
  }
  template <int BN>
  static __device__ __forceinline__ void prologue(const Params&, const EpiMaps&, const GemmGeom&, const TileCtx&, int,
                                                  int, float*, EpiIO&, int) {}

  template <int KT, int BN>
  static __device__ __forceinline__ void body(const Params& p, const EpiMaps& maps, const GemmGeom& g,
                                              const TileCtx& t, uint32_t tmem_acc, int quarter, int lane, int half,
                                              const float* cst, const RopeView& rs, EpiIO& io) {
    const int y = t.row0 + quarter * 32;
    const int grp = (t.row0 >> 5) + quarter;
    const bool grp_ok = grp < p.causal.groups && t.rows_valid > 0;
    uint8_t* out = io.buf0;          // hp first | hp partner | pre first | pre partner
    uint8_t* scr = io.buf0 + 4096;   // transposition block
#pragma unroll 1
    for (int su = half; su < BN / 32; su += kEpiColSplit) {
      const PairPos pp = pair_pos(g, t, 16 * su);
      if (!pp.ok) break;  // warp-uniform
      const bool stepped = p.rope.step_of(pp.sec) != 0;
      float v[32];
      tmem_ld16<0>(tmem_acc + 16 * su, v);
      tmem_ld16<16>(tmem_acc + BN / 2 + 16 * su, v);
      tmem_ld_wait();
      uint32_t pk1[8], pk2[8];
      round_pack16<0>(v, pk1);
      round_pack16<16>(v, pk2);
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        float a1[4], a2[4], f1[4], f2[4], c[4], s[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) a1[e] = act_fast(v[i + e]), a2[e] = act_fast(v[16 + i + e]);
        poly4<KT, BN>(cst + 16 * su + i, p.K, a1, f1);
        poly4<KT, BN>(cst + BN / 2 + 16 * su + i, p.K, a2, f2);
        rope_cs4<BN>(rs, stepped, quarter, lane, su, i, c, s);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[i + e] = f1[e] * c[e] - f2[e] * s[e];
          v[16 + i + e] = f2[e] * c[e] + f1[e] * s[e];
        }
      }
      // rows past the end of the batch hold poly(act(0)) = 0: they extend the running sums by nothing
      tr_write_row(scr, lane, v);
      if (lane == 0) bulk_wait_read<0>();  // the previous sub-unit's stores have left the output blocks
      __syncwarp();
      if (p.save_hp) {
        write_block16(out, lane, pk1);
        write_block16(out + 1024, lane, pk2);
      }
      const float total = scan_column<false>(scr, out + 2048, lane);
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && t.rows_valid > 0) {
        if (p.save_hp) {
          tma_store_4d(&maps.out0, out, pp.u, 2 * pp.sec, y, t.b);
          tma_store_4d(&maps.out0, out + 1024, pp.u, 2 * pp.sec + 1, y, t.b);
        }
        tma_store_4d(&maps.out1, out + 2048, pp.u, 2 * pp.sec, y, t.b);
        tma_store_4d(&maps.out1, out + 3072, pp.u, 2 * pp.sec + 1, y, t.b);
        bulk_commit();
      }
      if (grp_ok && pp.u + (lane & 15) < g.pair_q) {
        const int col = pp.col + (lane < 16 ? 0 : g.pair_q) + (lane & 15);
        p.causal.group_sums[(static_cast<long long>(t.b) * p.causal.groups + grp) * p.causal.P + col] = total;
      }
    }
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int, float* scratch,
                                             EpiIO& io, int iter) {
    const Scratch<BN> sc(scratch);
    const int slot = iter & 1;
    const float* cst = sc.cols();
    const RopeView rs{sc.base_cos(slot), sc.base_sin(slot), sc.lane()};
    switch (p.K) {
      case 1: body<1, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, cst, rs, io); break;
      case 2: body<2, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, cst, rs, io); break;
      case 3: body<3, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, cst, rs, io); break;
      default: body<4, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, cst, rs, io); break;
    }
  }
};

// --------------------------------------------------------------- query phase, token-causal
struct EpiGateCausal {
  struct Params {
    const float* bias;
    int save_z;
    RopeEpi rope;
    CausalEpi causal;
  };
  // per warp: two alternating input sets {pre first, pre partner} (2 KiB each), then z first | z partner |
  // SH first | SH partner output blocks
  static constexpr int kStageBytes = 8192;
  static constexpr int kSmemBytes = 0;
  static constexpr bool kStager = true;
  template <int BN>
  using Scratch = PairScratch<BN, 1, 4, 0>;  // columns: bias; tile: carries of the four row groups
  template <int BN>
  static constexpr int smem_bytes() {
    return Scratch<BN>::kBytes;
  }

  static __device__ __forceinline__ void fetch_pre(const EpiMaps& maps, const TileCtx& t, const PairPos& pp,
                                                   EpiIO& io, int quarter, int lane, int set) {
    if (lane == 0) {
      uint8_t* blk = io.buf0 + set * 2048;
      mbar_expect_tx(io.bar, 2048);
      tma_load_4d(blk, &maps.in0, io.bar, pp.u, 2 * pp.sec, t.row0 + quarter * 32, t.b);
      tma_load_4d(blk + 1024, &maps.in0, io.bar, pp.u, 2 * pp.sec + 1, t.row0 + quarter * 32, t.b);
    }
  }

  template <int BN>
  static __device__ __forceinline__ uint32_t stage_cols(const Params& p, const EpiMaps& maps, const GemmGeom& g,
                                                        const TileCtx& t, int lane, float* scratch, uint64_t* bar) {
    const Scratch<BN> sc(scratch);
    const uint32_t tx = rope_stage_lane<BN>(p.rope, maps, g, t, lane, sc.lane(), bar);
    stage_paired_vector<BN>(sc.cols(), p.bias, g, t, lane);
    return tx;
  }
  template <int BN>
  static __device__ __forceinline__ void stage_tile(const Params& p, const EpiMaps&, const GemmGeom& g,
                                                    const TileCtx& t, int lane, float* scratch, int slot) {
    const Scratch<BN> sc(scratch);
    rope_stage_base<BN>(p.rope, g, t, lane, sc.base_cos(slot), sc.base_sin(slot));
    stage_carry<BN>(sc.tile(slot), p.causal, g, t, lane);
  }
  // Each warp starts the load of its first `pre` blocks while the tile's main loop is still running.
  template <int BN>
  static __device__ __forceinline__ void prologue(const Params&, const EpiMaps& maps, const GemmGeom& g,
                                                  const TileCtx& t, int warp_in_epi, int epi_tid, float*, EpiIO& io,
                                                  int) {
    const int half = warp_in_epi >> 2, quarter = (warp_in_epi + 2) & 3;
    const PairPos pp = pair_pos(g, t, 16 * half);
    if (pp.ok) fetch_pre(maps, t, pp, io, quarter, epi_tid & 31, 0);
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int, float* scratch,
                                             EpiIO& io, int iter) {
    const Scratch<BN> sc(scratch);
    const int slot = iter & 1;
    const float* bias = sc.cols();
    const float* carry = sc.tile(slot) + quarter * BN;
    const RopeView rs{sc.base_cos(slot), sc.base_sin(slot), sc.lane()};
    const int y = t.row0 + quarter * 32;
    const float inv_n = 1.f / static_cast<float>(p.causal.token_offset + y + lane + 1);
    uint8_t* out = io.buf0 + 4096;
    bool alive = true;
    int set = 0;
#pragma unroll 1
    for (int su = half; su < BN / 32; su += kEpiColSplit) {
      const PairPos pp = pair_pos(g, t, 16 * su);
      if (!pp.ok) break;  // warp-uniform
      const bool stepped = p.rope.step_of(pp.sec) != 0;
      float v[32];
      tmem_ld16<0>(tmem_acc + 16 * su, v);
      tmem_ld16<16>(tmem_acc + BN / 2 + 16 * su, v);
      if (alive) alive = mbar_wait(io.bar, io.load_phase, io.abort_flag, io.status, kStatusEpilogueTimeout);
      alive = __all_sync(0xffffffffu, alive);
      io.load_phase ^= 1u;
      const int nsu = su + kEpiColSplit;
      __syncwarp();  // every lane has finished reading the other set (previous sub-unit)
      if (alive && nsu < BN / 32) {
        const PairPos np = pair_pos(g, t, 16 * nsu);
        if (np.ok) fetch_pre(maps, t, np, io, quarter, lane, set ^ 1);
      }
      const uint8_t* in = io.buf0 + set * 2048;
      set ^= 1;
      tmem_ld_wait();
      if (t.rows_valid <= 0) continue;
      uint32_t pz1[8], pz2[8], ps1[8], ps2[8];
      round_pack16<0>(v, pz1);
      round_pack16<16>(v, pz2);
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 b1 = *reinterpret_cast<const float4*>(bias + 16 * su + i);
        const float4 b2 = *reinterpret_cast<const float4*>(bias + BN / 2 + 16 * su + i);
        const float4 k1 = *reinterpret_cast<const float4*>(carry + 16 * su + i);
        const float4 k2 = *reinterpret_cast<const float4*>(carry + BN / 2 + 16 * su + i);
        const float bb1[4] = {b1.x, b1.y, b1.z, b1.w}, bb2[4] = {b2.x, b2.y, b2.z, b2.w};
        const float kk1[4] = {k1.x, k1.y, k1.z, k1.w}, kk2[4] = {k2.x, k2.y, k2.z, k2.w};
        float pr1[4], pr2[4], c[4], s[4];
        read_block16_4(in, lane, i, pr1);
        read_block16_4(in + 1024, lane, i, pr2);
        rope_cs4<BN>(rs, stepped, quarter, lane, su, i, c, s);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float s1 = pom_hardsigmoid(v[i + e] + bb1[e]);
          const float s2 = pom_hardsigmoid(v[16 + i + e] + bb2[e]);
          v[i + e] = (s1 * c[e] - s2 * s[e]) * ((pr1[e] + kk1[e]) * inv_n);
          v[16 + i + e] = (s2 * c[e] + s1 * s[e]) * ((pr2[e] + kk2[e]) * inv_n);
        }
      }
      pack16<0>(v, ps1);
      pack16<16>(v, ps2);
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
      if (p.save_z) {
        write_block16(out, lane, pz1);
        write_block16(out + 1024, lane, pz2);
      }
      write_block16(out + 2048, lane, ps1);
      write_block16(out + 3072, lane, ps2);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (p.save_z) {
          tma_store_4d(&maps.out0, out, pp.u, 2 * pp.sec, y, t.b);
          tma_store_4d(&maps.out0, out + 1024, pp.u, 2 * pp.sec + 1, y, t.b);
        }
        tma_store_4d(&maps.out1, out + 2048, pp.u, 2 * pp.sec, y, t.b);
        tma_store_4d(&maps.out1, out + 3072, pp.u, 2 * pp.sec + 1, y, t.b);
        bulk_commit();
      }
    }
  }
};

// --------------------------------------------------------------- query phase backward, token-causal
// acc = dSH.  With z and pre re-read (maps.in0, maps.in1) and the carries of the forward group scan:
//   s = hardsigmoid(z + b), rs = R·s, H = (pre + carry) / (n + 1)
//   dz = Rᵀ·(dSH ⊙ H) ⊙ hardsigmoid'(z + b)      -> maps.out0;   dbias partial = column sums of dz
//   u  = dSH ⊙ rs / (n + 1)                       -> running sums UP the rows -> maps.out1 (`suf`) + group totals
struct EpiGateBwdCausal {
  struct Params {
    const float* bias;
    float* db_partial;
    RopeEpi rope;
    CausalEpi causal;  // carry: forward carries; group_sums: totals of u for the reverse scan
  };
  // per warp: two alternating input sets {z first, z partner, pre first, pre partner} (the set in use becomes the
  // transposition block once its rows are in registers, while the other one receives the next sub-unit's
  // blocks), then dz first | dz partner | suf first | suf partner output blocks
  static constexpr int kStageBytes = 12288;
  static constexpr int kSmemBytes = 0;
  static constexpr bool kStager = true;
  template <int BN>
  using Scratch = PairScratch<BN, 1, 4, 1>;  // columns: bias; tile: forward carries; sums: dbias
  template <int BN>
  static constexpr int smem_bytes() {
    return Scratch<BN>::kBytes;
  }

  static __device__ __forceinline__ void fetch_in(const EpiMaps& maps, const TileCtx& t, const PairPos& pp, EpiIO& io,
                                                  int quarter, int lane, int set) {
    if (lane == 0) {
      const int y = t.row0 + quarter * 32;
      uint8_t* blk = io.buf0 + set * 4096;
      mbar_expect_tx(io.bar, 4096);
      tma_load_4d(blk, &maps.in0, io.bar, pp.u, 2 * pp.sec, y, t.b);
      tma_load_4d(blk + 1024, &maps.in0, io.bar, pp.u, 2 * pp.sec + 1, y, t.b);
      tma_load_4d(blk + 2048, &maps.in1, io.bar, pp.u, 2 * pp.sec, y, t.b);
      tma_load_4d(blk + 3072, &maps.in1, io.bar, pp.u, 2 * pp.sec + 1, y, t.b);
    }
  }

  template <int BN>
  static __device__ __forceinline__ uint32_t stage_cols(const Params& p, const EpiMaps& maps, const GemmGeom& g,
                                                        const TileCtx& t, int lane, float* scratch, uint64_t* bar) {
    const Scratch<BN> sc(scratch);
    const uint32_t tx = rope_stage_lane<BN>(p.rope, maps, g, t, lane, sc.lane(), bar);
    stage_paired_vector<BN>(sc.cols(), p.bias, g, t, lane);
    return tx;
  }
  template <int BN>
  static __device__ __forceinline__ void stage_tile(const Params& p, const EpiMaps&, const GemmGeom& g,
                                                    const TileCtx& t, int lane, float* scratch, int slot) {
    const Scratch<BN> sc(scratch);
    rope_stage_base<BN>(p.rope, g, t, lane, sc.base_cos(slot), sc.base_sin(slot));
    stage_carry<BN>(sc.tile(slot), p.causal, g, t, lane);
  }
  // Each warp starts the load of its first input blocks while the tile's main loop is still running.
  template <int BN>
  static __device__ __forceinline__ void prologue(const Params&, const EpiMaps& maps, const GemmGeom& g,
                                                  const TileCtx& t, int warp_in_epi, int epi_tid, float*, EpiIO& io,
                                                  int) {
    const int half = warp_in_epi >> 2, quarter = (warp_in_epi + 2) & 3;
    const PairPos pp = pair_pos(g, t, 16 * half);
    if (pp.ok) fetch_in(maps, t, pp, io, quarter, epi_tid & 31, 0);
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int,
                                             float* scratch, EpiIO& io, int iter) {
    const Scratch<BN> sc(scratch);
    const int slot = iter & 1;
    float* buf_b = sc.sums(slot);
    const float* bias = sc.cols();
    const float* carry = sc.tile(slot) + quarter * BN;
    const RopeView rs{sc.base_cos(slot), sc.base_sin(slot), sc.lane()};
    const int y = t.row0 + quarter * 32;
    const int grp = (t.row0 >> 5) + quarter;
    const bool grp_ok = grp < p.causal.groups && t.rows_valid > 0;
    const float inv_n = 1.f / static_cast<float>(p.causal.token_offset + y + lane + 1);
    uint8_t* out = io.buf0 + 8192;
    bool alive = true;
    int set = 0;
#pragma unroll 1
    for (int su = half; su < BN / 32; su += kEpiColSplit) {
      float* b1p = buf_b + quarter * BN + 16 * su;
      const PairPos pp = pair_pos(g, t, 16 * su);
      const bool stepped = p.rope.step_of(pp.sec) != 0;
      if (!pp.ok) {  // warp-uniform
        if (lane < 16) b1p[lane] = 0.f;
        else b1p[BN / 2 + lane - 16] = 0.f;
        continue;
      }
      float v[32], z[32];
      tmem_ld16<0>(tmem_acc + 16 * su, v);
      tmem_ld16<16>(tmem_acc + BN / 2 + 16 * su, v);
      if (alive) alive = mbar_wait(io.bar, io.load_phase, io.abort_flag, io.status, kStatusEpilogueTimeout);
      alive = __all_sync(0xffffffffu, alive);
      io.load_phase ^= 1u;
      // the other set was last touched (as the transposition block) one sub-unit ago by every lane: refill it
      const int nsu = su + kEpiColSplit;
      __syncwarp();
      if (alive && nsu < BN / 32) {
        const PairPos np = pair_pos(g, t, 16 * nsu);
        if (np.ok) fetch_in(maps, t, np, io, quarter, lane, set ^ 1);
      }
      uint8_t* in = io.buf0 + set * 4096;
      set ^= 1;
      read_block16<0>(in, lane, z);
      read_block16<16>(in + 1024, lane, z);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 b1 = *reinterpret_cast<const float4*>(bias + 16 * su + i);
        const float4 b2 = *reinterpret_cast<const float4*>(bias + BN / 2 + 16 * su + i);
        const float4 k1 = *reinterpret_cast<const float4*>(carry + 16 * su + i);
        const float4 k2 = *reinterpret_cast<const float4*>(carry + BN / 2 + 16 * su + i);
        const float bb1[4] = {b1.x, b1.y, b1.z, b1.w}, bb2[4] = {b2.x, b2.y, b2.z, b2.w};
        const float kk1[4] = {k1.x, k1.y, k1.z, k1.w}, kk2[4] = {k2.x, k2.y, k2.z, k2.w};
        float pr1[4], pr2[4], c[4], s[4];
        read_block16_4(in + 2048, lane, i, pr1);
        read_block16_4(in + 3072, lane, i, pr2);
        rope_cs4<BN>(rs, stepped, quarter, lane, su, i, c, s);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float zz1 = z[i + e] + bb1[e], zz2 = z[16 + i + e] + bb2[e];
          const float s1 = pom_hardsigmoid(zz1), s2 = pom_hardsigmoid(zz2);
          const float d1 = v[i + e], d2 = v[16 + i + e];
          const float g1 = d1 * ((pr1[e] + kk1[e]) * inv_n), g2 = d2 * ((pr2[e] + kk2[e]) * inv_n);
          v[i + e] = d1 * (s1 * c[e] - s2 * s[e]) * inv_n;  // gradient of the running sum this token closes
          v[16 + i + e] = d2 * (s2 * c[e] + s1 * s[e]) * inv_n;
          z[i + e] = (g1 * c[e] + g2 * s[e]) * pom_hardsigmoid_grad(zz1);  // dz
          z[16 + i + e] = (g2 * c[e] - g1 * s[e]) * pom_hardsigmoid_grad(zz2);
        }
      }
      // rows past the end of the batch carry dSH = 0: they add nothing to the sums
      __syncwarp();                 // every lane has read its z and pre rows: the input set becomes the
      tr_write_row(in, lane, v);    // transposition block
      uint32_t pk1[8], pk2[8];
      pack16<0>(z, pk1);
      pack16<16>(z, pk2);
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
      write_block16(out, lane, pk1);
      write_block16(out + 1024, lane, pk2);
      const float total = scan_column<true>(in, out + 2048, lane);
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && t.rows_valid > 0) {
        tma_store_4d(&maps.out0, out, pp.u, 2 * pp.sec, y, t.b);
        tma_store_4d(&maps.out0, out + 1024, pp.u, 2 * pp.sec + 1, y, t.b);
        tma_store_4d(&maps.out1, out + 2048, pp.u, 2 * pp.sec, y, t.b);
        tma_store_4d(&maps.out1, out + 3072, pp.u, 2 * pp.sec + 1, y, t.b);
        bulk_commit();
      }
      if (grp_ok && pp.u + (lane & 15) < g.pair_q) {
        const int col = pp.col + (lane < 16 ? 0 : g.pair_q) + (lane & 15);
        p.causal.group_sums[(static_cast<long long>(t.b) * p.causal.groups + grp) * p.causal.P + col] = total;
      }
      warp_colsum32(z, lane);
      if (lane < 16) b1p[lane] = z[0];
      else b1p[BN / 2 + lane - 16] = z[0];
    }
    if (!tail_last_warp(io, slot, lane)) return;
    for (int c = lane; c < BN; c += 32) {
      bool ok;
      const int col = paired_col<BN>(g, t, c, &ok);
      if (ok && t.rows_valid > 0) {
        const long long o = (static_cast<long long>(t.b) * g.m_tiles_per_batch + t.mt) * p.causal.P + col;
        p.db_partial[o] = (buf_b[c] + buf_b[BN + c]) + (buf_b[2 * BN + c] + buf_b[3 * BN + c]);
      }
    }
  }
};

}  // namespace pomk
