// Epilogues of the tcgen05 GEMM engine with rotary position embedding folded in
// (reference pom/pom_rope.py:152-235 and its use in pom/pom_rope.py:513-522).
//
// Rotation mixes channel p1 with a partner p2 = p1 + q (1-D: q = P/2; 2-D: q = P/4 inside each half of
// the channels, the first half turning with the row position and the second with the column position).
// The GEMM is launched with column pairing (GemmGeom::pair_q): a tile's left half holds BN/2 first
// channels and its right half their partners, so both members of a pair sit in the same accumulator
// rows of one CTA.  An epilogue warp walks the tile in sub-units of 16 pairs.
//
// cos/sin of (token, channel) never come from memory per element.  The tokens of a 32-row group (one
// epilogue warp = one TMEM lane quarter) either share one position or hold consecutive positions
// (RopeEpi::step, checked on the host), so
//     angle(lane, j) = angle(group base, j) + lane * step * freq_j
// and the epilogue combines, per pair,
//     the table row of the group's base position (staged one tile ahead by the stager warp: 4 groups x BN/2
//     channels), and
//     rows 0..31 of the same table (cos/sin of lane * freq_j; one 32 x 16 block per sub-unit, bulk-loaded once per
//     column block)
// with the angle-addition formulas: 4 multiply-adds instead of two table reads per element.
#pragma once
#include "epilogues.cuh"

namespace pomk {

struct RopeEpi {
  const float* cos[2];   // table of section s: (len[s], q) fp32
  const float* sin[2];
  const long long* pos;  // (rows, pos_stride) int64 token positions; section s reads column s (pos_stride 2)
  int pos_stride;
  int len[2];
  int step[2];           // 0: the tokens of an aligned 32-token group share one position; 1: consecutive
  int rotate;            // 0: no rotation at all (cos = 1, sin = 0; tables and positions are not read)
  // selections by ternary keep the kernel parameters out of local memory (no dynamically indexed arrays)
  __device__ __forceinline__ int step_of(int sec) const { return sec ? step[1] : step[0]; }
  __device__ __forceinline__ int len_of(int sec) const { return sec ? len[1] : len[0]; }
  __device__ __forceinline__ const float* cos_of(int sec) const { return sec ? cos[1] : cos[0]; }
  __device__ __forceinline__ const float* sin_of(int sec) const { return sec ? sin[1] : sin[0]; }
};

// 16-byte piece j (0..1) of row `lane` inside a 32-row x 32-byte block stored with the 32-byte swizzle.
__device__ __forceinline__ uint32_t swz32(int lane, int j) { return lane * 32 + ((j ^ ((lane >> 2) & 1)) << 4); }

// Scratch shared by the epilogue warps and the stager warp of a paired epilogue (floats unless noted):
//   [column constants: COLF x BN]                       kept while consecutive tiles of the CTA share their columns
//   [slot 0 | slot 1: tile constants TILEF x BN, cos | sin of the base position of the four row groups: 4 x BN]
//   [column-sum exchange: 2 tile parities x SUMS x 4 quarters x BN]
//   [lane tables, 1 KiB aligned: per 16-pair sub-unit a 32 x 16 cos block and a 32 x 16 sin block]
// The stager fills slot (i & 1) for tile i while the epilogue warps read slot ((i - 1) & 1).
template <int BN, int COLF, int TILEF, int SUMS>
struct PairScratch {
  static constexpr int kHalf = BN / 2;
  static constexpr int kSubs = BN / 32;
  static constexpr int kSlotFloats = TILEF * BN + 4 * BN;
  static constexpr int kSumFloats = SUMS * 4 * BN;
  static constexpr int kFloats = COLF * BN + 2 * kSlotFloats + 2 * kSumFloats;
  static constexpr int kLaneBytes = kSubs * 4096;
  static constexpr int kBytes = kFloats * 4 + kLaneBytes + 1024;  // + slack to align the lane blocks
  float* p;
  __device__ __forceinline__ explicit PairScratch(float* scratch) : p(scratch) {}
  __device__ __forceinline__ float* cols() const { return p; }
  __device__ __forceinline__ float* tile(int slot) const { return p + COLF * BN + slot * kSlotFloats; }
  __device__ __forceinline__ float* base_cos(int slot) const { return tile(slot) + TILEF * BN; }
  __device__ __forceinline__ float* base_sin(int slot) const { return base_cos(slot) + 4 * kHalf; }
  __device__ __forceinline__ float* sums(int parity) const { return p + COLF * BN + 2 * kSlotFloats + parity * kSumFloats; }
  __device__ __forceinline__ uint8_t* lane() const {
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p + kFloats) + 1023) & ~uintptr_t(1023));
  }
};

// What an epilogue warp needs of the rotary constants of its tile.
struct RopeView {
  const float* base_cos;  // [4 quarters][BN/2]
  const float* base_sin;
  const uint8_t* lane;
};

// Stager warp: starts the bulk loads of the lane tables of the tile's columns on `bar`; returns their bytes.
template <int BN>
__device__ __forceinline__ uint32_t rope_stage_lane(const RopeEpi& r, const EpiMaps& maps, const GemmGeom& g,
                                                    const TileCtx& t, int lane, uint8_t* lane_tab, uint64_t* bar) {
  if (!r.rotate) return 0;
  uint32_t bytes = 0;
  for (int su = 0; su < BN / 32; ++su) {
    const PairPos pp = pair_pos(g, t, 16 * su);
    if (!pp.ok || r.step_of(pp.sec) == 0) continue;  // no pairs, or one position per row group: no lane table
    if (lane == 0) {
      tma_load_2d(lane_tab + su * 4096, &maps.lane[2 * pp.sec], bar, pp.u, 0);
      tma_load_2d(lane_tab + su * 4096 + 2048, &maps.lane[2 * pp.sec + 1], bar, pp.u, 0);
    }
    bytes += 4096u;
  }
  return bytes;
}

// Stager warp: cos / sin of the base position of the tile's four 32-row groups for its BN/2 pairs, four pairs per
// load (pair_q and the tile's first pair are multiples of 4, the tables 16-byte aligned: the lane-table tensor maps
// have the same needs).
template <int BN>
__device__ __forceinline__ void rope_stage_base(const RopeEpi& r, const GemmGeom& g, const TileCtx& t, int lane,
                                                float* base_cos, float* base_sin) {
  constexpr int kHalf = BN / 2;
  constexpr int kVec = kHalf / 4;  // float4 per row group
  long long pos[4][2];  // [row group][section]; the host validates positions: the clamp only keeps reads inside the table
#pragma unroll
  for (int quarter = 0; quarter < 4; ++quarter) {
    const int n = t.row0 + 32 * quarter;
#pragma unroll
    for (int sec = 0; sec < 2; ++sec) {
      long long p = 0;
      if (r.rotate && n < g.rows_per_batch && (sec == 0 || r.pos_stride == 2))
        p = __ldg(r.pos + static_cast<long long>(n) * r.pos_stride + sec);
      const long long len = r.len_of(sec);
      pos[quarter][sec] = p < 0 ? 0 : (p >= len ? len - 1 : p);
    }
  }
  static_assert((4 * kVec) % 32 == 0, "tile width");
#pragma unroll
  for (int k = 0; k < 4 * kVec / 32; ++k) {
    const int idx = lane + 32 * k;
    const int quarter = idx / kVec, j = (idx - quarter * kVec) * 4;
    const int n = t.row0 + 32 * quarter;
    const PairPos pp = pair_pos(g, t, j);
    float4 c = make_float4(1.f, 1.f, 1.f, 1.f), s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r.rotate && n < g.rows_per_batch && pp.ok) {
      const int which = r.pos_stride == 2 ? pp.sec : 0;
      const long long p0 = quarter == 0 ? pos[0][0] : quarter == 1 ? pos[1][0] : quarter == 2 ? pos[2][0] : pos[3][0];
      const long long p1 = quarter == 0 ? pos[0][1] : quarter == 1 ? pos[1][1] : quarter == 2 ? pos[2][1] : pos[3][1];
      const long long p = which ? p1 : p0;
      c = __ldg(reinterpret_cast<const float4*>(r.cos_of(pp.sec) + p * g.pair_q + pp.u));
      s = __ldg(reinterpret_cast<const float4*>(r.sin_of(pp.sec) + p * g.pair_q + pp.u));
    }
    *reinterpret_cast<float4*>(base_cos + 4 * idx) = c;
    *reinterpret_cast<float4*>(base_sin + 4 * idx) = s;
  }
}

// Every epilogue warp, when its entries of the column-sum exchange buffers of this tile are written: returns true in
// the warp that arrives last, which then adds the four quarters up and owns the buffers until it returns from run().
__device__ __forceinline__ bool tail_last_warp(EpiIO& io, int parity, int lane) {
  __syncwarp();
  int old = 0;
  if (lane == 0) {
    __threadfence_block();
    old = atomicAdd(&io.tail_count[parity], 1);
  }
  old = __shfl_sync(0xffffffffu, old, 0);
  if (old != kEpiWarps - 1) return false;
  if (lane == 0) io.tail_count[parity] = 0;
  __threadfence_block();
  return true;
}

// cos/sin of this lane's token for pairs [16 su + i, 16 su + i + 4) of the tile.
template <int BN>
__device__ __forceinline__ void rope_cs4(const RopeView& rs, bool stepped, int quarter, int lane, int su, int i,
                                         float (&c)[4], float (&s)[4]) {
  const float4 C0 = *reinterpret_cast<const float4*>(rs.base_cos + quarter * (BN / 2) + 16 * su + i);
  const float4 S0 = *reinterpret_cast<const float4*>(rs.base_sin + quarter * (BN / 2) + 16 * su + i);
  if (stepped) {
    const uint8_t* blk = rs.lane + su * 4096;
    const float4 cl = *reinterpret_cast<const float4*>(blk + swz64(lane, i >> 2));
    const float4 sl = *reinterpret_cast<const float4*>(blk + 2048 + swz64(lane, i >> 2));
    c[0] = C0.x * cl.x - S0.x * sl.x, s[0] = S0.x * cl.x + C0.x * sl.x;
    c[1] = C0.y * cl.y - S0.y * sl.y, s[1] = S0.y * cl.y + C0.y * sl.y;
    c[2] = C0.z * cl.z - S0.z * sl.z, s[2] = S0.z * cl.z + C0.z * sl.z;
    c[3] = C0.w * cl.w - S0.w * sl.w, s[3] = S0.w * cl.w + C0.w * sl.w;
  } else {
    c[0] = C0.x, c[1] = C0.y, c[2] = C0.z, c[3] = C0.w;
    s[0] = S0.x, s[1] = S0.y, s[2] = S0.z, s[3] = S0.w;
  }
}

// Global column of tile column c (left half: first channels, right half: partners) and whether it exists.
template <int BN>
__device__ __forceinline__ int paired_col(const GemmGeom& g, const TileCtx& t, int c, bool* ok) {
  const PairPos pp = pair_pos(g, t, c < BN / 2 ? c : c - BN / 2);
  *ok = pp.ok;
  return pp.col + (c < BN / 2 ? 0 : g.pair_q);
}

// Round 16 fp32 values v[OFF..OFF+16) to bf16 in place and keep the packed form.
template <int OFF>
__device__ __forceinline__ void round_pack16(float (&v)[32], uint32_t (&pk)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    pk[j] = pack_bf16x2(v[OFF + 2 * j], v[OFF + 2 * j + 1]);
    v[OFF + 2 * j] = __uint_as_float(pk[j] << 16);
    v[OFF + 2 * j + 1] = __uint_as_float(pk[j] & 0xffff0000u);
  }
}
template <int OFF>
__device__ __forceinline__ void pack16(const float (&v)[32], uint32_t (&pk)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) pk[j] = pack_bf16x2(v[OFF + 2 * j], v[OFF + 2 * j + 1]);
}
// Row `lane` of a 32 x 16 bf16 block (32-byte swizzle) <- pk.
__device__ __forceinline__ void write_block16(uint8_t* buf, int lane, const uint32_t (&pk)[8]) {
  *reinterpret_cast<uint4*>(buf + swz32(lane, 0)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  *reinterpret_cast<uint4*>(buf + swz32(lane, 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
}
template <int OFF>
__device__ __forceinline__ void read_block16(const uint8_t* buf, int lane, float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint4 q = *reinterpret_cast<const uint4*>(buf + swz32(lane, j));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[OFF + 8 * j + 2 * e] = __uint_as_float(w[e] << 16);
      v[OFF + 8 * j + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
  }
}

// --------------------------------------------------------------- context phase with rotation
// acc = X·Wpoᵀ for 16 first channels and their 16 partners at a time: round to bf16 (saved for backward),
// activation + polynomial on both, rotate the pair by the token's angle, weigh, sum over the tile's tokens.
struct EpiCtxRope {
  struct Params {
    const float* coeff;
    int K;
    const float* row_weight;
    int save_hp;
    float* partial;
    int P;
    RopeEpi rope;
  };
  static constexpr int kMaxK = 4;
  static constexpr int kStageBytes = kEpiStageBytes;  // two alternating sets of {first, partner} 1 KiB blocks
  static constexpr int kSmemBytes = 0;
  static constexpr bool kStager = true;
  template <int BN>
  using Scratch = PairScratch<BN, kMaxK, 0, 1>;  // columns: coefficients [degree][BN]; sums: the token sums
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
                                              float* buf, const float* cst, const RopeView& rs, EpiIO& io) {
    const int row = quarter * 32 + lane;
    const bool weighted = p.row_weight != nullptr;
    float w = 1.f;
    if (weighted)
      w = row < t.rows_valid ? __ldg(p.row_weight + static_cast<long long>(t.b) * g.rows_per_batch + t.row0 + row) : 0.f;
    const int y = t.row0 + quarter * 32;
    int flip = 0;
#pragma unroll 1
    for (int su = half; su < BN / 32; su += kEpiColSplit) {
      float* b1 = buf + quarter * BN + 16 * su;
      float* b2 = b1 + BN / 2;
      const PairPos pp = pair_pos(g, t, 16 * su);
      const bool stepped = p.rope.step_of(pp.sec) != 0;
      if (!pp.ok || !t.live) {  // warp-uniform
        if (lane < 16) b1[lane] = 0.f;
        else b2[lane - 16] = 0.f;
        continue;
      }
      float v[32];  // [0, 16): first channels, [16, 32): their partners
      tmem_ld16<0>(tmem_acc + 16 * su, v);
      tmem_ld16<16>(tmem_acc + BN / 2 + 16 * su, v);
      tmem_ld_wait();
      uint32_t pk1[8], pk2[8];
      round_pack16<0>(v, pk1);
      round_pack16<16>(v, pk2);
      if (p.save_hp && t.rows_valid > 0) {
        uint8_t* blk = io.buf0 + flip * 2048;
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        write_block16(blk, lane, pk1);
        write_block16(blk + 1024, lane, pk2);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(&maps.out0, blk, pp.u, 2 * pp.sec, y, t.b);
          tma_store_4d(&maps.out0, blk + 1024, pp.u, 2 * pp.sec + 1, y, t.b);
          bulk_commit();
        }
        flip ^= 1;
      }
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
          const float r1 = f1[e] * c[e] - f2[e] * s[e];
          const float r2 = f2[e] * c[e] + f1[e] * s[e];
          v[i + e] = weighted ? w * r1 : r1;
          v[16 + i + e] = weighted ? w * r2 : r2;
        }
      }
      // rows past the end of the batch were zero-filled: act(0) = 0, poly(0) = 0, and they add nothing
      warp_colsum32(v, lane);
      if (lane < 16) b1[lane] = v[0];
      else b2[lane - 16] = v[0];
    }
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int,
                                             float* scratch, EpiIO& io, int iter) {
    const Scratch<BN> sc(scratch);
    const int slot = iter & 1;
    float* buf = sc.sums(slot);
    const float* cst = sc.cols();
    const RopeView rs{sc.base_cos(slot), sc.base_sin(slot), sc.lane()};
    switch (p.K) {
      case 1: body<1, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, rs, io); break;
      case 2: body<2, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, rs, io); break;
      case 3: body<3, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, rs, io); break;
      default: body<4, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, rs, io); break;
    }
    if (!tail_last_warp(io, slot, lane)) return;
    for (int c = lane; c < BN; c += 32) {
      bool ok;
      const int col = paired_col<BN>(g, t, c, &ok);
      if (ok && t.rows_valid > 0) {
        const float s = (buf[c] + buf[BN + c]) + (buf[2 * BN + c] + buf[3 * BN + c]);
        p.partial[(static_cast<long long>(t.b) * g.m_tiles_per_batch + t.mt) * p.P + col] = s;
      }
    }
  }
};

// Stager warp: one per-column vector (bias) for the tile's paired columns.
template <int BN>
__device__ __forceinline__ void stage_paired_vector(float* dst, const float* src, const GemmGeom& g, const TileCtx& t,
                                                    int lane) {
  for (int c = lane; c < BN; c += 32) {
    bool ok;
    const int col = paired_col<BN>(g, t, c, &ok);
    dst[c] = ok ? __ldg(src + col) : 0.f;
  }
}

// --------------------------------------------------------------- query phase with rotation
// acc = X·Wseᵀ.  z = bf16(acc) is kept for backward (maps.out0); SH = R·hardsigmoid(z + bias) ⊙ H (maps.out1).
struct EpiGateRope {
  struct Params {
    const float* bias;
    const float* H;
    long long h_batch_stride;
    int save_z;
    RopeEpi rope;
  };
  static constexpr int kStageBytes = kEpiStageBytes;  // z first | z partner | SH first | SH partner, 1 KiB each
  static constexpr int kSmemBytes = 0;
  static constexpr bool kStager = true;
  template <int BN>
  using Scratch = PairScratch<BN, 1, 1, 0>;  // columns: bias; tile: H of the tile's batch
  template <int BN>
  static constexpr int smem_bytes() {
    return Scratch<BN>::kBytes;
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
    stage_paired_vector<BN>(sc.tile(slot), p.H + static_cast<long long>(t.b) * p.h_batch_stride, g, t, lane);
  }
  template <int BN>
  static __device__ __forceinline__ void prologue(const Params&, const EpiMaps&, const GemmGeom&, const TileCtx&, int,
                                                  int, float*, EpiIO&, int) {}

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int, float* scratch,
                                             EpiIO& io, int iter) {
    const Scratch<BN> sc(scratch);
    const int slot = iter & 1;
    const float* bias = sc.cols();
    const float* hrow = sc.tile(slot);
    const RopeView rs{sc.base_cos(slot), sc.base_sin(slot), sc.lane()};
    const int y = t.row0 + quarter * 32;
#pragma unroll 1
    for (int su = half; su < BN / 32; su += kEpiColSplit) {
      const PairPos pp = pair_pos(g, t, 16 * su);
      if (!pp.ok) break;  // warp-uniform
      const bool stepped = p.rope.step_of(pp.sec) != 0;
      float v[32];
      tmem_ld16<0>(tmem_acc + 16 * su, v);
      tmem_ld16<16>(tmem_acc + BN / 2 + 16 * su, v);
      tmem_ld_wait();
      if (t.rows_valid <= 0) continue;
      uint32_t pz1[8], pz2[8], ps1[8], ps2[8];
      round_pack16<0>(v, pz1);
      round_pack16<16>(v, pz2);
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 b1 = *reinterpret_cast<const float4*>(bias + 16 * su + i);
        const float4 b2 = *reinterpret_cast<const float4*>(bias + BN / 2 + 16 * su + i);
        const float4 h1 = *reinterpret_cast<const float4*>(hrow + 16 * su + i);
        const float4 h2 = *reinterpret_cast<const float4*>(hrow + BN / 2 + 16 * su + i);
        const float bb1[4] = {b1.x, b1.y, b1.z, b1.w}, bb2[4] = {b2.x, b2.y, b2.z, b2.w};
        const float hh1[4] = {h1.x, h1.y, h1.z, h1.w}, hh2[4] = {h2.x, h2.y, h2.z, h2.w};
        float c[4], s[4];
        rope_cs4<BN>(rs, stepped, quarter, lane, su, i, c, s);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float s1 = pom_hardsigmoid(v[i + e] + bb1[e]);
          const float s2 = pom_hardsigmoid(v[16 + i + e] + bb2[e]);
          v[i + e] = (s1 * c[e] - s2 * s[e]) * hh1[e];
          v[16 + i + e] = (s2 * c[e] + s1 * s[e]) * hh2[e];
        }
      }
      pack16<0>(v, ps1);
      pack16<16>(v, ps2);
      // the previous sub-unit's stores were issued a whole sub-unit of arithmetic ago: this wait is short
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
      if (p.save_z) {
        write_block16(io.buf0, lane, pz1);
        write_block16(io.buf0 + 1024, lane, pz2);
      }
      write_block16(io.buf0 + 2048, lane, ps1);
      write_block16(io.buf0 + 3072, lane, ps2);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (p.save_z) {
          tma_store_4d(&maps.out0, io.buf0, pp.u, 2 * pp.sec, y, t.b);
          tma_store_4d(&maps.out0, io.buf0 + 1024, pp.u, 2 * pp.sec + 1, y, t.b);
        }
        tma_store_4d(&maps.out1, io.buf0 + 2048, pp.u, 2 * pp.sec, y, t.b);
        tma_store_4d(&maps.out1, io.buf0 + 3072, pp.u, 2 * pp.sec + 1, y, t.b);
        bulk_commit();
      }
    }
  }
};

// --------------------------------------------------------------- query phase with rotation, backward
// acc = dY·Wo = dSH (the B operand is the transposed output weight, K-major).  With z re-read (maps.in0):
//   s   = hardsigmoid(z + bias),  rs = R·s
//   dH partial  = sum_rows dSH ⊙ rs
//   ds  = Rᵀ·(dSH ⊙ H),  dz = ds ⊙ hardsigmoid'(z + bias)        -> maps.out0 (bf16)
//   dbias partial = sum_rows dz
struct EpiGateBwdRope {
  struct Params {
    const float* bias;
    const float* H;
    long long h_batch_stride;
    float* dh_partial;
    float* db_partial;
    int P;
    RopeEpi rope;
  };
  // per warp: the {z first, z partner} input blocks (refilled for the next sub-unit as soon as their rows are in
  // registers), then the {dz first, dz partner} output blocks.  4 KiB per warp leave room for a fourth pipeline stage.
  static constexpr int kStageBytes = 4096;
  static constexpr int kSmemBytes = 0;
  static constexpr bool kStager = true;
  template <int BN>
  using Scratch = PairScratch<BN, 1, 1, 2>;  // columns: bias; tile: H of the batch; sums: dH then dbias
  template <int BN>
  static constexpr int smem_bytes() {
    return Scratch<BN>::kBytes;
  }

  static __device__ __forceinline__ void fetch_z(const EpiMaps& maps, const TileCtx& t, const PairPos& pp, EpiIO& io,
                                                 int quarter, int lane) {
    if (lane == 0) {
      uint8_t* blk = io.buf0;
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
    stage_paired_vector<BN>(sc.tile(slot), p.H + static_cast<long long>(t.b) * p.h_batch_stride, g, t, lane);
  }
  // Each warp starts the load of its first z blocks while the tile's main loop is still running.
  template <int BN>
  static __device__ __forceinline__ void prologue(const Params&, const EpiMaps& maps, const GemmGeom& g,
                                                  const TileCtx& t, int warp_in_epi, int epi_tid, float*, EpiIO& io,
                                                  int) {
    const int half = warp_in_epi >> 2, quarter = (warp_in_epi + 2) & 3;
    const PairPos pp = pair_pos(g, t, 16 * half);
    if (pp.ok) fetch_z(maps, t, pp, io, quarter, epi_tid & 31);
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int,
                                             float* scratch, EpiIO& io, int iter) {
    const Scratch<BN> sc(scratch);
    const int slot = iter & 1;
    float* buf_h = sc.sums(slot);
    float* buf_b = buf_h + 4 * BN;
    const float* bias = sc.cols();
    const float* hrow = sc.tile(slot);
    const RopeView rs{sc.base_cos(slot), sc.base_sin(slot), sc.lane()};
    const int y = t.row0 + quarter * 32;
    uint8_t* out_blk = io.buf0 + 2048;
    bool alive = true;
#pragma unroll 1
    for (int su = half; su < BN / 32; su += kEpiColSplit) {
      float* h1p = buf_h + quarter * BN + 16 * su;
      float* b1p = buf_b + quarter * BN + 16 * su;
      const PairPos pp = pair_pos(g, t, 16 * su);
      const bool stepped = p.rope.step_of(pp.sec) != 0;
      if (!pp.ok) {  // warp-uniform
        if (lane < 16) h1p[lane] = 0.f, b1p[lane] = 0.f;
        else h1p[BN / 2 + lane - 16] = 0.f, b1p[BN / 2 + lane - 16] = 0.f;
        continue;
      }
      float v[32], z[32];
      tmem_ld16<0>(tmem_acc + 16 * su, v);
      tmem_ld16<16>(tmem_acc + BN / 2 + 16 * su, v);
      if (alive) alive = mbar_wait(io.bar, io.load_phase, io.abort_flag, io.status, kStatusEpilogueTimeout);
      alive = __all_sync(0xffffffffu, alive);
      io.load_phase ^= 1u;
      read_block16<0>(io.buf0, lane, z);
      read_block16<16>(io.buf0 + 1024, lane, z);
      // every lane holds its z rows: the blocks are refilled for this warp's next sub-unit
      const int nsu = su + kEpiColSplit;
      __syncwarp();
      if (alive && nsu < BN / 32) {
        const PairPos np = pair_pos(g, t, 16 * nsu);
        if (np.ok) fetch_z(maps, t, np, io, quarter, lane);
      }
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 b1 = *reinterpret_cast<const float4*>(bias + 16 * su + i);
        const float4 b2 = *reinterpret_cast<const float4*>(bias + BN / 2 + 16 * su + i);
        const float4 h1 = *reinterpret_cast<const float4*>(hrow + 16 * su + i);
        const float4 h2 = *reinterpret_cast<const float4*>(hrow + BN / 2 + 16 * su + i);
        const float bb1[4] = {b1.x, b1.y, b1.z, b1.w}, bb2[4] = {b2.x, b2.y, b2.z, b2.w};
        const float hh1[4] = {h1.x, h1.y, h1.z, h1.w}, hh2[4] = {h2.x, h2.y, h2.z, h2.w};
        float c[4], s[4];
        rope_cs4<BN>(rs, stepped, quarter, lane, su, i, c, s);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float zz1 = z[i + e] + bb1[e], zz2 = z[16 + i + e] + bb2[e];
          const float s1 = pom_hardsigmoid(zz1), s2 = pom_hardsigmoid(zz2);
          const float d1 = v[i + e], d2 = v[16 + i + e];
          const float g1 = d1 * hh1[e], g2 = d2 * hh2[e];  // gradient of the rotated gate
          v[i + e] = d1 * (s1 * c[e] - s2 * s[e]);          // dH contributions
          v[16 + i + e] = d2 * (s2 * c[e] + s1 * s[e]);
          z[i + e] = (g1 * c[e] + g2 * s[e]) * pom_hardsigmoid_grad(zz1);       // dz
          z[16 + i + e] = (g2 * c[e] - g1 * s[e]) * pom_hardsigmoid_grad(zz2);
        }
      }
      if (t.rows_valid > 0) {
        uint32_t pk1[8], pk2[8];
        pack16<0>(z, pk1);
        pack16<16>(z, pk2);
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
        write_block16(out_blk, lane, pk1);
        write_block16(out_blk + 1024, lane, pk2);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(&maps.out0, out_blk, pp.u, 2 * pp.sec, y, t.b);
          tma_store_4d(&maps.out0, out_blk + 1024, pp.u, 2 * pp.sec + 1, y, t.b);
          bulk_commit();
        }
      }
      warp_colsum32(v, lane);
      warp_colsum32(z, lane);
      if (lane < 16) h1p[lane] = v[0], b1p[lane] = z[0];
      else h1p[BN / 2 + lane - 16] = v[0], b1p[BN / 2 + lane - 16] = z[0];
    }
    if (!tail_last_warp(io, slot, lane)) return;
    for (int c = lane; c < BN; c += 32) {
      bool ok;
      const int col = paired_col<BN>(g, t, c, &ok);
      if (ok && t.rows_valid > 0) {
        const long long o = (static_cast<long long>(t.b) * g.m_tiles_per_batch + t.mt) * p.P + col;
        p.dh_partial[o] = (buf_h[c] + buf_h[BN + c]) + (buf_h[2 * BN + c] + buf_h[3 * BN + c]);
        p.db_partial[o] = (buf_b[c] + buf_b[BN + c]) + (buf_b[2 * BN + c] + buf_b[3 * BN + c]);
      }
    }
  }
};

}  // namespace pomk
