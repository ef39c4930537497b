// Epilogues of the tcgen05 GEMM engine.
//
// Each epilogue warp owns 32 accumulator rows (one per lane) and walks its share of
// the tile 32 columns at a time (tcgen05.ld 32x32b.x32).
//
//  * Per-column constants (polynomial coefficients, gate bias, aggregated state H) are
//    staged in shared memory once per tile by `prologue`, which runs while the tile's
//    main loop is still in flight, and are read back with broadcast 128-bit loads.
//  * bf16 outputs leave through shared memory: the warp writes its 32 x 32 block (2 KiB,
//    64-byte swizzle) and one lane hands it to the TMA engine as a tiled bulk store.  The
//    store is clipped by the tensor map, so rows past the end of a batch and columns past
//    the end of the matrix need no predicate, and the load/store unit sees 4 wavefronts
//    per 512 bytes instead of 32.  Saved activations that the backward epilogue re-reads
//    come in the same way (tiled bulk load into the warp's staging buffer).
#pragma once
#include "gemm_sm100.cuh"

namespace pomk {

// 16-byte piece j (0..3) of row `lane` inside a 32-row x 64-byte block stored with the 64-byte swizzle.
__device__ __forceinline__ uint32_t swz64(int lane, int j) { return lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4); }

// Hands the warp's 32 x 32 bf16 block (row `lane` = pk) to the TMA engine.  `pending_ok` is how many of
// this lane-0's earlier bulk stores may still be reading shared memory: 1 when the caller alternates two
// buffers, 0 when it reuses one.
template <int PENDING_OK>
__device__ __forceinline__ void store_block(uint8_t* buf, const CUtensorMap* map, const uint32_t (&pk)[16], int lane,
                                            int x, int y, int z) {
  if (lane == 0) bulk_wait_read<PENDING_OK>();
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(buf + swz64(lane, j)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
  fence_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_3d(map, buf, x, y, z);
    bulk_commit();
  }
}

// Reads row `lane` of a 32 x 32 bf16 block that a bulk load placed in `buf`.
__device__ __forceinline__ void read_block(const uint8_t* buf, int lane, float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 q = *reinterpret_cast<const uint4*>(buf + swz64(lane, j));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[8 * j + 2 * e] = __uint_as_float(w[e] << 16);
      v[8 * j + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
  }
}

// Round 32 fp32 values to bf16 in place (v keeps the rounded values as fp32) and keep the packed form.
__device__ __forceinline__ void round_pack32(float (&v)[32], uint32_t (&pk)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    v[2 * j] = __uint_as_float(pk[j] << 16);
    v[2 * j + 1] = __uint_as_float(pk[j] & 0xffff0000u);
  }
}

__device__ __forceinline__ void pack32(const float (&v)[32], uint32_t (&pk)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
}

// Branch-free form of clamp(leaky_relu(x, 0.01), -0.1, 6).
__device__ __forceinline__ float act_fast(float x) { return fminf(fmaxf(x, fmaxf(0.01f * x, -0.1f)), 6.f); }

// sum_{i<K} c_i a^(i+1) in Horner form; coefficients of column j live at cst[i * BN + j].
template <int KT, int BN>
__device__ __forceinline__ void poly4(const float* cst, int K, const float (&a)[4], float (&out)[4]) {
  const int top = KT > 0 ? KT : K;
  float4 c = *reinterpret_cast<const float4*>(cst + (top - 1) * BN);
  float r[4] = {c.x, c.y, c.z, c.w};
  if constexpr (KT > 0) {
#pragma unroll
    for (int i = KT - 2; i >= 0; --i) {
      c = *reinterpret_cast<const float4*>(cst + i * BN);
      r[0] = fmaf(r[0], a[0], c.x), r[1] = fmaf(r[1], a[1], c.y), r[2] = fmaf(r[2], a[2], c.z), r[3] = fmaf(r[3], a[3], c.w);
    }
  } else {
    for (int i = K - 2; i >= 0; --i) {
      c = *reinterpret_cast<const float4*>(cst + i * BN);
      r[0] = fmaf(r[0], a[0], c.x), r[1] = fmaf(r[1], a[1], c.y), r[2] = fmaf(r[2], a[2], c.z), r[3] = fmaf(r[3], a[3], c.w);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) out[e] = r[e] * a[e];
}

// --------------------------------------------------------------- plain store
struct EpiStore {
  struct Params {
    void* C;                 // fp32 modes only (bf16 output goes through maps.out0)
    long long ldc;           // elements
    long long batch_stride;  // elements between batches
    int mode;                // 0: bf16 store, 1: fp32 store, 2: fp32 atomic add (split-K)
    float alpha;
    int act;                 // bf16 store only: 0 none, 1 exact GELU 0.5 x (1 + erf(x / sqrt 2))
    const __nv_bfloat16* residual;  // bf16 store only: added after the activation (row stride ldr), or null
    long long ldr;
  };
  static constexpr int kSmemBytes = 0;
  static constexpr int kStageBytes = kEpiStageBytes;
  static constexpr bool kStager = false;
  template <int BN>
  static constexpr int smem_bytes() { return kSmemBytes; }

  template <int BN>
  static __device__ __forceinline__ void prologue(const Params&, const EpiMaps&, const GemmGeom&, const TileCtx&, int,
                                                  int, float*, EpiIO&, int) {}

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int, float*,
                                             EpiIO& io, int) {
    const int row = quarter * 32 + lane;
    const bool row_ok = row < t.rows_valid;
    const long long off = static_cast<long long>(t.b) * p.batch_stride + static_cast<long long>(t.row0 + row) * p.ldc;
    int flip = 0;
#pragma unroll 1
    for (int c = half; c < BN / 32; c += kEpiColSplit) {
      const int col = t.col0 + c * 32;
      if (col >= g.n_cols) break;  // warp-uniform
      float v[32];
      tmem_ld32(tmem_acc + c * 32, v);
      tmem_ld_wait();
      if (p.alpha != 1.f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
      }
      if (p.mode == 0) {
        if (t.rows_valid <= 0) continue;
        if (p.act == 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.5f * v[i] * (1.f + erff(v[i] * 0.70710678118654752f));
        }
        if (p.residual && row_ok) {
          const __nv_bfloat16* r = p.residual + (static_cast<long long>(t.b) * g.rows_per_batch + t.row0 + row) * p.ldr + col;
          const int left = g.n_cols - col;
          if (left >= 32 && (reinterpret_cast<uintptr_t>(r) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 q = __ldg(reinterpret_cast<const uint4*>(r) + j);
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[8 * j + 2 * e] += __uint_as_float(w[e] << 16);
                v[8 * j + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < left) v[i] += __bfloat162float(r[i]);
          }
        }
        uint32_t pk[16];
        pack32(v, pk);
        store_block<1>(flip ? io.buf1 : io.buf0, &maps.out0, pk, lane, col, t.row0 + quarter * 32, t.b);
        flip ^= 1;
      } else {
        if (!row_ok) continue;
        const int left = g.n_cols - col;
        float* dst = reinterpret_cast<float*>(p.C) + off + col;
        const bool vec = left >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
        if (p.mode == 1) {
          if (vec) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < left) dst[i] = v[i];
          }
        } else {
          if (vec) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j), "f"(v[4 * j]),
                           "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                           : "memory");
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < left) atomicAdd(dst + i, v[i]);
          }
        }
      }
    }
  }
};

// --------------------------------------------------------------- context phase
// acc = X·Wpoᵀ.  Rounds to bf16 (what the backward pass re-reads), stores it when
// asked (maps.out0), applies act + polynomial (+ per-token weight) and reduces over the
// tile's tokens.  Per-tile column sums go to partial[(b * MT + mt), :] in a fixed
// order, so the result is run-to-run deterministic.
struct EpiCtx {
  struct Params {
    const float* coeff;       // (P, K) fp32
    int K;
    const float* row_weight;  // (B, rows_per_batch) fp32 or null (key-padding mask weights)
    int save_hp;              // store the rounded projection through maps.out0
    float* partial;           // (B * MT, P) fp32
    int P;
  };
  // two column-sum buffers [4 quarters][256] + coefficients [16][256]
  static constexpr int kSumFloats = 2 * 4 * 256;
  static constexpr int kSmemBytes = (kSumFloats + kMaxDegree * 256) * 4;
  static constexpr int kStageBytes = kEpiStageBytes;
  static constexpr bool kStager = false;
  template <int BN>
  static constexpr int smem_bytes() { return kSmemBytes; }

  template <int BN>
  static __device__ __forceinline__ void prologue(const Params& p, const EpiMaps&, const GemmGeom& g, const TileCtx& t,
                                                  int, int epi_tid, float* scratch, EpiIO&, int) {
    // The barrier that ends the previous tile's `run` guarantees nobody still reads the old constants.
    float* cst = scratch + kSumFloats;
    const int K = p.K;
    for (int idx = epi_tid; idx < BN * K; idx += kEpiThreads) {
      const int j = idx / K, i = idx - j * K;
      const int col = t.col0 + j;
      cst[i * BN + j] = col < g.n_cols ? __ldg(p.coeff + static_cast<long long>(col) * K + i) : 0.f;
    }
    named_bar_sync(kEpiBarrier, kEpiThreads);
  }

  template <int KT, int BN>
  static __device__ __forceinline__ void body(const Params& p, const EpiMaps& maps, const GemmGeom& g,
                                              const TileCtx& t, uint32_t tmem_acc, int quarter, int lane, int half,
                                              float* buf, const float* cst, EpiIO& io) {
    const int row = quarter * 32 + lane;
    const bool row_ok = row < t.rows_valid;
    const bool weighted = p.row_weight != nullptr;
    float w = 1.f;
    if (weighted)
      w = row_ok ? __ldg(p.row_weight + static_cast<long long>(t.b) * g.rows_per_batch + t.row0 + row) : 0.f;
    int flip = 0;
#pragma unroll 1
    for (int c = half; c < BN / 32; c += kEpiColSplit) {
      const int col = t.col0 + c * 32;
      if (col >= g.n_cols || !t.live) {  // warp-uniform; a skipped tile has no accumulator and adds nothing
        buf[quarter * 256 + c * 32 + lane] = 0.f;
        continue;
      }
      float v[32];
      uint32_t pk[16];
      tmem_ld32(tmem_acc + c * 32, v);
      tmem_ld_wait();
      round_pack32(v, pk);
      if (p.save_hp && t.rows_valid > 0) {
        store_block<1>(flip ? io.buf1 : io.buf0, &maps.out0, pk, lane, col, t.row0 + quarter * 32, t.b);
        flip ^= 1;
      }
      // Rows past the end of the batch were zero-filled by TMA: act(0) = 0 and poly(0) = 0, so they
      // add nothing.  Columns past n_cols have zero coefficients.
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float a[4], o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) a[e] = act_fast(v[i + e]);
        poly4<KT, BN>(cst + c * 32 + i, p.K, a, o);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[i + e] = weighted ? w * o[e] : o[e];
      }
      warp_colsum32(v, lane);
      buf[quarter * 256 + c * 32 + lane] = v[0];
    }
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int epi_tid,
                                             float* scratch, EpiIO& io, int iter) {
    float* buf = scratch + (iter & 1) * (4 * 256);
    const float* cst = scratch + kSumFloats;
    switch (p.K) {
      case 1: body<1, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, io); break;
      case 2: body<2, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, io); break;
      case 3: body<3, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, io); break;
      case 4: body<4, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, io); break;
      default: body<0, BN>(p, maps, g, t, tmem_acc, quarter, lane, half, buf, cst, io); break;
    }
    named_bar_sync(kEpiBarrier, kEpiThreads);
    for (int c = epi_tid; c < BN; c += kEpiThreads) {
      const int col = t.col0 + c;
      if (col < g.n_cols && t.rows_valid > 0) {  // a tile hanging over the end of its batch owns no slot
        const float s = (buf[c] + buf[256 + c]) + (buf[512 + c] + buf[768 + c]);
        p.partial[(static_cast<long long>(t.b) * g.m_tiles_per_batch + t.mt) * p.P + col] = s;
      }
    }
  }
};

// Stage bias and one H vector for the tile's columns: cst[0..BN) = bias, cst[BN..2BN) = H[b, :].
template <int BN>
__device__ __forceinline__ void stage_bias_h(float* cst, const float* bias, const float* hrow, const GemmGeom& g,
                                             const TileCtx& t, int epi_tid) {
  for (int j = epi_tid; j < BN; j += kEpiThreads) {
    const int col = t.col0 + j;
    const bool ok = col < g.n_cols;
    cst[j] = ok ? __ldg(bias + col) : 0.f;
    cst[BN + j] = ok ? __ldg(hrow + col) : 0.f;
  }
  named_bar_sync(kEpiBarrier, kEpiThreads);
}

// --------------------------------------------------------------- query phase
// acc = X·Wseᵀ.  z = bf16(acc) is kept for the backward pass (maps.out0); the gated
// feature s ⊙ H with s = hardsigmoid(z + bias) is written as bf16 (maps.out1), ready to
// be the A operand of the output projection.  H is one fp32 vector per sample.
struct EpiGate {
  struct Params {
    const float* bias;  // (P) fp32
    const float* H;     // (B, P) fp32
    long long h_batch_stride;
    int save_z;
  };
  static constexpr int kSmemBytes = 2 * 2 * 256 * 4;  // double-buffered {bias, H}
  static constexpr int kStageBytes = kEpiStageBytes;
  static constexpr bool kStager = false;
  template <int BN>
  static constexpr int smem_bytes() { return kSmemBytes; }

  template <int BN>
  static __device__ __forceinline__ void prologue(const Params& p, const EpiMaps&, const GemmGeom& g, const TileCtx& t,
                                                  int, int epi_tid, float* scratch, EpiIO&, int iter) {
    stage_bias_h<BN>(scratch + (iter & 1) * 512, p.bias, p.H + static_cast<long long>(t.b) * p.h_batch_stride, g, t,
                     epi_tid);
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int, float* scratch,
                                             EpiIO& io, int iter) {
    const float* cst = scratch + (iter & 1) * 512;
    const int y = t.row0 + quarter * 32;
    int flip = 0;
#pragma unroll 1
    for (int c = half; c < BN / 32; c += kEpiColSplit) {
      const int col = t.col0 + c * 32;
      if (col >= g.n_cols) break;
      float v[32];
      uint32_t pk[16];
      tmem_ld32(tmem_acc + c * 32, v);
      tmem_ld_wait();
      if (t.rows_valid <= 0) continue;
      round_pack32(v, pk);
      if (p.save_z) store_block<1>(io.buf0, &maps.out0, pk, lane, col, y, t.b);
      else flip ^= 1;  // without the z store the SH blocks alternate between the two buffers
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 bb = *reinterpret_cast<const float4*>(cst + c * 32 + i);
        const float4 hh = *reinterpret_cast<const float4*>(cst + BN + c * 32 + i);
        v[i + 0] = pom_hardsigmoid(v[i + 0] + bb.x) * hh.x;
        v[i + 1] = pom_hardsigmoid(v[i + 1] + bb.y) * hh.y;
        v[i + 2] = pom_hardsigmoid(v[i + 2] + bb.z) * hh.z;
        v[i + 3] = pom_hardsigmoid(v[i + 3] + bb.w) * hh.w;
      }
      pack32(v, pk);
      store_block<1>(flip ? io.buf0 : io.buf1, &maps.out1, pk, lane, col, y, t.b);
    }
  }
};

// --------------------------------------------------------------- query phase, backward
// acc = dY·Wo = dSH.  With z re-read from the forward pass (maps.in0):
//   s  = hardsigmoid(z + bias)
//   dH partial  = sum_rows dSH ⊙ s                      -> dh_partial[(b*MT+mt), :]
//   dz          = dSH ⊙ H ⊙ hardsigmoid'(z + bias)      -> maps.out0 (bf16), the se half of [dhp | dz]
//   dbias part. = sum_rows dz                            -> db_partial[(b*MT+mt), :]
// Rows past the end of the batch carry dSH = 0 (zero-filled A rows) and add nothing.
struct EpiGateBwd {
  struct Params {
    const float* bias;
    const float* H;
    long long h_batch_stride;
    float* dh_partial;
    float* db_partial;
    int P;
  };
  static constexpr int kSumFloats = 2 * 2 * 4 * 256;
  static constexpr int kSmemBytes = (kSumFloats + 2 * 2 * 256) * 4;
  static constexpr int kStageBytes = kEpiStageBytes;
  static constexpr bool kStager = false;
  template <int BN>
  static constexpr int smem_bytes() { return kSmemBytes; }

  // Starts the bulk load of the z block for column chunk c of tile t into buf0 (one lane per warp).
  static __device__ __forceinline__ void fetch_z(const EpiMaps& maps, const TileCtx& t, EpiIO& io, int quarter,
                                                 int lane, int col) {
    if (lane == 0) {
      mbar_expect_tx(io.bar, 32 * 64);
      tma_load_3d(io.buf0, &maps.in0, io.bar, col, t.row0 + quarter * 32, t.b);
    }
  }

  template <int BN>
  static __device__ __forceinline__ void prologue(const Params& p, const EpiMaps& maps, const GemmGeom& g,
                                                  const TileCtx& t, int warp_in_epi, int epi_tid, float* scratch,
                                                  EpiIO& io, int iter) {
    const int half = warp_in_epi >> 2, quarter = (warp_in_epi + 2) & 3;
    const int col = t.col0 + half * 32;
    if (col < g.n_cols) fetch_z(maps, t, io, quarter, epi_tid & 31, col);
    stage_bias_h<BN>(scratch + kSumFloats + (iter & 1) * 512, p.bias,
                     p.H + static_cast<long long>(t.b) * p.h_batch_stride, g, t, epi_tid);
  }

  template <int BN>
  static __device__ __forceinline__ void run(const Params& p, const EpiMaps& maps, const GemmGeom& g, const TileCtx& t,
                                             uint32_t tmem_acc, int quarter, int lane, int half, int epi_tid,
                                             float* scratch, EpiIO& io, int iter) {
    const float* cst = scratch + kSumFloats + (iter & 1) * 512;
    float* buf_h = scratch + (iter & 1) * (2 * 4 * 256);
    float* buf_b = buf_h + 4 * 256;
    bool alive = true;
#pragma unroll 1
    for (int c = half; c < BN / 32; c += kEpiColSplit) {
      const int col = t.col0 + c * 32;
      if (col >= g.n_cols) {
        buf_h[quarter * 256 + c * 32 + lane] = 0.f;
        buf_b[quarter * 256 + c * 32 + lane] = 0.f;
        continue;
      }
      float v[32], z[32];
      tmem_ld32(tmem_acc + c * 32, v);
      if (alive) alive = mbar_wait(io.bar, io.load_phase, io.abort_flag, io.status, kStatusEpilogueTimeout);
      alive = __all_sync(0xffffffffu, alive);
      io.load_phase ^= 1u;
      read_block(io.buf0, lane, z);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 bb = *reinterpret_cast<const float4*>(cst + c * 32 + i);
        const float4 hh = *reinterpret_cast<const float4*>(cst + BN + c * 32 + i);
        const float b4[4] = {bb.x, bb.y, bb.z, bb.w};
        const float h4[4] = {hh.x, hh.y, hh.z, hh.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float zz = z[i + e] + b4[e];
          const float dsh = v[i + e];
          z[i + e] = dsh * h4[e] * pom_hardsigmoid_grad(zz);  // dz
          v[i + e] = dsh * pom_hardsigmoid(zz);                // dH contribution
        }
      }
      // every lane has consumed its z row: the block may be refilled for this warp's next chunk
      __syncwarp();
      const int ncol = t.col0 + (c + kEpiColSplit) * 32;
      if (alive && c + kEpiColSplit < BN / 32 && ncol < g.n_cols) fetch_z(maps, t, io, quarter, lane, ncol);
      if (t.rows_valid > 0) {
        uint32_t pk[16];
        pack32(z, pk);
        store_block<0>(io.buf1, &maps.out0, pk, lane, col, t.row0 + quarter * 32, t.b);
      }
      warp_colsum32(v, lane);
      warp_colsum32(z, lane);
      buf_h[quarter * 256 + c * 32 + lane] = v[0];
      buf_b[quarter * 256 + c * 32 + lane] = z[0];
    }
    named_bar_sync(kEpiBarrier, kEpiThreads);
    for (int c = epi_tid; c < BN; c += kEpiThreads) {
      const int col = t.col0 + c;
      if (col < g.n_cols && t.rows_valid > 0) {
        const long long o = (static_cast<long long>(t.b) * g.m_tiles_per_batch + t.mt) * p.P + col;
        p.dh_partial[o] = (buf_h[c] + buf_h[256 + c]) + (buf_h[512 + c] + buf_h[768 + c]);
        p.db_partial[o] = (buf_b[c] + buf_b[256 + c]) + (buf_b[512 + c] + buf_b[768 + c]);
      }
    }
  }
};

}  // namespace pomk
