// Stand-alone PoM operators (HBM-bound SIMT kernels): polynomial aggregation with
// mean / weighted / causal-prefix reduction, the gated selection, their
// backward passes, optional rotary embedding in all of them, and the small
// reductions that finish the per-tile partial sums of the fused GEMM epilogues.
//
// Common traversal: grid = (column blocks, token chunks, batch); one thread owns
// VEC adjacent channels (16 bytes when alignment allows, plus their rotary
// partners) and walks the tokens of its chunk four at a time, so every global
// access is a coalesced 16-byte vector, several are in flight per thread, and every
// sum is formed in a fixed order (deterministic, no float atomics).
#include "common.cuh"
#include "gemm_launch.cuh"
#include "pom_math.cuh"
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>
#include <initializer_list>
#include <mutex>
#include <type_traits>

using namespace pomk;
using namespace pomh;

namespace {

constexpr int kChunk = 64;  // tokens per chunk
constexpr int kTB = 4;      // tokens loaded per batch of independent loads

// ------------------------------------------------------------------ element access
template <typename T, int VEC>
struct Vec {
  static __device__ __forceinline__ void ld(const T* __restrict__ p, float (&v)[VEC]) {
    if constexpr (std::is_same<T, float>::value) {
      if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int j = 0; j < VEC / 4; ++j) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(p) + j);
          v[4 * j] = f.x, v[4 * j + 1] = f.y, v[4 * j + 2] = f.z, v[4 * j + 3] = f.w;
        }
      } else if constexpr (VEC == 2) {
        const float2 f = __ldg(reinterpret_cast<const float2*>(p));
        v[0] = f.x, v[1] = f.y;
      } else {
        v[0] = __ldg(p);
      }
    } else {
      if constexpr (VEC == 8) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] = __uint_as_float(w[e] << 16);
          v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
      } else if constexpr (VEC == 2) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(p));
        v[0] = __uint_as_float(w << 16);
        v[1] = __uint_as_float(w & 0xffff0000u);
      } else {
        v[0] = __bfloat162float(*p);
      }
    }
  }
  static __device__ __forceinline__ void st(T* __restrict__ p, const float (&v)[VEC]) {
    if constexpr (std::is_same<T, float>::value) {
      if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int j = 0; j < VEC / 4; ++j)
          reinterpret_cast<float4*>(p)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      } else if constexpr (VEC == 2) {
        *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
      } else {
        p[0] = v[0];
      }
    } else {
      if constexpr (VEC == 8) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
          w[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
      } else if constexpr (VEC == 2) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
      } else {
        p[0] = __float2bfloat16_rn(v[0]);
      }
    }
  }
};

template <int VEC>
__device__ __forceinline__ void ld_f32(const float* __restrict__ p, float (&v)[VEC]) {
  Vec<float, VEC>::ld(p, v);
}

// ------------------------------------------------------------------ channel map
// One work item = VEC adjacent "first" channels.  Without rotary embedding every
// channel is a first channel.  With it, channel p1 is rotated together with its
// partner p2 (reference pom/pom_rope.py:171-180 for 1-D: p2 = p1 + P/2;
// pom/pom_rope.py:208-235 for 2-D: the first half of the channels pairs p1 with
// p1 + P/4 using the row position, the second half likewise with the column position).
struct ColMap {
  int p1, p2, j, tab_ld, which;
  bool valid;
};

__device__ __forceinline__ ColMap map_unit(int u, int P, int rope_kind) {
  ColMap m;
  m.p1 = u;
  m.p2 = u;
  m.j = u;
  m.tab_ld = 0;
  m.which = 0;
  if (rope_kind == POM_ROPE_NONE) {
    m.valid = u < P;
  } else if (rope_kind == POM_ROPE_1D) {
    const int half = P >> 1;
    m.valid = u < half;
    m.p2 = u + half;
    m.tab_ld = half;
  } else {
    const int half = P >> 1, q = P >> 2;
    m.valid = u < half;
    m.tab_ld = q;
    if (u < q) {
      m.p2 = u + q;
    } else {
      m.j = u - q;
      m.p1 = half + m.j;
      m.p2 = half + q + m.j;
      m.which = 1;
    }
  }
  return m;
}

inline int first_channels(int P, int rope_kind) { return rope_kind == POM_ROPE_NONE ? P : P / 2; }

template <int VEC>
__device__ __forceinline__ void rope_coeffs(const pom_rope& r, const ColMap& m, long long n, float (&c)[VEC],
                                            float (&s)[VEC]) {
  long long idx = r.pos[n * r.pos_stride + m.which];
  const long long len = m.which ? r.len1 : r.len0;  // the host validates positions; a bad one never reads outside
  if (len > 0) idx = idx < 0 ? 0 : (idx >= len ? len - 1 : idx);
  ld_f32<VEC>((m.which ? r.cos1 : r.cos0) + idx * m.tab_ld + m.j, c);
  ld_f32<VEC>((m.which ? r.sin1 : r.sin0) + idx * m.tab_ld + m.j, s);
}

template <int VEC, int KR>
struct Coefs {
  float c1[VEC][KR];
  float c2[VEC][KR];
  __device__ __forceinline__ void load(const float* coeff, const ColMap& m, int K, bool rope) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
      for (int i = 0; i < KR; ++i) {
        c1[e][i] = (i < K) ? __ldg(coeff + static_cast<long long>(m.p1 + e) * K + i) : 0.f;
        c2[e][i] = (rope && i < K) ? __ldg(coeff + static_cast<long long>(m.p2 + e) * K + i) : 0.f;
      }
  }
};

// Coefficients beyond K are zero, so the unrolled evaluation needs no predicate.
template <int KR>
__device__ __forceinline__ float poly_reg(float a, const float (&c)[KR]) {
  float r = c[KR - 1];
#pragma unroll
  for (int i = KR - 2; i >= 0; --i) r = fmaf(r, a, c[i]);
  return r * a;
}
// Two bf16 values packed in a word -> two fp32 values.
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

template <int KR>
__device__ __forceinline__ float poly_grad_reg(float a, const float (&c)[KR]) {
  float r = static_cast<float>(KR) * c[KR - 1];
#pragma unroll
  for (int i = KR - 2; i >= 0; --i) r = fmaf(r, a, static_cast<float>(i + 1) * c[i]);
  return r;
}

struct AggDev {
  const void* x;
  const float* coeff;
  const float* row_weight;
  float* partial;
  void* out;
  long long ldx, ld_out, token_offset;
  int B, N, P, K, chunks;
  int per_token;  // PREFIX kernel only: write each token's own (rotated) features, no running sum
  pom_rope rope;
};

// ------------------------------------------------------------------ forward: chunk sums / prefix apply
// PREFIX == false: partial[b, c, :] = sum over the chunk of w * R·poly.
// PREFIX == true : partial holds the exclusive prefix per chunk; writes out[b, n, :].
template <typename T, int VEC, int KR, bool PREFIX, bool ROPE>
__global__ void __launch_bounds__(128) agg_fwd_kernel(const AggDev a) {
  const int u = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  constexpr bool rope = ROPE;
  const ColMap m = map_unit(u, a.P, a.rope.kind);
  if (!m.valid) return;
  Coefs<VEC, KR> cf;
  cf.load(a.coeff, m, a.K, rope);
  const T* __restrict__ x = static_cast<const T*>(a.x) + static_cast<long long>(b) * a.N * a.ldx;
  T* __restrict__ out = PREFIX ? static_cast<T*>(a.out) + static_cast<long long>(b) * a.N * a.ld_out : nullptr;
  float* part = a.partial + (static_cast<long long>(b) * a.chunks + c) * a.P;
  float acc1[VEC], acc2[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    acc1[e] = (PREFIX && !a.per_token) ? part[m.p1 + e] : 0.f;
    acc2[e] = (PREFIX && rope && !a.per_token) ? part[m.p2 + e] : 0.f;
  }
  const int n0 = c * kChunk, n1 = min(a.N, n0 + kChunk);
  for (int nb = n0; nb < n1; nb += kTB) {
    float x1[kTB][VEC], x2[kTB][VEC], cs[kTB][VEC], sn[kTB][VEC], w[kTB];
#pragma unroll
    for (int q = 0; q < kTB; ++q) {
      const int n = min(nb + q, n1 - 1);
      Vec<T, VEC>::ld(x + n * a.ldx + m.p1, x1[q]);
      if (rope) {
        Vec<T, VEC>::ld(x + n * a.ldx + m.p2, x2[q]);
        rope_coeffs<VEC>(a.rope, m, n, cs[q], sn[q]);
      }
      w[q] = (!PREFIX && a.row_weight) ? __ldg(a.row_weight + static_cast<long long>(b) * a.N + n) : 1.f;
    }
#pragma unroll
    for (int q = 0; q < kTB; ++q) {
      const int n = nb + q;
      if (n >= n1) break;
      if (PREFIX && a.per_token) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc1[e] = acc2[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float f1 = poly_reg<KR>(pom_act(x1[q][e]), cf.c1[e]);
        if (rope) {
          const float f2 = poly_reg<KR>(pom_act(x2[q][e]), cf.c2[e]);
          acc1[e] += w[q] * (f1 * cs[q][e] - f2 * sn[q][e]);
          acc2[e] += w[q] * (f2 * cs[q][e] + f1 * sn[q][e]);
        } else {
          acc1[e] += w[q] * f1;
        }
      }
      if (PREFIX) {
        const float inv = a.per_token ? 1.f : 1.f / static_cast<float>(a.token_offset + n + 1);
        float o[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = acc1[e] * inv;
        Vec<T, VEC>::st(out + n * a.ld_out + m.p1, o);
        if (rope) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = acc2[e] * inv;
          Vec<T, VEC>::st(out + n * a.ld_out + m.p2, o);
        }
      }
    }
  }
  if (!PREFIX) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      part[m.p1 + e] = acc1[e];
      if (rope) part[m.p2 + e] = acc2[e];
    }
  }
}

// Exclusive scan over chunks (forward: prefix; reverse: suffix) seeded with `carry`.
__global__ void chunk_scan_kernel(float* partial, const float* carry, float* total, int chunks, int P, int reverse) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (p >= P) return;
  float* base = partial + static_cast<long long>(b) * chunks * P + p;
  float run = carry ? carry[static_cast<long long>(b) * P + p] : 0.f;
  float own = 0.f;
  for (int i0 = 0; i0 < chunks; i0 += 8) {
    float t[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int i = i0 + q;
      const int c = reverse ? chunks - 1 - i : i;
      t[q] = i < chunks ? base[static_cast<long long>(c) * P] : 0.f;
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int i = i0 + q;
      if (i < chunks) {
        const int c = reverse ? chunks - 1 - i : i;
        base[static_cast<long long>(c) * P] = run;
        run += t[q];
        own += t[q];
      }
    }
  }
  if (total) total[static_cast<long long>(b) * P + p] = own;
}

// out[b, p] = scale * sum_c partial[b, c, p] / denom[b].  Block = 32 columns x 8 chunk lanes; each
// lane adds every 8th chunk, then the 8 lane sums are combined in lane order.
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                               const float* __restrict__ denom, float scale, int chunks,
                                                               int P) {
  pomk::griddep_wait();  // launched with programmatic stream serialization
  pomk::griddep_launch();
  __shared__ float sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int p = blockIdx.x * 32 + tx;
  const int b = blockIdx.y;
  float s = 0.f;
  if (p < P) {
    const float* base = partial + static_cast<long long>(b) * chunks * P + p;
    float s0 = 0.f, s1 = 0.f;
    int c = ty;
    for (; c + 8 < chunks; c += 16) {
      s0 += base[static_cast<long long>(c) * P];
      s1 += base[static_cast<long long>(c + 8) * P];
    }
    if (c < chunks) s0 += base[static_cast<long long>(c) * P];
    s = s0 + s1;
  }
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && p < P) {
    float t = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) t += sm[q][tx];
    t *= scale;
    if (denom) {
      const float d = denom[b];
      t = d != 0.f ? t / d : 0.f;  // a sample with no valid token aggregates to zero
    }
    out[static_cast<long long>(b) * P + p] = t;
  }
}

// ------------------------------------------------------------------ backward
struct AggBwdDev {
  const void* x;
  const float* coeff;
  const float* row_weight;
  const float* denom;
  const float* dH;
  const void* dout;
  float* partial;
  void* dx;
  float* dcoeff_partial;
  long long ldx, ld_dx, ld_dout, token_offset;
  float scale;
  int B, N, P, K, chunks;
  int per_token;  // CAUSAL kernel only: dout[n] is the gradient of token n's own features (no suffix sum)
  pom_rope rope;
};

// Causal backward, pass 1: partial[b, c, :] = sum over the chunk of dout[b, n, :] / (n + 1 + offset).
template <typename T, int VEC>
__global__ void __launch_bounds__(128) causal_bwd_sum_kernel(const AggBwdDev a) {
  const int p = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  if (p >= a.P) return;
  const T* __restrict__ g = static_cast<const T*>(a.dout) + static_cast<long long>(b) * a.N * a.ld_dout + p;
  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
  const int n0 = c * kChunk, n1 = min(a.N, n0 + kChunk);
  for (int nb = n0; nb < n1; nb += kTB) {
    float v[kTB][VEC];
#pragma unroll
    for (int q = 0; q < kTB; ++q) Vec<T, VEC>::ld(g + static_cast<long long>(min(nb + q, n1 - 1)) * a.ld_dout, v[q]);
#pragma unroll
    for (int q = 0; q < kTB; ++q) {
      if (nb + q >= n1) break;
      const float inv = 1.f / static_cast<float>(a.token_offset + nb + q + 1);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(v[q][e], inv, acc[e]);
    }
  }
  float* part = a.partial + (static_cast<long long>(b) * a.chunks + c) * a.P + p;
#pragma unroll
  for (int e = 0; e < VEC; ++e) part[e] = acc[e];
}

// CAUSAL == false: the gradient reaching every token is w[b,n] * dH[b, :].
// CAUSAL == true : walk the chunk backwards; W[n] = suffix + sum_{m >= n} dout[m]/(m+1+offset).
// Either way: un-rotate, then dx = g * poly'(a) * act'(x) and the coefficient gradient sums.
template <typename T, int VEC, int KR, bool CAUSAL, bool ROPE>
__global__ void __launch_bounds__(128) agg_bwd_kernel(const AggBwdDev a) {
  const int u = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  constexpr bool rope = ROPE;
  const ColMap m = map_unit(u, a.P, a.rope.kind);
  if (!m.valid) return;
  Coefs<VEC, KR> cf;
  cf.load(a.coeff, m, a.K, rope);
  const T* __restrict__ x = static_cast<const T*>(a.x) + static_cast<long long>(b) * a.N * a.ldx;
  T* __restrict__ dx = static_cast<T*>(a.dx) + static_cast<long long>(b) * a.N * a.ld_dx;
  const T* __restrict__ dout =
      CAUSAL ? static_cast<const T*>(a.dout) + static_cast<long long>(b) * a.N * a.ld_dout : nullptr;
  float g1[VEC], g2[VEC];
  float dc1[VEC][KR], dc2[VEC][KR];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    if (CAUSAL) {
      const float* part = a.partial + (static_cast<long long>(b) * a.chunks + c) * a.P;
      g1[e] = a.per_token ? 0.f : part[m.p1 + e];
      g2[e] = (rope && !a.per_token) ? part[m.p2 + e] : 0.f;
    } else {
      g1[e] = a.dH[static_cast<long long>(b) * a.P + m.p1 + e];
      g2[e] = rope ? a.dH[static_cast<long long>(b) * a.P + m.p2 + e] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < KR; ++i) {
      dc1[e][i] = 0.f;
      dc2[e][i] = 0.f;
    }
  }
  float wb = a.scale;
  if (!CAUSAL && a.denom) {
    const float dn = a.denom[b];
    wb = dn != 0.f ? wb / dn : 0.f;
  }
  const int n0 = c * kChunk, n1 = min(a.N, n0 + kChunk);
  const int cnt = n1 - n0;
  constexpr int TBW = !ROPE ? 8 : (CAUSAL && VEC > 2) ? 2 : kTB;  // tokens in flight, as registers allow
  for (int ib = 0; ib < cnt; ib += TBW) {
    float x1[TBW][VEC], x2[TBW][VEC], cs[TBW][VEC], sn[TBW][VEC], go1[TBW][VEC], go2[TBW][VEC], w[TBW];
#pragma unroll
    for (int q = 0; q < TBW; ++q) {
      const int i = min(ib + q, cnt - 1);
      const int n = CAUSAL ? (n1 - 1 - i) : (n0 + i);
      Vec<T, VEC>::ld(x + n * a.ldx + m.p1, x1[q]);
      if (rope) {
        Vec<T, VEC>::ld(x + n * a.ldx + m.p2, x2[q]);
        rope_coeffs<VEC>(a.rope, m, n, cs[q], sn[q]);
      }
      if (CAUSAL) {
        Vec<T, VEC>::ld(dout + n * a.ld_dout + m.p1, go1[q]);
        if (rope) Vec<T, VEC>::ld(dout + n * a.ld_dout + m.p2, go2[q]);
        w[q] = 1.f;
      } else {
        w[q] = a.row_weight ? wb * __ldg(a.row_weight + static_cast<long long>(b) * a.N + n) : wb;
      }
    }
#pragma unroll
    for (int q = 0; q < TBW; ++q) {
      const int i = ib + q;
      if (i >= cnt) break;
      const int n = CAUSAL ? (n1 - 1 - i) : (n0 + i);
      if (CAUSAL) {
        const float inv = a.per_token ? 1.f : 1.f / static_cast<float>(a.token_offset + n + 1);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          g1[e] = fmaf(go1[q][e], inv, a.per_token ? 0.f : g1[e]);
          if (rope) g2[e] = fmaf(go2[q][e], inv, a.per_token ? 0.f : g2[e]);
        }
      }
      float o1[VEC], o2[VEC];
      if (!CAUSAL && w[q] == 0.f) {  // a token of weight zero: its saved projection may never have been written
#pragma unroll
        for (int e = 0; e < VEC; ++e) x1[q][e] = 0.f, x2[q][e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float d1, d2 = 0.f;
        if (rope) {
          d1 = w[q] * (g1[e] * cs[q][e] + g2[e] * sn[q][e]);
          d2 = w[q] * (g2[e] * cs[q][e] - g1[e] * sn[q][e]);
        } else {
          d1 = w[q] * g1[e];
        }
        const float av = pom_act(x1[q][e]);
        o1[e] = d1 * poly_grad_reg<KR>(av, cf.c1[e]) * pom_act_grad(x1[q][e]);
        float pw = av;
#pragma unroll
        for (int k = 0; k < KR; ++k) {
          dc1[e][k] = fmaf(d1, pw, dc1[e][k]);
          pw *= av;
        }
        if (rope) {
          const float bv = pom_act(x2[q][e]);
          o2[e] = d2 * poly_grad_reg<KR>(bv, cf.c2[e]) * pom_act_grad(x2[q][e]);
          float pv = bv;
#pragma unroll
          for (int k = 0; k < KR; ++k) {
            dc2[e][k] = fmaf(d2, pv, dc2[e][k]);
            pv *= bv;
          }
        }
      }
      Vec<T, VEC>::st(dx + n * a.ld_dx + m.p1, o1);
      if (rope) Vec<T, VEC>::st(dx + n * a.ld_dx + m.p2, o2);
    }
  }
  float* dcp = a.dcoeff_partial + (static_cast<long long>(b) * a.chunks + c) * a.P * a.K;
#pragma unroll
  for (int e = 0; e < VEC; ++e)
#pragma unroll
    for (int k = 0; k < KR; ++k)
      if (k < a.K) {
        dcp[static_cast<long long>(m.p1 + e) * a.K + k] = dc1[e][k];
        if (rope) dcp[static_cast<long long>(m.p2 + e) * a.K + k] = dc2[e][k];
      }
}

// ------------------------------------------------------------------ streamed backward
// The bf16, non-causal, no-rotary backward (the one on the fused layer path) as a staged stream: a CTA owns
// 256 channels of one sample and a run of 64-token tiles; warp 0 brings each tile's rows into a 3-deep shared
// memory ring with 512-byte bulk copies that complete on a "full" mbarrier, so the bytes in flight sit in shared
// memory (96 KiB per CTA, two CTAs per SM) instead of in registers; all 8 warps read 16 bytes per thread,
// compute, store dx straight from registers and release the stage on an "empty" mbarrier (one arrival per
// warp) — no CTA-wide barrier inside the loop.  The coefficient sums stay in registers over the whole run
// and are combined across the 8 row groups in a fixed order at the end: one partial per (sample, run).
constexpr int kStTok = 64;
constexpr int kStCols = 256;
constexpr int kStStages = 3;
constexpr int kStVec = 8;       // channels per thread (16-byte accesses): 256 threads per CTA
constexpr int kStTileBytes = kStTok * kStCols * 2;
constexpr int kStSmemBytes = kStStages * kStTileBytes + 128;  // ring + full/empty barriers + abort flag
constexpr int kStatusStreamTimeout = 201;

__device__ int g_ops_status;  // first bounded wait of an operator kernel that expired (0 = none)

__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct StreamPlan {
  int col_blocks, tiles, tiles_per_cta, splits;
};

// Enough CTAs for two per SM on every SM, each with a contiguous run of tiles.
inline StreamPlan stream_plan(int B, int N, int P) {
  StreamPlan s;
  s.col_blocks = static_cast<int>(ceil_div(P, kStCols));
  s.tiles = static_cast<int>(ceil_div(N, kStTok));
  const long long pairs = static_cast<long long>(s.col_blocks) * B;
  long long want = ceil_div(4LL * sm_count(), pairs);
  if (want < 1) want = 1;
  if (want > s.tiles) want = s.tiles;
  s.tiles_per_cta = static_cast<int>(ceil_div(s.tiles, want));
  s.splits = static_cast<int>(ceil_div(s.tiles, s.tiles_per_cta));
  return s;
}

// PROD: a ninth warp does nothing but issue the copies (fastest, but 288 threads leave 112 registers per thread,
// which the degree-3/4 variant would spill); otherwise warp 0 issues them between its own tiles.
template <int KR, int VEC, bool PROD>
__global__ void __launch_bounds__(kStCols / VEC * 8 + (PROD ? 32 : 0), 2)
agg_bwd_stream_kernel(const __grid_constant__ CUtensorMap tmx, const AggBwdDev a, int tiles_per_cta, int splits,
                      int* status) {
  extern __shared__ __align__(128) uint8_t st_smem[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(st_smem);
  uint64_t* full = reinterpret_cast<uint64_t*>(st_smem + kStStages * kStTileBytes);
  uint64_t* empty = full + kStStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kStStages);
  constexpr int kLanes = kStCols / VEC;   // threads across one row
  constexpr int kGroups = 8;              // row groups
  constexpr int kConsumers = kLanes * kGroups;
  const int tid = threadIdx.x, tx = tid % kLanes, ty = tid / kLanes;
  const int warp = tid >> 5, lane = tid & 31;
  const int p0 = blockIdx.x * kStCols, split = blockIdx.y, b = blockIdx.z;
  const int width = min(kStCols, a.P - p0);  // channels of this block (multiple of 8)
  const int tiles_total = (a.N + kStTok - 1) / kStTok;
  const int t_begin = split * tiles_per_cta;
  const int my_tiles = min(tiles_total, t_begin + tiles_per_cta) - t_begin;
  if (tid == 0) {
    for (int s = 0; s < kStStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumers / 32);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  griddep_wait();  // launched with programmatic stream serialization: the set-up above overlapped the previous kernel
  griddep_launch();

  __nv_bfloat16* dxb = static_cast<__nv_bfloat16*>(a.dx) + static_cast<long long>(b) * a.N * a.ld_dx + p0;
  // One tiled bulk load brings the whole 64-token x 256-channel tile (rows and channels past the end are
  // zero-filled): per-row bulk copies were bound by the copy engine's per-request cost, not by bandwidth.
  auto issue = [&](int i) {  // producer warp
    const int stage = i % kStStages;
    if (lane == 0) {
      mbar_expect_tx(&full[stage], static_cast<uint32_t>(kStTileBytes));
      tma_load_3d(ring + stage * kStTok * kStCols, &tmx, &full[stage], p0, (t_begin + i) * kStTok, b);
    }
    __syncwarp();
  };
  const bool consumer = !PROD || warp < kConsumers / 32;
  if (PROD && !consumer) {
    // producer warp: refill a stage as soon as every consumer warp has released it
    for (int i = 0; i < my_tiles; ++i) {
      if (i >= kStStages &&
          !mbar_wait(&empty[i % kStStages], static_cast<uint32_t>(i / kStStages - 1) & 1u, abort_flag, status,
                     kStatusStreamTimeout))
        break;
      issue(i);
    }
  }
  if (!PROD && warp == 0)
    for (int i = 0; i < kStStages - 1 && i < my_tiles; ++i) issue(i);

  const int c = tx * VEC;
  const bool live = consumer && c < width;
  // Two channels per register pair: the arithmetic of the loop is issued as packed fp32 pairs (fma.rn.f32x2 ...),
  // each the IEEE operation of its two halves, which halves its instruction count in an issue-bound kernel.
  constexpr int H = VEC / 2;
  float2 pf[H][KR], g[H], dc[H][KR];  // pf: (k + 1) * coeff[k], the factors of the polynomial's derivative
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const long long ch = p0 + c + 2 * h;
    g[h] = live ? make_float2(a.dH[static_cast<long long>(b) * a.P + ch], a.dH[static_cast<long long>(b) * a.P + ch + 1])
                : make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < KR; ++k) {
      const bool on = live && k < a.K;
      const float f = static_cast<float>(k + 1);
      pf[h][k] = make_float2(on ? f * __ldg(a.coeff + ch * a.K + k) : 0.f, on ? f * __ldg(a.coeff + (ch + 1) * a.K + k) : 0.f);
      dc[h][k] = make_float2(0.f, 0.f);
    }
  }
  float wb = a.scale;
  if (a.denom) {
    const float dn = a.denom[b];
    wb = dn != 0.f ? wb / dn : 0.f;
  }

  for (int i = 0; i < my_tiles && consumer; ++i) {
    const int stage = i % kStStages;
    if (!PROD && warp == 0) {
      // refill the stage of tile i-1 with tile i+S-1 once every warp has released it (no CTA-wide barrier)
      const int j = i + kStStages - 1;
      if (j < my_tiles) {
        if (j >= kStStages && !mbar_wait(&empty[j % kStStages], static_cast<uint32_t>(j / kStStages - 1) & 1u,
                                         abort_flag, status, kStatusStreamTimeout))
          break;
        issue(j);
      }
    }
    if (!mbar_wait(&full[stage], static_cast<uint32_t>(i / kStStages) & 1u, abort_flag, status, kStatusStreamTimeout))
      break;
    const int n0 = (t_begin + i) * kStTok;
    const int rows = min(kStTok, a.N - n0);
    if (live) {
#pragma unroll 2
      for (int r = ty; r < rows; r += kGroups) {
        const int n = n0 + r;
        float2 x[H], o[H];
        {
          const __nv_bfloat16* src = ring + (stage * kStTok + r) * kStCols + c;
          uint32_t w4[VEC / 2];
          if constexpr (VEC == 8) {
            const uint4 q = *reinterpret_cast<const uint4*>(src);
            w4[0] = q.x, w4[1] = q.y, w4[2] = q.z, w4[3] = q.w;
          } else {
            const uint2 q = *reinterpret_cast<const uint2*>(src);
            w4[0] = q.x, w4[1] = q.y;
          }
#pragma unroll
          for (int h = 0; h < H; ++h) x[h] = bf16x2_to_float2(w4[h]);
        }
        const float w = a.row_weight ? wb * __ldg(a.row_weight + static_cast<long long>(b) * a.N + n) : wb;
        if (w == 0.f) {  // a token of weight zero: its saved projection may never have been written
#pragma unroll
          for (int h = 0; h < H; ++h) x[h] = make_float2(0.f, 0.f);
        }
        const float2 w2 = make_float2(w, w);
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 d = __fmul2_rn(w2, g[h]);
          const float2 av = make_float2(pom_act(x[h].x), pom_act(x[h].y));
          float2 rr = pf[h][KR - 1];
#pragma unroll
          for (int k = KR - 2; k >= 0; --k) rr = __ffma2_rn(rr, av, pf[h][k]);
          o[h] = __fmul2_rn(__fmul2_rn(d, rr), make_float2(pom_act_grad(x[h].x), pom_act_grad(x[h].y)));
          float2 pw = av;
#pragma unroll
          for (int k = 0; k < KR; ++k) {
            dc[h][k] = __ffma2_rn(d, pw, dc[h][k]);
            if (k + 1 < KR) pw = __fmul2_rn(pw, av);
          }
        }
        {
          uint32_t pk[VEC / 2];
#pragma unroll
          for (int h = 0; h < H; ++h) pk[h] = pack_bf16x2(o[h].x, o[h].y);
          __nv_bfloat16* dst = dxb + static_cast<long long>(n) * a.ld_dx + c;
          if constexpr (VEC == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          else *reinterpret_cast<uint2*>(dst) = make_uint2(pk[0], pk[1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);  // this warp is done reading the stage
  }
  // every bulk copy issued above has been waited for: the ring is free to hold the coefficient sums
  __syncthreads();
  if (*abort_flag) return;  // a wait expired (status word set): leave the outputs incomplete rather than wrong
  float* red = reinterpret_cast<float*>(st_smem);  // [row group 1..7][value][thread of the row]
  if (ty > 0 && consumer) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
      for (int k = 0; k < KR; ++k)
        red[((ty - 1) * VEC * KR + e * KR + k) * kLanes + tx] = (e & 1) ? dc[e >> 1][k].y : dc[e >> 1][k].x;
  }
  __syncthreads();
  if (ty == 0 && live) {
    float* dcp = a.dcoeff_partial + (static_cast<long long>(b) * splits + split) * a.P * a.K;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        float s = (e & 1) ? dc[e >> 1][k].y : dc[e >> 1][k].x;
        for (int q = 0; q < kGroups - 1; ++q) s += red[(q * VEC * KR + e * KR + k) * kLanes + tx];
        if (k < a.K) dcp[static_cast<long long>(p0 + c + e) * a.K + k] = s;
      }
  }
}

// The same stream with rotary embedding: a CTA owns up to 128 first channels of one section and their 128
// rotation partners (two 256-byte bulk copies per token row: [first | partner]), a thread 4 first channels and
// their 4 partners.  The gradient reaching token n is the transposed rotation of dH by that token's angle
// (reference pom/pom_rope.py:171-180, 208-235; backward of pom_triton_rope.py:227-475).
//
// No table row is read per token.  The positions of every aligned group of 32 tokens are constant or consecutive
// (pom_rope::step0/1), so angle(token) = angle(group base) + lane * step * freq: a thread visits rows ty, ty + 8,
// ... of each 64-token tile, i.e. four lane offsets that never change, whose cos/sin it keeps in registers for the
// whole run; per tile it fetches the table rows of the two group bases (two 16-byte loads each) while the tile is
// still landing, and combines both with the angle-addition formulas.
constexpr int kStHalf = kStCols / 2;

// CAUSAL (the fused token-causal layer): tiles are one 32-token group; beside hp the ring carries `suf`, the
// running sums (up the group's rows) of the gradient of the prefix means written by the causal gate-backward
// epilogue, and the gradient of token n's features is suf[n] + carry[group] instead of w[n]·dH.
template <int KR, bool CAUSAL>
__global__ void __launch_bounds__(256, 2)
agg_bwd_stream_pair_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tms,
                           const AggBwdDev a, int tiles_per_cta, int splits, int q, int blocks_per_section,
                           int* status) {
  extern __shared__ __align__(128) uint8_t st_smem[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(st_smem);
  uint64_t* full = reinterpret_cast<uint64_t*>(st_smem + kStStages * kStTileBytes);
  uint64_t* empty = full + kStStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kStStages);
  constexpr int VEC = 4;
  constexpr int kLanes = kStHalf / VEC;  // 32 threads across one row
  constexpr int kGroups = 8;             // row groups of the CTA (not to be confused with 32-token groups)
  constexpr int kConsumers = kLanes * kGroups;
  constexpr int TT = CAUSAL ? 32 : 64;   // tokens per tile
  constexpr int kBox = TT * kStHalf;     // elements of one [TT x 128] box of the tile
  static_assert(kStTileBytes == (CAUSAL ? 4 : 2) * kBox * 2, "ring stage must hold the tile's boxes");
  const int tid = threadIdx.x, tx = tid % kLanes, ty = tid / kLanes;
  const int warp = tid >> 5, lane = tid & 31;
  const int sec = blockIdx.x / blocks_per_section;
  const int u0 = (blockIdx.x - sec * blocks_per_section) * kStHalf;  // first channel index inside the section
  const int split = blockIdx.y, b = blockIdx.z;
  const int width = min(kStHalf, q - u0);  // pairs of this block (multiple of 8)
  const int p1_0 = sec * 2 * q + u0, p2_0 = p1_0 + q;
  const int tiles_total = (a.N + TT - 1) / TT;
  const int t_begin = split * tiles_per_cta;
  const int my_tiles = min(tiles_total, t_begin + tiles_per_cta) - t_begin;
  if (tid == 0) {
    for (int s = 0; s < kStStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumers / 32);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  griddep_wait();  // launched with programmatic stream serialization: the set-up above overlapped the previous kernel
  griddep_launch();

  __nv_bfloat16* dxb = static_cast<__nv_bfloat16*>(a.dx) + static_cast<long long>(b) * a.N * a.ld_dx;
  // tiled bulk loads per tile: [TT tokens x 128 first channels], [TT x 128 partners] (and the same two boxes of suf)
  auto issue = [&](int i) {  // warp 0
    const int stage = i % kStStages;
    if (lane == 0) {
      __nv_bfloat16* dst = ring + stage * (kStTileBytes / 2);
      const int n0 = (t_begin + i) * TT;
      mbar_expect_tx(&full[stage], static_cast<uint32_t>(kStTileBytes));
      tma_load_3d(dst, &tmx, &full[stage], p1_0, n0, b);
      tma_load_3d(dst + kBox, &tmx, &full[stage], p2_0, n0, b);
      if (CAUSAL) {
        tma_load_3d(dst + 2 * kBox, &tms, &full[stage], p1_0, n0, b);
        tma_load_3d(dst + 3 * kBox, &tms, &full[stage], p2_0, n0, b);
      }
    }
    __syncwarp();
  };
  if (warp == 0)
    for (int i = 0; i < kStStages - 1 && i < my_tiles; ++i) issue(i);

  const int c = tx * VEC;
  const bool live = c < width;
  // Two channels per register pair: the arithmetic below is issued as packed fp32 pairs (fma.rn.f32x2 ...), which
  // halves its instruction count in a kernel that is bound by instruction issue.  Every packed operation is the
  // IEEE operation of its two halves.
  constexpr int H = VEC / 2;
  float2 pf1[H][KR], pf2[H][KR];  // (k + 1) * coeff[k]: the factors of the polynomial's derivative
  float2 g1[H], g2[H], dc1[H][KR], dc2[H][KR];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const long long ch1 = p1_0 + c + 2 * h, ch2 = p2_0 + c + 2 * h;
    g1[h] = g2[h] = make_float2(0.f, 0.f);
    if (live && !CAUSAL) {
      g1[h] = make_float2(a.dH[static_cast<long long>(b) * a.P + ch1], a.dH[static_cast<long long>(b) * a.P + ch1 + 1]);
      g2[h] = make_float2(a.dH[static_cast<long long>(b) * a.P + ch2], a.dH[static_cast<long long>(b) * a.P + ch2 + 1]);
    }
#pragma unroll
    for (int k = 0; k < KR; ++k) {
      const bool on = live && k < a.K;
      const float f = static_cast<float>(k + 1);
      pf1[h][k] = make_float2(on ? f * __ldg(a.coeff + ch1 * a.K + k) : 0.f, on ? f * __ldg(a.coeff + (ch1 + 1) * a.K + k) : 0.f);
      pf2[h][k] = make_float2(on ? f * __ldg(a.coeff + ch2 * a.K + k) : 0.f, on ? f * __ldg(a.coeff + (ch2 + 1) * a.K + k) : 0.f);
      dc1[h][k] = dc2[h][k] = make_float2(0.f, 0.f);
    }
  }
  float wb = a.scale;
  if (!CAUSAL && a.denom) {
    const float dn = a.denom[b];
    wb = dn != 0.f ? wb / dn : 0.f;
  }
  const bool rotate = a.rope.kind != POM_ROPE_NONE;
  const int which = a.rope.pos_stride == 2 ? sec : 0;
  const float* __restrict__ cos_t = (sec ? a.rope.cos1 : a.rope.cos0) + u0 + c;
  const float* __restrict__ sin_t = (sec ? a.rope.sin1 : a.rope.sin0) + u0 + c;
  const long long tab_len = sec ? a.rope.len1 : a.rope.len0;
  const bool stepped = rotate && (sec ? a.rope.step1 : a.rope.step0) != 0;
  // cos/sin of (lane offset * freq) for this thread's four lane offsets ty, ty + 8, ty + 16, ty + 24
  float4 cl[4], sl[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    cl[j] = make_float4(1.f, 1.f, 1.f, 1.f);
    sl[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (stepped && live) {
      long long row = ty + 8 * j;
      row = row >= tab_len ? tab_len - 1 : row;  // offsets past the table belong to tokens that do not exist
      cl[j] = __ldg(reinterpret_cast<const float4*>(cos_t + row * q));
      sl[j] = __ldg(reinterpret_cast<const float4*>(sin_t + row * q));
    }
  }
  const int token_groups = (a.N + 31) / 32;

  for (int i = 0; i < my_tiles; ++i) {
    const int stage = i % kStStages;
    if (warp == 0) {
      // refill the stage of tile i-1 with tile i+S-1 once every warp has released it (no CTA-wide barrier)
      const int j = i + kStStages - 1;
      if (j < my_tiles) {
        if (j >= kStStages && !mbar_wait(&empty[j % kStStages], static_cast<uint32_t>(j / kStStages - 1) & 1u,
                                         abort_flag, status, kStatusStreamTimeout))
          break;
        issue(j);
      }
    }
    const int n0 = (t_begin + i) * TT;
    const int rows = min(TT, a.N - n0);
    // table rows of the base positions of the tile's 32-token groups (and, causal, the group's carry), requested
    // while the tile is landing
    float4 c0[TT / 32], s0[TT / 32], kb1, kb2;
    kb1 = kb2 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int g = 0; g < TT / 32; ++g) {
      c0[g] = make_float4(1.f, 1.f, 1.f, 1.f);
      s0[g] = make_float4(0.f, 0.f, 0.f, 0.f);
      const int n = n0 + 32 * g;
      if (rotate && live && n < a.N) {
        long long idx = __ldg(a.rope.pos + static_cast<long long>(n) * a.rope.pos_stride + which);
        idx = idx < 0 ? 0 : (idx >= tab_len ? tab_len - 1 : idx);
        c0[g] = __ldg(reinterpret_cast<const float4*>(cos_t + idx * q));
        s0[g] = __ldg(reinterpret_cast<const float4*>(sin_t + idx * q));
      }
    }
    if (CAUSAL && live) {
      const float* kb = a.partial + (static_cast<long long>(b) * token_groups + (t_begin + i)) * a.P;
      kb1 = __ldg(reinterpret_cast<const float4*>(kb + p1_0 + c));
      kb2 = __ldg(reinterpret_cast<const float4*>(kb + p2_0 + c));
    }
    if (!mbar_wait(&full[stage], static_cast<uint32_t>(i / kStStages) & 1u, abort_flag, status, kStatusStreamTimeout))
      break;
    if (live) {
      const __nv_bfloat16* tile = ring + stage * (kStTileBytes / 2);
#pragma unroll
      for (int k = 0; k < TT / kGroups; ++k) {
        const int r = ty + kGroups * k;
        if (r >= rows) break;
        const int n = n0 + r;
        const int g = k >> 2, j = k & 3;
        float2 x1[H], x2[H], o1[H], o2[H], gg1[H], gg2[H];
        {
          const __nv_bfloat16* src = tile + r * kStHalf + c;
          const uint2 qa = *reinterpret_cast<const uint2*>(src);
          const uint2 qb = *reinterpret_cast<const uint2*>(src + kBox);
          x1[0] = bf16x2_to_float2(qa.x), x1[1] = bf16x2_to_float2(qa.y);
          x2[0] = bf16x2_to_float2(qb.x), x2[1] = bf16x2_to_float2(qb.y);
          if (CAUSAL) {
            const uint2 sa = *reinterpret_cast<const uint2*>(src + 2 * kBox);
            const uint2 sb = *reinterpret_cast<const uint2*>(src + 3 * kBox);
            gg1[0] = __fadd2_rn(bf16x2_to_float2(sa.x), make_float2(kb1.x, kb1.y));
            gg1[1] = __fadd2_rn(bf16x2_to_float2(sa.y), make_float2(kb1.z, kb1.w));
            gg2[0] = __fadd2_rn(bf16x2_to_float2(sb.x), make_float2(kb2.x, kb2.y));
            gg2[1] = __fadd2_rn(bf16x2_to_float2(sb.y), make_float2(kb2.z, kb2.w));
          } else {
#pragma unroll
            for (int h = 0; h < H; ++h) gg1[h] = g1[h], gg2[h] = g2[h];
          }
        }
        float w = 1.f;
        if (!CAUSAL) {
          w = a.row_weight ? wb * __ldg(a.row_weight + static_cast<long long>(b) * a.N + n) : wb;
          if (w == 0.f) {  // a token of weight zero: its saved projection may never have been written
#pragma unroll
            for (int h = 0; h < H; ++h) x1[h] = x2[h] = make_float2(0.f, 0.f);
          }
        }
        const float2 w2 = make_float2(w, w), nw2 = make_float2(-w, -w);
        const float2 C0[H] = {make_float2(c0[g].x, c0[g].y), make_float2(c0[g].z, c0[g].w)};
        const float2 S0[H] = {make_float2(s0[g].x, s0[g].y), make_float2(s0[g].z, s0[g].w)};
        const float2 nS0[H] = {make_float2(-s0[g].x, -s0[g].y), make_float2(-s0[g].z, -s0[g].w)};
        const float2 CL[H] = {make_float2(cl[j].x, cl[j].y), make_float2(cl[j].z, cl[j].w)};
        const float2 SL[H] = {make_float2(sl[j].x, sl[j].y), make_float2(sl[j].z, sl[j].w)};
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 cc = __ffma2_rn(nS0[h], SL[h], __fmul2_rn(C0[h], CL[h]));  // cos(base + lane offset)
          const float2 ss = __ffma2_rn(C0[h], SL[h], __fmul2_rn(S0[h], CL[h]));   // sin(base + lane offset)
          // transposed rotation of the incoming gradient: d1 = w (g1 cc + g2 ss), d2 = w (g2 cc - g1 ss)
          const float2 d1 = __fmul2_rn(w2, __ffma2_rn(gg2[h], ss, __fmul2_rn(gg1[h], cc)));
          const float2 d2 = __fmul2_rn(nw2, __ffma2_rn(gg1[h], ss, __fmul2_rn(make_float2(-gg2[h].x, -gg2[h].y), cc)));
          const float2 av = make_float2(pom_act(x1[h].x), pom_act(x1[h].y));
          const float2 bv = make_float2(pom_act(x2[h].x), pom_act(x2[h].y));
          float2 ra = pf1[h][KR - 1], rb = pf2[h][KR - 1];
#pragma unroll
          for (int kk = KR - 2; kk >= 0; --kk) {
            ra = __ffma2_rn(ra, av, pf1[h][kk]);
            rb = __ffma2_rn(rb, bv, pf2[h][kk]);
          }
          o1[h] = __fmul2_rn(__fmul2_rn(d1, ra), make_float2(pom_act_grad(x1[h].x), pom_act_grad(x1[h].y)));
          o2[h] = __fmul2_rn(__fmul2_rn(d2, rb), make_float2(pom_act_grad(x2[h].x), pom_act_grad(x2[h].y)));
          float2 pa = av, pb = bv;
#pragma unroll
          for (int kk = 0; kk < KR; ++kk) {
            dc1[h][kk] = __ffma2_rn(d1, pa, dc1[h][kk]);
            dc2[h][kk] = __ffma2_rn(d2, pb, dc2[h][kk]);
            if (kk + 1 < KR) {
              pa = __fmul2_rn(pa, av);
              pb = __fmul2_rn(pb, bv);
            }
          }
        }
        __nv_bfloat16* dst = dxb + static_cast<long long>(n) * a.ld_dx;
        *reinterpret_cast<uint2*>(dst + p1_0 + c) = make_uint2(pack_bf16x2(o1[0].x, o1[0].y), pack_bf16x2(o1[1].x, o1[1].y));
        *reinterpret_cast<uint2*>(dst + p2_0 + c) = make_uint2(pack_bf16x2(o2[0].x, o2[0].y), pack_bf16x2(o2[1].x, o2[1].y));
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);  // this warp is done reading the stage
  }
  // every bulk copy issued above has been waited for: the ring is free to hold the coefficient sums
  __syncthreads();
  if (*abort_flag) return;  // a wait expired (status word set): leave the outputs incomplete rather than wrong
  float* red = reinterpret_cast<float*>(st_smem);  // [row group 1..7][value][thread of the row]
  if (ty > 0) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        red[((ty - 1) * 2 * VEC * KR + e * KR + k) * kLanes + tx] = (e & 1) ? dc1[e >> 1][k].y : dc1[e >> 1][k].x;
        red[((ty - 1) * 2 * VEC * KR + VEC * KR + e * KR + k) * kLanes + tx] = (e & 1) ? dc2[e >> 1][k].y : dc2[e >> 1][k].x;
      }
  }
  __syncthreads();
  if (ty == 0 && live) {
    float* dcp = a.dcoeff_partial + (static_cast<long long>(b) * splits + split) * a.P * a.K;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        float s1 = (e & 1) ? dc1[e >> 1][k].y : dc1[e >> 1][k].x;
        float s2 = (e & 1) ? dc2[e >> 1][k].y : dc2[e >> 1][k].x;
        for (int qg = 0; qg < kGroups - 1; ++qg) {
          s1 += red[(qg * 2 * VEC * KR + e * KR + k) * kLanes + tx];
          s2 += red[(qg * 2 * VEC * KR + VEC * KR + e * KR + k) * kLanes + tx];
        }
        if (k < a.K) {
          dcp[static_cast<long long>(p1_0 + c + e) * a.K + k] = s1;
          dcp[static_cast<long long>(p2_0 + c + e) * a.K + k] = s2;
        }
      }
  }
}

// Sections and first channels per section of the paired stream (0 sections: not a rotary call).
struct StreamPairs {
  int sections, q;
};
inline StreamPairs stream_pairs(const pom_agg_bwd_args* a) {
  if (a->rope.kind == POM_ROPE_1D) return StreamPairs{1, a->P / 2};
  if (a->rope.kind == POM_ROPE_2D) return StreamPairs{2, a->P / 4};
  if (a->causal == 3) return StreamPairs{1, a->P / 2};  // no rotation: first half | second half
  return StreamPairs{0, 0};
}
inline StreamPlan stream_plan_rope(int B, int N, const StreamPairs& sp, int tile_tokens = kStTok) {
  StreamPlan s;
  s.tiles = static_cast<int>(ceil_div(N, tile_tokens));
  s.col_blocks = sp.sections * static_cast<int>(ceil_div(sp.q, kStHalf));
  const long long pairs = static_cast<long long>(s.col_blocks) * B;
  long long want = ceil_div(4LL * sm_count(), pairs);
  // one coefficient-gradient partial per (sample, run of tiles): never more runs than the caller's capacity of
  // pom_agg_chunks(N) slots per sample, whatever the tile length
  const long long cap = ceil_div(N, kChunk);
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  if (want > s.tiles) want = s.tiles;
  s.tiles_per_cta = static_cast<int>(ceil_div(s.tiles, want));
  s.splits = static_cast<int>(ceil_div(s.tiles, s.tiles_per_cta));
  return s;
}

bool stream_bwd_rope_eligible(const pom_agg_bwd_args* a) {
  // non-causal degrees 3 and 4 would spill the paired register state: they take the chunked kernel (the fused
  // token-causal form, causal == 3, has no other kernel and accepts the spills)
  if (a->dtype != POM_BF16 || (a->causal != 0 && a->causal != 3) || a->K > (a->causal == 3 ? 4 : 2)) return false;
  const StreamPairs sp = stream_pairs(a);
  if (sp.sections == 0 || sp.q % 8 || sp.q * 2 * sp.sections != a->P) return false;
  if (a->causal == 3 && (!a->dout || !a->partial || a->ld_dout % 8 || !aligned16(a->dout))) return false;
  if (a->rope.kind == POM_ROPE_NONE)
    return a->ldx % 8 == 0 && a->ld_dx % 8 == 0 && aligned16(a->x) && aligned16(a->dx);
  if (a->rope.pos_stride != sp.sections || a->rope.len0 < 1 || (sp.sections == 2 && a->rope.len1 < 1)) return false;
  if ((a->rope.step0 != 0 && a->rope.step0 != 1) || (sp.sections == 2 && a->rope.step1 != 0 && a->rope.step1 != 1))
    return false;  // arbitrary positions: the chunked kernel reads a table row per token
  if (a->ldx % 8 || a->ld_dx % 8 || !aligned16(a->x) || !aligned16(a->dx)) return false;
  for (const void* t : {static_cast<const void*>(a->rope.cos0), static_cast<const void*>(a->rope.sin0),
                        static_cast<const void*>(a->rope.cos1), static_cast<const void*>(a->rope.sin1)})
    if (t && !aligned16(t)) return false;
  return true;
}

// (channels, tokens, samples) view of a bf16 activation for tiled bulk loads of box_cols x box_rows tiles
// (row-major in shared memory, no swizzle).
int stream_tile_map(CUtensorMap* m, const void* base, int64_t P, int64_t N, int64_t B, int64_t ld, int box_cols,
                    int box_rows) {
  uint64_t dims[3] = {static_cast<uint64_t>(P), static_cast<uint64_t>(N), static_cast<uint64_t>(B)};
  uint64_t str[2] = {static_cast<uint64_t>(ld), static_cast<uint64_t>(ld) * static_cast<uint64_t>(N)};
  uint32_t box[3] = {static_cast<uint32_t>(box_cols), static_cast<uint32_t>(box_rows), 1};
  return make_map(m, base, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

bool stream_bwd_eligible(const pom_agg_bwd_args* a) {
  return a->dtype == POM_BF16 && a->causal == 0 && a->rope.kind == POM_ROPE_NONE && a->K <= 4 && a->P % 8 == 0 &&
         a->ldx % 8 == 0 && a->ld_dx % 8 == 0 && aligned16(a->x) && aligned16(a->dx);
}

int* ops_status_ptr() {
  // one address per device (the symbol is per device)
  static std::mutex mu;
  static int* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_ops_status) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

// ------------------------------------------------------------------ selection
struct SelDev {
  const void* z;
  const float* bias;
  const void* H;
  void* sh;
  const void* dsh;
  void* dz;
  float* dbias_partial;
  float* dh_partial;
  void* dh_tok;
  long long ld_z, ld_h, ld_sh, ld_dsh, ld_dz, ld_dh;
  int B, T, P, chunks, h_per_token, activated;
  const float* row_denom;  // per-token H only: H[b,t,:] is divided by row_denom[b*T + t] (0 -> the row counts as 0)
  pom_rope rope;
};

template <typename T, int VEC, bool BWD, bool ROPE>
__global__ void __launch_bounds__(128) select_kernel(const SelDev a) {
  const int u = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  constexpr bool rope = ROPE;
  const ColMap m = map_unit(u, a.P, a.rope.kind);
  if (!m.valid) return;
  const long long rowb = static_cast<long long>(b) * a.T;
  const T* __restrict__ z = static_cast<const T*>(a.z) + rowb * a.ld_z;
  float b1[VEC], b2[VEC], hb1[VEC], hb2[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    b1[e] = a.activated ? 0.f : a.bias[m.p1 + e];
    b2[e] = (rope && !a.activated) ? a.bias[m.p2 + e] : 0.f;
    hb1[e] = hb2[e] = 0.f;
    if (!a.h_per_token) {
      const float* H = static_cast<const float*>(a.H) + static_cast<long long>(b) * a.P;
      hb1[e] = H[m.p1 + e];
      if (rope) hb2[e] = H[m.p2 + e];
    }
  }
  float accH1[VEC], accH2[VEC], accB1[VEC], accB2[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) accH1[e] = accH2[e] = accB1[e] = accB2[e] = 0.f;
  const int t0 = c * kChunk, t1 = min(a.T, t0 + kChunk);
  constexpr int TB = 2;
  for (int tb = t0; tb < t1; tb += TB) {
    float z1[TB][VEC], z2[TB][VEC], cs[TB][VEC], sn[TB][VEC], h1[TB][VEC], h2[TB][VEC], g1[TB][VEC], g2[TB][VEC];
    float rs[TB];
#pragma unroll
    for (int q = 0; q < TB; ++q) rs[q] = 1.f;
#pragma unroll
    for (int q = 0; q < TB; ++q) {
      const int t = min(tb + q, t1 - 1);
      Vec<T, VEC>::ld(z + t * a.ld_z + m.p1, z1[q]);
      if (rope) {
        Vec<T, VEC>::ld(z + t * a.ld_z + m.p2, z2[q]);
        rope_coeffs<VEC>(a.rope, m, t, cs[q], sn[q]);
      }
      if (a.h_per_token) {
        const T* __restrict__ H = static_cast<const T*>(a.H) + (rowb + t) * a.ld_h;
        Vec<T, VEC>::ld(H + m.p1, h1[q]);
        if (rope) Vec<T, VEC>::ld(H + m.p2, h2[q]);
        if (a.row_denom) {
          const float dn = __ldg(a.row_denom + rowb + t);
          rs[q] = dn != 0.f ? 1.f / dn : 0.f;
#pragma unroll
          for (int e = 0; e < VEC; ++e) h1[q][e] *= rs[q], h2[q][e] = rope ? h2[q][e] * rs[q] : 0.f;
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) h1[q][e] = hb1[e], h2[q][e] = hb2[e];
      }
      if (BWD) {
        const T* __restrict__ dsh = static_cast<const T*>(a.dsh) + (rowb + t) * a.ld_dsh;
        Vec<T, VEC>::ld(dsh + m.p1, g1[q]);
        if (rope) Vec<T, VEC>::ld(dsh + m.p2, g2[q]);
      }
    }
#pragma unroll
    for (int q = 0; q < TB; ++q) {
      const int t = tb + q;
      if (t >= t1) break;
      float s1[VEC], s2[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        z1[q][e] += b1[e];
        const float r1 = a.activated ? z1[q][e] : pom_hardsigmoid(z1[q][e]);
        if (rope) {
          z2[q][e] += b2[e];
          const float r2 = a.activated ? z2[q][e] : pom_hardsigmoid(z2[q][e]);
          s1[e] = r1 * cs[q][e] - r2 * sn[q][e];
          s2[e] = r2 * cs[q][e] + r1 * sn[q][e];
        } else {
          s1[e] = r1;
          s2[e] = 0.f;
        }
      }
      if (!BWD) {
        float o[VEC];
        T* __restrict__ sh = static_cast<T*>(a.sh) + (rowb + t) * a.ld_sh;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = s1[e] * h1[q][e];
        Vec<T, VEC>::st(sh + m.p1, o);
        if (rope) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = s2[e] * h2[q][e];
          Vec<T, VEC>::st(sh + m.p2, o);
        }
      } else {
        T* __restrict__ dz = static_cast<T*>(a.dz) + (rowb + t) * a.ld_dz;
        float dh1[VEC], dh2[VEC], o1[VEC], o2[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          dh1[e] = g1[q][e] * s1[e];
          accH1[e] += dh1[e];
          const float t1v = g1[q][e] * h1[q][e];  // gradient of the rotated gate
          float ds1 = t1v;
          dh2[e] = o2[e] = 0.f;
          if (rope) {
            dh2[e] = g2[q][e] * s2[e];
            accH2[e] += dh2[e];
            const float t2v = g2[q][e] * h2[q][e];
            ds1 = t1v * cs[q][e] + t2v * sn[q][e];
            const float ds2 = t2v * cs[q][e] - t1v * sn[q][e];
            o2[e] = a.activated ? ds2 : ds2 * pom_hardsigmoid_grad(z2[q][e]);
            accB2[e] += o2[e];
          }
          o1[e] = a.activated ? ds1 : ds1 * pom_hardsigmoid_grad(z1[q][e]);
          accB1[e] += o1[e];
        }
        Vec<T, VEC>::st(dz + m.p1, o1);
        if (rope) Vec<T, VEC>::st(dz + m.p2, o2);
        if (a.h_per_token) {
          T* __restrict__ dh = static_cast<T*>(a.dh_tok) + (rowb + t) * a.ld_dh;
#pragma unroll
          for (int e = 0; e < VEC; ++e) dh1[e] *= rs[q], dh2[e] *= rs[q];  // gradient of the un-normalised H
          Vec<T, VEC>::st(dh + m.p1, dh1);
          if (rope) Vec<T, VEC>::st(dh + m.p2, dh2);
        }
      }
    }
  }
  if (BWD) {
    const long long o = (static_cast<long long>(b) * a.chunks + c) * a.P;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      a.dbias_partial[o + m.p1 + e] = accB1[e];
      if (rope) a.dbias_partial[o + m.p2 + e] = accB2[e];
      if (!a.h_per_token) {
        a.dh_partial[o + m.p1 + e] = accH1[e];
        if (rope) a.dh_partial[o + m.p2 + e] = accH2[e];
      }
    }
  }
}

// ------------------------------------------------------------------ multi-head scalar gating
// One gate value per (token, head) multiplies every channel of that head
// (reference pom/pom.py:119-122).  The gate s (B, T, heads) is fp32 and already activated / rotated.
struct SelHeadsDev {
  const float* s;
  const void* H;
  const void* dsh;
  void* sh;
  float* ds;
  float* dh_partial;
  void* dh_tok;
  long long ld_h, ld_sh, ld_dsh, ld_dh;
  int B, T, P, heads, head_dim, chunks, h_per_token;
};

template <typename T, int VEC, bool BWD>
__global__ void __launch_bounds__(128) select_heads_kernel(const SelHeadsDev a) {
  const int p = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  if (p >= a.P) return;
  const int head = p / a.head_dim;  // VEC divides head_dim, so the thread's channels share one head
  const long long rowb = static_cast<long long>(b) * a.T;
  float hb[VEC], accH[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    hb[e] = a.h_per_token ? 0.f : static_cast<const float*>(a.H)[static_cast<long long>(b) * a.P + p + e];
    accH[e] = 0.f;
  }
  const int t0 = c * kChunk, t1 = min(a.T, t0 + kChunk);
  constexpr int TB = 4;
  for (int tb = t0; tb < t1; tb += TB) {
    float h[TB][VEC], g[TB][VEC], sv[TB];
#pragma unroll
    for (int q = 0; q < TB; ++q) {
      const int t = min(tb + q, t1 - 1);
      sv[q] = __ldg(a.s + (rowb + t) * a.heads + head);
      if (a.h_per_token) {
        Vec<T, VEC>::ld(static_cast<const T*>(a.H) + (rowb + t) * a.ld_h + p, h[q]);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) h[q][e] = hb[e];
      }
      if (BWD) Vec<T, VEC>::ld(static_cast<const T*>(a.dsh) + (rowb + t) * a.ld_dsh + p, g[q]);
    }
#pragma unroll
    for (int q = 0; q < TB; ++q) {
      const int t = tb + q;
      if (t >= t1) break;
      float o[VEC];
      if (!BWD) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = sv[q] * h[q][e];
        Vec<T, VEC>::st(static_cast<T*>(a.sh) + (rowb + t) * a.ld_sh + p, o);
      } else {
        float dsum = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          o[e] = g[q][e] * sv[q];      // gradient of H
          accH[e] += o[e];
          dsum = fmaf(g[q][e], h[q][e], dsum);  // gradient of the gate, summed over the head's channels
        }
        atomicAdd(a.ds + (rowb + t) * a.heads + head, dsum);
        if (a.h_per_token) Vec<T, VEC>::st(static_cast<T*>(a.dh_tok) + (rowb + t) * a.ld_dh + p, o);
      }
    }
  }
  if (BWD && !a.h_per_token) {
    float* dst = a.dh_partial + (static_cast<long long>(b) * a.chunks + c) * a.P + p;
#pragma unroll
    for (int e = 0; e < VEC; ++e) dst[e] = accH[e];
  }
}

// ------------------------------------------------------------------ small element-wise
__global__ void state_merge_kernel(const float* hp, const float* hc, float* hn, float n_past, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) hn[i] = (n_past * hp[i] + hc[i]) / (n_past + 1.f);
}
// out[b, t] = sum of the 128 mask weights of tile t of sample b (one warp per tile).
__global__ void tile_weights_kernel(const float* __restrict__ w, float* __restrict__ out, int N, int tiles) {
  const int t = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  float s = 0.f;
  for (int r = lane; r < 128; r += 32) {
    const int n = t * 128 + r;
    if (n < N) s += w[static_cast<long long>(b) * N + n];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[static_cast<long long>(b) * tiles + t] = s;
}

// Running mean over frames: forward out[b,f,:] = (1/(f+1)) sum_{g<=f} in[b,g,:];
// adjoint out[b,g,:] = sum_{f>=g} in[b,f,:]/(f+1).  One thread per (b, p).
__global__ void frame_prefix_kernel(const float* __restrict__ in, float* __restrict__ out, int F, int P, int adjoint) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= P) return;
  const long long base = static_cast<long long>(blockIdx.y) * F * P + p;
  float acc = 0.f;
  if (!adjoint) {
    for (int f = 0; f < F; ++f) {
      acc += in[base + static_cast<long long>(f) * P];
      out[base + static_cast<long long>(f) * P] = acc / static_cast<float>(f + 1);
    }
  } else {
    for (int f = F - 1; f >= 0; --f) {
      acc += in[base + static_cast<long long>(f) * P] / static_cast<float>(f + 1);
      out[base + static_cast<long long>(f) * P] = acc;
    }
  }
}
__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d, long long count) {
  pomk::griddep_wait();  // launched with programmatic stream serialization
  pomk::griddep_launch();
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= count && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(s + i));
    __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
    *reinterpret_cast<uint2*>(d + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  } else {
    for (long long j = i; j < count && j < i + 4; ++j) d[j] = __float2bfloat16_rn(s[j]);
  }
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) d[i] = __bfloat162float(s[i]);
}

// ------------------------------------------------------------------ host helpers
int check_rope(const pom_rope& r, int P) {
  if (r.kind == POM_ROPE_NONE) return POM_OK;
  if (r.kind == POM_ROPE_1D) {
    if (P % 2) return POM_ERR_BAD_SHAPE;
    if (!r.cos0 || !r.sin0 || !r.pos || r.pos_stride < 1) return POM_ERR_NULL;
    return POM_OK;
  }
  if (r.kind == POM_ROPE_2D) {
    if (P % 4) return POM_ERR_BAD_SHAPE;
    if (!r.cos0 || !r.sin0 || !r.cos1 || !r.sin1 || !r.pos || r.pos_stride < 2) return POM_ERR_NULL;
    return POM_OK;
  }
  return POM_ERR_UNSUPPORTED;
}

// Channels per thread: a 16-byte vector (8 bf16 / 4 fp32) when every access stays aligned and the
// degree fits the register-resident coefficient set, else 2, else 1.
int pick_vec(int P, const pom_rope& rope, int dtype, int K, std::initializer_list<long long> lds,
             std::initializer_list<const void*> ptrs) {
  const int unit = rope.kind == POM_ROPE_2D ? P / 4 : rope.kind == POM_ROPE_1D ? P / 2 : P;
  const int wide = dtype == POM_BF16 ? 8 : 4;
  auto ok = [&](int v) {
    if (unit % v) return false;
    for (long long ld : lds)
      if (ld % v) return false;
    const uintptr_t mask = static_cast<uintptr_t>(v * (dtype == POM_BF16 ? 2 : 4) - 1);
    for (const void* p : ptrs)
      if (p && (reinterpret_cast<uintptr_t>(p) & mask)) return false;
    if (rope.kind != POM_ROPE_NONE) {
      const uintptr_t tmask = static_cast<uintptr_t>((v >= 4 ? 16 : v * 4) - 1);
      for (const void* p : {static_cast<const void*>(rope.cos0), static_cast<const void*>(rope.sin0),
                            static_cast<const void*>(rope.cos1), static_cast<const void*>(rope.sin1)})
        if (p && (reinterpret_cast<uintptr_t>(p) & tmask)) return false;
    }
    return true;
  };
  if (K <= 4 && ok(wide)) return wide;
  if (ok(2)) return 2;
  return 1;
}

struct WalkLaunch {
  dim3 grid;
  int block;
};

WalkLaunch walk_launch(int P, int rope_kind, int vec, int chunks, int B) {
  const int units = static_cast<int>(ceil_div(first_channels(P, rope_kind), vec));
  // block size: a multiple of 32 up to 128 that wastes the fewest lanes
  int best = 128;
  long long best_waste = -1;
  for (int bs = 128; bs >= 32; bs -= 32) {
    const long long waste = ceil_div(units, bs) * bs - units;
    if (best_waste < 0 || waste < best_waste) {
      best_waste = waste;
      best = bs;
    }
  }
  WalkLaunch w;
  w.block = best;
  w.grid = dim3(static_cast<unsigned>(ceil_div(units, best)), static_cast<unsigned>(chunks), static_cast<unsigned>(B));
  return w;
}

// CALL(T, VEC, KR) for the (dtype, vec) pair picked above.
#define POM_DISPATCH(dtype, vec, CALL)                  \
  do {                                                  \
    if ((dtype) == POM_BF16) {                          \
      if ((vec) == 8) { CALL(__nv_bfloat16, 8, 4); }    \
      else if ((vec) == 2) { CALL(__nv_bfloat16, 2, kMaxDegree); } \
      else { CALL(__nv_bfloat16, 1, kMaxDegree); }      \
    } else {                                            \
      if ((vec) == 4) { CALL(float, 4, 4); }            \
      else if ((vec) == 2) { CALL(float, 2, kMaxDegree); } \
      else { CALL(float, 1, kMaxDegree); }              \
    }                                                   \
  } while (0)

// Same, for kernels that keep the polynomial coefficients in registers: degrees 1-2 get their own
// instantiation (half the arithmetic of the 4-coefficient form).
#define POM_DISPATCH_K(dtype, vec, K, CALL)                                   \
  do {                                                                        \
    if ((dtype) == POM_BF16 && (vec) == 8) {                                  \
      if ((K) <= 2) { CALL(__nv_bfloat16, 8, 2); } else { CALL(__nv_bfloat16, 8, 4); } \
    } else if ((dtype) != POM_BF16 && (vec) == 4) {                           \
      if ((K) <= 2) { CALL(float, 4, 2); } else { CALL(float, 4, 4); }        \
    } else {                                                                  \
      POM_DISPATCH(dtype, vec, CALL);                                         \
    }                                                                         \
  } while (0)

}  // namespace

// =========================================================================== C ABI
extern "C" {

int32_t pom_agg_chunks(int32_t N) { return N <= 0 ? 0 : static_cast<int32_t>(ceil_div(N, kChunk)); }

int pom_reduce_partials(const float* partial, float* out, const float* denom, float scale, int32_t B,
                        int32_t chunks, int32_t P, void* stream) {
  if (!partial || !out) return POM_ERR_NULL;
  if (B <= 0 || chunks <= 0 || P <= 0) return POM_ERR_BAD_SHAPE;
  if (B > 65535) return POM_ERR_TOO_LARGE;
  dim3 grid(static_cast<unsigned>(ceil_div(P, 32)), static_cast<unsigned>(B));
  (void)launch_pdl(reduce_partials_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), partial, out, denom, scale, chunks,
                                                                             P);
  count_launch();
  return check_launch();
}

int pom_poly_agg_fwd(const pom_agg_args* a, void* stream) {
  if (!a || !a->x || !a->coeff || (!a->partial && a->causal != 2)) return POM_ERR_NULL;
  if (a->causal < 0 || a->causal > 2) return POM_ERR_UNSUPPORTED;
  if (a->B <= 0 || a->N <= 0 || a->P <= 0 || a->K < 1) return POM_ERR_BAD_SHAPE;
  if (a->K > kMaxDegree) return POM_ERR_K_TOO_LARGE;
  if (a->B > 65535 || pom_agg_chunks(a->N) > 65535) return POM_ERR_TOO_LARGE;
  if (a->dtype != POM_BF16 && a->dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  if (a->ldx < a->P) return POM_ERR_BAD_STRIDE;
  int rc = check_rope(a->rope, a->P);
  if (rc) return rc;
  if (a->causal && (!a->out || a->ld_out < a->P)) return POM_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AggDev d;
  d.x = a->x;
  d.coeff = a->coeff;
  d.row_weight = a->causal ? nullptr : a->row_weight;
  d.partial = a->partial;
  d.out = a->out;
  d.ldx = a->ldx;
  d.ld_out = a->ld_out;
  d.token_offset = a->token_offset;
  d.B = a->B;
  d.N = a->N;
  d.P = a->P;
  d.K = a->K;
  d.chunks = pom_agg_chunks(a->N);
  d.per_token = a->causal == 2;
  d.rope = a->rope;
  const int vec = pick_vec(a->P, a->rope, a->dtype, a->K, {a->ldx, a->causal ? a->ld_out : 0},
                           {a->x, a->causal ? a->out : nullptr});
  const WalkLaunch wl = walk_launch(a->P, a->rope.kind, vec, d.chunks, a->B);
  const bool has_rope = a->rope.kind != POM_ROPE_NONE;
  if (a->causal != 2) {  // per-token features (causal == 2) need neither the sums nor the scan
#define CALL_SUM(T, V, KR)                                                                    \
  if (has_rope) agg_fwd_kernel<T, V, KR, false, true><<<wl.grid, wl.block, 0, st>>>(d);        \
  else agg_fwd_kernel<T, V, KR, false, false><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH_K(a->dtype, vec, a->K, CALL_SUM);
#undef CALL_SUM
    count_launch();
    rc = check_launch();
    if (rc || !a->causal) return rc;
    dim3 sgrid(static_cast<unsigned>(ceil_div(a->P, 128)), static_cast<unsigned>(a->B));
    chunk_scan_kernel<<<sgrid, 128, 0, st>>>(a->partial, a->carry, a->total, d.chunks, a->P, 0);
    count_launch();
  }
#define CALL_PFX(T, V, KR)                                                                   \
  if (has_rope) agg_fwd_kernel<T, V, KR, true, true><<<wl.grid, wl.block, 0, st>>>(d);        \
  else agg_fwd_kernel<T, V, KR, true, false><<<wl.grid, wl.block, 0, st>>>(d)
  POM_DISPATCH_K(a->dtype, vec, a->K, CALL_PFX);
#undef CALL_PFX
  count_launch();
  return check_launch();
}

// ------------------------------------------------------------------ aggregation without any allocation
// Built-in workspace for pom_poly_agg_mean_noalloc: 4 Mi floats (16 MiB) that every GPU loading this
// library keeps resident until the process exits.
constexpr long long kNoAllocFloats = 4ll << 20;
static __device__ __align__(256) float g_noalloc_workspace[kNoAllocFloats];

// Device address of the workspace on the current device.  In host code the array's name is only a
// handle for the runtime, not something a kernel can dereference, so the address is looked up once
// per device and cached.
static int noalloc_workspace(float** out) {
  static std::mutex mu;
  static float* cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_workspace) != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return POM_ERR_CUDA;
    }
    cache[dev] = static_cast<float*>(p);
  }
  *out = cache[dev];
  return POM_OK;
}

int pom_poly_agg_mean_noalloc(const pom_agg_args* a, const float* denom, float scale, float* out, void* stream) {
  if (!a || !a->x || !a->coeff || !out) return POM_ERR_NULL;
  if (a->causal) return POM_ERR_UNSUPPORTED;
  if (a->B <= 0 || a->N <= 0 || a->P <= 0 || a->K < 1) return POM_ERR_BAD_SHAPE;
  if (a->K > kMaxDegree) return POM_ERR_K_TOO_LARGE;
  const int chunks = pom_agg_chunks(a->N);
  if (a->B > 65535 || chunks > 65535) return POM_ERR_TOO_LARGE;
  if (1ll * a->B * chunks * a->P > kNoAllocFloats) return POM_ERR_TOO_LARGE;  // does not fit the built-in workspace
  if (a->dtype != POM_BF16 && a->dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  if (a->ldx < a->P) return POM_ERR_BAD_STRIDE;
  int rc = check_rope(a->rope, a->P);
  if (rc) return rc;
  float* ws = nullptr;
  if ((rc = noalloc_workspace(&ws))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AggDev d;
  d.x = a->x;
  d.coeff = a->coeff;
  d.row_weight = a->row_weight;
  d.partial = ws;
  d.out = nullptr;
  d.ldx = a->ldx;
  d.ld_out = 0;
  d.token_offset = 0;
  d.B = a->B;
  d.N = a->N;
  d.P = a->P;
  d.K = a->K;
  d.chunks = chunks;
  d.per_token = 0;
  d.rope = a->rope;
  const int vec = pick_vec(a->P, a->rope, a->dtype, a->K, {a->ldx}, {a->x});
  const WalkLaunch wl = walk_launch(a->P, a->rope.kind, vec, chunks, a->B);
  const bool has_rope = a->rope.kind != POM_ROPE_NONE;
  // Every (sample, chunk, channel) slot that the reduction below reads is written by this launch first,
  // so nothing left in the workspace by an earlier call can leak into the result.
#define CALL_NA(T, V, KR)                                                                      \
  if (has_rope) agg_fwd_kernel<T, V, KR, false, true><<<wl.grid, wl.block, 0, st>>>(d);        \
  else agg_fwd_kernel<T, V, KR, false, false><<<wl.grid, wl.block, 0, st>>>(d)
  POM_DISPATCH_K(a->dtype, vec, a->K, CALL_NA);
#undef CALL_NA
  count_launch();
  if ((rc = check_launch())) return rc;
  dim3 grid(static_cast<unsigned>(ceil_div(a->P, 32)), static_cast<unsigned>(a->B));
  (void)launch_pdl(reduce_partials_kernel, grid, dim3(256), 0, st, ws, out, denom, scale, chunks, a->P);
  count_launch();
  return check_launch();
}

int32_t pom_poly_agg_bwd_slots(const pom_agg_bwd_args* a) {
  if (!a || a->B <= 0 || a->N <= 0 || a->P <= 0) return 0;
  if (stream_bwd_eligible(a)) return a->B * stream_plan(a->B, a->N, a->P).splits;
  if (stream_bwd_rope_eligible(a))
    return a->B * stream_plan_rope(a->B, a->N, stream_pairs(a), a->causal == 3 ? 32 : kStTok).splits;
  return a->B * pom_agg_chunks(a->N);
}

int pom_ops_status(int32_t* value_out) {
  if (!value_out) return POM_ERR_NULL;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ops_status, sizeof(int)) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  *value_out = v;
  return POM_OK;
}

int pom_poly_agg_bwd(const pom_agg_bwd_args* a, void* stream) {
  if (!a || !a->x || !a->coeff || !a->dx || !a->dcoeff_partial) return POM_ERR_NULL;
  if (a->B <= 0 || a->N <= 0 || a->P <= 0 || a->K < 1) return POM_ERR_BAD_SHAPE;
  if (a->K > kMaxDegree) return POM_ERR_K_TOO_LARGE;
  if (a->B > 65535 || pom_agg_chunks(a->N) > 65535) return POM_ERR_TOO_LARGE;
  if (a->dtype != POM_BF16 && a->dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  if (a->ldx < a->P || a->ld_dx < a->P) return POM_ERR_BAD_STRIDE;
  if (a->causal < 0 || a->causal > 3) return POM_ERR_UNSUPPORTED;
  if (a->causal ? (!a->dout || (!a->partial && a->causal != 2) || a->ld_dout < a->P) : !a->dH) return POM_ERR_NULL;
  int rc = check_rope(a->rope, a->P);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  AggBwdDev d;
  d.x = a->x;
  d.coeff = a->coeff;
  d.row_weight = a->row_weight;
  d.denom = a->denom;
  d.dH = a->dH;
  d.dout = a->dout;
  d.partial = a->partial;
  d.dx = a->dx;
  d.dcoeff_partial = a->dcoeff_partial;
  d.ldx = a->ldx;
  d.ld_dx = a->ld_dx;
  d.ld_dout = a->ld_dout;
  d.token_offset = a->token_offset;
  d.scale = a->causal ? 1.f : a->scale;
  d.B = a->B;
  d.N = a->N;
  d.P = a->P;
  d.K = a->K;
  d.chunks = pom_agg_chunks(a->N);
  d.per_token = a->causal == 2;
  d.rope = a->rope;
  if (stream_bwd_eligible(a)) {
    int* status = ops_status_ptr();
    if (!status) return POM_ERR_CUDA;
    const StreamPlan sp = stream_plan(a->B, a->N, a->P);
    const dim3 sgrid(static_cast<unsigned>(sp.col_blocks), static_cast<unsigned>(sp.splits),
                     static_cast<unsigned>(a->B));
    if (sp.splits > 65535) return POM_ERR_TOO_LARGE;
    static std::atomic<uint64_t> attr_done{0};
    (void)once_per_device(attr_done, [] {
      cudaFuncSetAttribute(agg_bwd_stream_kernel<2, kStVec, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kStSmemBytes);
      cudaFuncSetAttribute(agg_bwd_stream_kernel<4, kStVec, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kStSmemBytes);
      return static_cast<int>(POM_OK);
    });
    constexpr int threads = kStCols / kStVec * 8;
    CUtensorMap tmx;
    if ((rc = stream_tile_map(&tmx, a->x, a->P, a->N, a->B, a->ldx, kStCols, kStTok))) return rc;
    if (a->K <= 2)
      (void)launch_pdl(agg_bwd_stream_kernel<2, kStVec, true>, sgrid, dim3(threads + 32), kStSmemBytes, st, tmx, d,
                       sp.tiles_per_cta, sp.splits, status);
    else
      (void)launch_pdl(agg_bwd_stream_kernel<4, kStVec, false>, sgrid, dim3(threads), kStSmemBytes, st, tmx, d,
                       sp.tiles_per_cta, sp.splits, status);
    count_launch();
    return check_launch();
  }
  if (stream_bwd_rope_eligible(a)) {
    int* status = ops_status_ptr();
    if (!status) return POM_ERR_CUDA;
    const bool fused_causal = a->causal == 3;
    const int tt = fused_causal ? 32 : kStTok;
    const StreamPairs pr = stream_pairs(a);
    const StreamPlan sp = stream_plan_rope(a->B, a->N, pr, tt);
    if (sp.splits > 65535) return POM_ERR_TOO_LARGE;
    const dim3 sgrid(static_cast<unsigned>(sp.col_blocks), static_cast<unsigned>(sp.splits),
                     static_cast<unsigned>(a->B));
    static std::atomic<uint64_t> attr_done_rope{0};
    (void)once_per_device(attr_done_rope, [] {
      cudaFuncSetAttribute(agg_bwd_stream_pair_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStSmemBytes);
      cudaFuncSetAttribute(agg_bwd_stream_pair_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStSmemBytes);
      cudaFuncSetAttribute(agg_bwd_stream_pair_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStSmemBytes);
      return static_cast<int>(POM_OK);
    });
    const int bps = sp.col_blocks / pr.sections;
    CUtensorMap tmx, tms;
    if ((rc = stream_tile_map(&tmx, a->x, a->P, a->N, a->B, a->ldx, kStHalf, tt))) return rc;
    tms = tmx;
    if (fused_causal && (rc = stream_tile_map(&tms, a->dout, a->P, a->N, a->B, a->ld_dout, kStHalf, tt))) return rc;
    if (!fused_causal)
      (void)launch_pdl(agg_bwd_stream_pair_kernel<2, false>, sgrid, dim3(256), kStSmemBytes, st, tmx, tms, d,
                       sp.tiles_per_cta, sp.splits, pr.q, bps, status);
    else if (a->K <= 2)
      (void)launch_pdl(agg_bwd_stream_pair_kernel<2, true>, sgrid, dim3(256), kStSmemBytes, st, tmx, tms, d,
                       sp.tiles_per_cta, sp.splits, pr.q, bps, status);
    else
      (void)launch_pdl(agg_bwd_stream_pair_kernel<4, true>, sgrid, dim3(256), kStSmemBytes, st, tmx, tms, d,
                       sp.tiles_per_cta, sp.splits, pr.q, bps, status);
    count_launch();
    return check_launch();
  }
  if (a->causal == 3) return POM_ERR_UNSUPPORTED;  // the fused token-causal form exists only as the paired stream
  const int vec = pick_vec(a->P, a->rope, a->dtype, a->K, {a->ldx, a->ld_dx, a->causal ? a->ld_dout : 0},
                           {a->x, a->dx, a->causal ? a->dout : nullptr});
  const WalkLaunch wl = walk_launch(a->P, a->rope.kind, vec, d.chunks, a->B);
  const bool has_rope = a->rope.kind != POM_ROPE_NONE;
  if (a->causal) {
    if (a->causal == 1) {
      // Plain column walk (no channel pairing) for the scaled chunk sums.
      pom_rope none{};
      const int v2 = pick_vec(a->P, none, a->dtype, 1, {a->ld_dout}, {a->dout});
      const WalkLaunch w1 = walk_launch(a->P, POM_ROPE_NONE, v2, d.chunks, a->B);
#define CALL_CS(T, V, KR) causal_bwd_sum_kernel<T, V><<<w1.grid, w1.block, 0, st>>>(d)
      POM_DISPATCH(a->dtype, v2, CALL_CS);
#undef CALL_CS
      count_launch();
      dim3 sgrid(static_cast<unsigned>(ceil_div(a->P, 128)), static_cast<unsigned>(a->B));
      chunk_scan_kernel<<<sgrid, 128, 0, st>>>(a->partial, a->carry, a->total, d.chunks, a->P, 1);
      count_launch();
      if (a->phase == 1) return check_launch();  // totals only
    }
#define CALL_BC(T, V, KR)                                                                    \
  if (has_rope) agg_bwd_kernel<T, V, KR, true, true><<<wl.grid, wl.block, 0, st>>>(d);        \
  else agg_bwd_kernel<T, V, KR, true, false><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH_K(a->dtype, vec, a->K, CALL_BC);
#undef CALL_BC
  } else {
#define CALL_BN(T, V, KR)                                                                    \
  if (has_rope) agg_bwd_kernel<T, V, KR, false, true><<<wl.grid, wl.block, 0, st>>>(d);       \
  else agg_bwd_kernel<T, V, KR, false, false><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH_K(a->dtype, vec, a->K, CALL_BN);
#undef CALL_BN
  }
  count_launch();
  return check_launch();
}

static int select_common(SelDev& d, int dtype, bool bwd, std::initializer_list<long long> lds,
                         std::initializer_list<const void*> ptrs, cudaStream_t st) {
  if (d.B <= 0 || d.T <= 0 || d.P <= 0) return POM_ERR_BAD_SHAPE;
  if (dtype != POM_BF16 && dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  d.chunks = pom_agg_chunks(d.T);
  if (d.B > 65535 || d.chunks > 65535) return POM_ERR_TOO_LARGE;
  int rc = check_rope(d.rope, d.P);
  if (rc) return rc;
  const int vec = pick_vec(d.P, d.rope, dtype, 1, lds, ptrs);
  const WalkLaunch wl = walk_launch(d.P, d.rope.kind, vec, d.chunks, d.B);
  const bool has_rope = d.rope.kind != POM_ROPE_NONE;
  if (bwd) {
#define CALL_SB(T, V, KR)                                                          \
  if (has_rope) select_kernel<T, V, true, true><<<wl.grid, wl.block, 0, st>>>(d);   \
  else select_kernel<T, V, true, false><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH(dtype, vec, CALL_SB);
#undef CALL_SB
  } else {
#define CALL_SF(T, V, KR)                                                          \
  if (has_rope) select_kernel<T, V, false, true><<<wl.grid, wl.block, 0, st>>>(d);  \
  else select_kernel<T, V, false, false><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH(dtype, vec, CALL_SF);
#undef CALL_SF
  }
  count_launch();
  return check_launch();
}

int pom_select_fwd(const pom_select_args* a, void* stream) {
  if (!a || !a->z || (!a->bias && !a->activated) || !a->H || !a->sh) return POM_ERR_NULL;
  if (a->ld_z < a->P || a->ld_sh < a->P || (a->h_per_token && a->ld_h < a->P)) return POM_ERR_BAD_STRIDE;
  SelDev d{};
  d.z = a->z;
  d.bias = a->bias;
  d.H = a->H;
  d.sh = a->sh;
  d.ld_z = a->ld_z;
  d.ld_h = a->ld_h;
  d.ld_sh = a->ld_sh;
  d.B = a->B;
  d.T = a->T;
  d.P = a->P;
  d.h_per_token = a->h_per_token;
  d.activated = a->activated;
  d.row_denom = a->h_per_token ? a->row_denom : nullptr;
  d.rope = a->rope;
  return select_common(d, a->dtype, false, {a->ld_z, a->ld_sh, a->h_per_token ? a->ld_h : 0},
                       {a->z, a->sh, a->h_per_token ? a->H : nullptr}, static_cast<cudaStream_t>(stream));
}

int pom_select_bwd(const pom_select_bwd_args* a, void* stream) {
  if (!a || !a->dsh || !a->z || (!a->bias && !a->activated) || !a->H || !a->dz || !a->dbias_partial)
    return POM_ERR_NULL;
  if (a->h_per_token ? !a->dh_tok : !a->dh_partial) return POM_ERR_NULL;
  if (a->ld_z < a->P || a->ld_dsh < a->P || a->ld_dz < a->P) return POM_ERR_BAD_STRIDE;
  if (a->h_per_token && (a->ld_h < a->P || a->ld_dh < a->P)) return POM_ERR_BAD_STRIDE;
  SelDev d{};
  d.z = a->z;
  d.bias = a->bias;
  d.H = a->H;
  d.dsh = a->dsh;
  d.dz = a->dz;
  d.dbias_partial = a->dbias_partial;
  d.dh_partial = a->dh_partial;
  d.dh_tok = a->dh_tok;
  d.ld_z = a->ld_z;
  d.ld_h = a->ld_h;
  d.ld_dsh = a->ld_dsh;
  d.ld_dz = a->ld_dz;
  d.ld_dh = a->ld_dh;
  d.B = a->B;
  d.T = a->T;
  d.P = a->P;
  d.h_per_token = a->h_per_token;
  d.activated = a->activated;
  d.row_denom = a->h_per_token ? a->row_denom : nullptr;
  d.rope = a->rope;
  return select_common(d, a->dtype, true,
                       {a->ld_z, a->ld_dsh, a->ld_dz, a->h_per_token ? a->ld_h : 0, a->h_per_token ? a->ld_dh : 0},
                       {a->z, a->dsh, a->dz, a->h_per_token ? a->H : nullptr, a->h_per_token ? a->dh_tok : nullptr},
                       static_cast<cudaStream_t>(stream));
}

static int select_heads_common(const pom_select_heads_args* a, bool bwd, void* stream) {
  if (!a || !a->s || !a->H) return POM_ERR_NULL;
  if (bwd ? (!a->dsh || !a->ds || (a->h_per_token ? !a->dh_tok : !a->dh_partial)) : !a->sh) return POM_ERR_NULL;
  if (a->B <= 0 || a->T <= 0 || a->P <= 0 || a->heads <= 0 || a->P % a->heads) return POM_ERR_BAD_SHAPE;
  if (a->dtype != POM_BF16 && a->dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  SelHeadsDev d{};
  d.s = a->s;
  d.H = a->H;
  d.dsh = a->dsh;
  d.sh = a->sh;
  d.ds = a->ds;
  d.dh_partial = a->dh_partial;
  d.dh_tok = a->dh_tok;
  d.ld_h = a->ld_h;
  d.ld_sh = a->ld_sh;
  d.ld_dsh = a->ld_dsh;
  d.ld_dh = a->ld_dh;
  d.B = a->B;
  d.T = a->T;
  d.P = a->P;
  d.heads = a->heads;
  d.head_dim = a->P / a->heads;
  d.chunks = pom_agg_chunks(a->T);
  d.h_per_token = a->h_per_token;
  if (d.B > 65535 || d.chunks > 65535) return POM_ERR_TOO_LARGE;
  pom_rope none{};
  // the channel vector must not straddle two heads: treat head_dim as the unit the vector has to divide
  int vec = pick_vec(d.head_dim, none, a->dtype, 1,
                     {a->h_per_token ? a->ld_h : 0, bwd ? a->ld_dsh : a->ld_sh, (bwd && a->h_per_token) ? a->ld_dh : 0},
                     {a->h_per_token ? a->H : nullptr, bwd ? a->dsh : a->sh, (bwd && a->h_per_token) ? a->dh_tok : nullptr});
  const WalkLaunch wl = walk_launch(a->P, POM_ROPE_NONE, vec, d.chunks, a->B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (bwd) {
#define CALL_HB(T, V, KR) select_heads_kernel<T, V, true><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH(a->dtype, vec, CALL_HB);
#undef CALL_HB
  } else {
#define CALL_HF(T, V, KR) select_heads_kernel<T, V, false><<<wl.grid, wl.block, 0, st>>>(d)
    POM_DISPATCH(a->dtype, vec, CALL_HF);
#undef CALL_HF
  }
  count_launch();
  return check_launch();
}

int pom_select_heads_fwd(const pom_select_heads_args* a, void* stream) { return select_heads_common(a, false, stream); }
int pom_select_heads_bwd(const pom_select_heads_args* a, void* stream) { return select_heads_common(a, true, stream); }

int pom_state_merge(const float* h_past, const float* h_cur, float* h_new, float n_past, int64_t count, void* stream) {
  if (!h_past || !h_cur || !h_new) return POM_ERR_NULL;
  if (count <= 0) return POM_ERR_BAD_SHAPE;
  state_merge_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      h_past, h_cur, h_new, n_past, count);
  count_launch();
  return check_launch();
}

int pom_tile_weights(const float* w, float* out, int32_t B, int32_t N, void* stream) {
  if (!w || !out) return POM_ERR_NULL;
  if (B <= 0 || N <= 0) return POM_ERR_BAD_SHAPE;
  if (B > 65535) return POM_ERR_TOO_LARGE;
  const int tiles = (N + 127) / 128;
  tile_weights_kernel<<<dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(B)), 32, 0,
                        static_cast<cudaStream_t>(stream)>>>(w, out, N, tiles);
  count_launch();
  return check_launch();
}

int pom_frame_prefix_mean(const float* in, float* out, int32_t B, int32_t F, int32_t P, int32_t adjoint, void* stream) {
  if (!in || !out) return POM_ERR_NULL;
  if (B <= 0 || F <= 0 || P <= 0) return POM_ERR_BAD_SHAPE;
  if (B > 65535) return POM_ERR_TOO_LARGE;
  dim3 grid(static_cast<unsigned>(ceil_div(P, 128)), static_cast<unsigned>(B));
  frame_prefix_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(in, out, F, P, adjoint);
  count_launch();
  return check_launch();
}

int pom_copy_bytes(void* dst, const void* src, int64_t bytes, void* stream) {
  if (!dst || !src) return POM_ERR_NULL;
  if (bytes < 0) return POM_ERR_BAD_SHAPE;
  if (bytes == 0) return POM_OK;
  if (cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice,
                      static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  return POM_OK;
}

int pom_fill_zero(void* dst, int64_t bytes, void* stream) {
  if (!dst) return POM_ERR_NULL;
  if (bytes <= 0) return POM_ERR_BAD_SHAPE;
  if (cudaMemsetAsync(dst, 0, static_cast<size_t>(bytes), static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  return POM_OK;
}

int pom_cast_f32_to_bf16(const float* src, void* dst, int64_t count, void* stream) {
  if (!src || !dst) return POM_ERR_NULL;
  if (count <= 0) return POM_ERR_BAD_SHAPE;
  (void)launch_pdl(cast_f32_bf16_kernel, dim3(static_cast<unsigned>(ceil_div(ceil_div(count, 4), 256))), dim3(256), 0,
                   static_cast<cudaStream_t>(stream), src, static_cast<__nv_bfloat16*>(dst), count);
  count_launch();
  return check_launch();
}

int pom_cast_bf16_to_f32(const void* src, float* dst, int64_t count, void* stream) {
  if (!src || !dst) return POM_ERR_NULL;
  if (count <= 0) return POM_ERR_BAD_SHAPE;
  cast_bf16_f32_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), dst, count);
  count_launch();
  return check_launch();
}

int pom_abi_version(void) { return POM_ABI_VERSION; }

const char* pom_strerror(int code) {
  switch (code) {
    case POM_OK: return "ok";
    case POM_ERR_BAD_SHAPE: return "bad shape";
    case POM_ERR_BAD_STRIDE: return "bad stride (leading dimension too small or not a multiple of 8 elements)";
    case POM_ERR_BAD_ALIGN: return "bad alignment (16-byte aligned base address and row pitch required)";
    case POM_ERR_UNSUPPORTED: return "unsupported combination of options";
    case POM_ERR_K_TOO_LARGE: return "polynomial degree above 16 is not implemented";
    case POM_ERR_CUDA: return "CUDA runtime or driver error";
    case POM_ERR_TIMEOUT: return "device-side wait timed out";
    case POM_ERR_NULL: return "required pointer is null";
    case POM_ERR_TOO_LARGE: return "dimension exceeds the supported range";
    default: return "unknown error";
  }
}

int pom_device_check(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  return major == 10 ? POM_OK : POM_ERR_UNSUPPORTED;
}

long long pom_launch_count(void) { return g_launches.load(); }

}  // extern "C"
