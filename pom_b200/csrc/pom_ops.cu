// Stand-alone PoM operators (HBM-bound SIMT kernels): polynomial aggregation with
// mean / weighted / causal-prefix reduction, the gated selection, their
// backward passes, optional rotary embedding in all of them, and the small
// reductions that finish the per-tile partial sums of the fused GEMM epilogues.
//
// Common traversal: grid = (column blocks, token chunks, batch); one thread owns
// VEC adjacent channels (plus their rotary partners) and walks the tokens of its
// chunk, so global accesses are coalesced across the block and every sum is
// formed in a fixed order (deterministic, no float atomics).
#include "common.cuh"
#include "pom_math.cuh"
#include <cuda_bf16.h>

using namespace pomk;
using namespace pomh;

namespace {

constexpr int kChunk = 64;     // tokens per chunk
constexpr int kThreads = 128;  // threads per block

// ------------------------------------------------------------------ element access
template <typename T, int VEC>
struct Vec;
template <>
struct Vec<float, 1> {
  static __device__ __forceinline__ void ld(const float* p, float (&v)[1]) { v[0] = __ldg(p); }
  static __device__ __forceinline__ void st(float* p, const float (&v)[1]) { p[0] = v[0]; }
};
template <>
struct Vec<float, 2> {
  static __device__ __forceinline__ void ld(const float* p, float (&v)[2]) {
    float2 f = __ldg(reinterpret_cast<const float2*>(p));
    v[0] = f.x;
    v[1] = f.y;
  }
  static __device__ __forceinline__ void st(float* p, const float (&v)[2]) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  }
};
template <>
struct Vec<__nv_bfloat16, 1> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[1]) { v[0] = __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[1]) { p[0] = __float2bfloat16_rn(v[0]); }
};
template <>
struct Vec<__nv_bfloat16, 2> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[2]) {
    unsigned int raw = __ldg(reinterpret_cast<const unsigned int*>(p));
    float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw));
    v[0] = f.x;
    v[1] = f.y;
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[2]) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
  }
};

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

__host__ __device__ inline int first_channels(int P, int rope_kind) { return rope_kind == POM_ROPE_NONE ? P : P / 2; }

template <int VEC>
__device__ __forceinline__ void rope_coeffs(const pom_rope& r, const ColMap& m, long long n, float (&c)[VEC],
                                            float (&s)[VEC]) {
  const long long idx = r.pos[n * r.pos_stride + m.which];
  const float* ct = (m.which ? r.cos1 : r.cos0) + idx * m.tab_ld + m.j;
  const float* stb = (m.which ? r.sin1 : r.sin0) + idx * m.tab_ld + m.j;
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    c[e] = __ldg(ct + e);
    s[e] = __ldg(stb + e);
  }
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

template <int KR>
__device__ __forceinline__ float poly_reg(float a, const float (&c)[KR], int K) {
  float p = a;
  float acc = c[0] * p;
#pragma unroll
  for (int i = 1; i < KR; ++i) {
    if (i < K) {
      p *= a;
      acc = fmaf(c[i], p, acc);
    }
  }
  return acc;
}
template <int KR>
__device__ __forceinline__ float poly_grad_reg(float a, const float (&c)[KR], int K) {
  float p = 1.f;
  float acc = c[0];
#pragma unroll
  for (int i = 1; i < KR; ++i) {
    if (i < K) {
      p *= a;
      acc = fmaf(static_cast<float>(i + 1) * c[i], p, acc);
    }
  }
  return acc;
}

struct AggDev {
  const void* x;
  const float* coeff;
  const float* row_weight;
  float* partial;
  void* out;
  long long ldx, ld_out, token_offset;
  int B, N, P, K, chunks;
  pom_rope rope;
};

// ------------------------------------------------------------------ forward: chunk sums / prefix apply
// PREFIX == false: partial[b, c, :] = sum over the chunk of w * R·poly.
// PREFIX == true : partial holds the exclusive prefix per chunk; writes out[b, n, :].
template <typename T, int VEC, int KR, bool PREFIX>
__global__ void __launch_bounds__(kThreads) agg_fwd_kernel(const AggDev a) {
  const int u = (blockIdx.x * kThreads + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  const bool rope = a.rope.kind != POM_ROPE_NONE;
  const ColMap m = map_unit(u, a.P, a.rope.kind);
  if (!m.valid) return;
  Coefs<VEC, KR> cf;
  cf.load(a.coeff, m, a.K, rope);
  const T* x = static_cast<const T*>(a.x) + static_cast<long long>(b) * a.N * a.ldx;
  T* out = PREFIX ? static_cast<T*>(a.out) + static_cast<long long>(b) * a.N * a.ld_out : nullptr;
  float* part = a.partial + (static_cast<long long>(b) * a.chunks + c) * a.P;
  float acc1[VEC], acc2[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    acc1[e] = PREFIX ? part[m.p1 + e] : 0.f;
    acc2[e] = (PREFIX && rope) ? part[m.p2 + e] : 0.f;
  }
  const int n0 = c * kChunk, n1 = min(a.N, n0 + kChunk);
#pragma unroll 4
  for (int n = n0; n < n1; ++n) {
    float x1[VEC], x2[VEC], f1[VEC], f2[VEC];
    Vec<T, VEC>::ld(x + n * a.ldx + m.p1, x1);
    if (rope) Vec<T, VEC>::ld(x + n * a.ldx + m.p2, x2);
    float w = 1.f;
    if (!PREFIX && a.row_weight) w = __ldg(a.row_weight + static_cast<long long>(b) * a.N + n);
#pragma unroll
    for (int e = 0; e < VEC; ++e) f1[e] = poly_reg<KR>(pom_act(x1[e]), cf.c1[e], a.K);
    if (rope) {
      float cs[VEC], sn[VEC];
      rope_coeffs<VEC>(a.rope, m, n, cs, sn);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        f2[e] = poly_reg<KR>(pom_act(x2[e]), cf.c2[e], a.K);
        acc1[e] += w * (f1[e] * cs[e] - f2[e] * sn[e]);
        acc2[e] += w * (f2[e] * cs[e] + f1[e] * sn[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc1[e] += w * f1[e];
    }
    if (PREFIX) {
      const float inv = 1.f / static_cast<float>(a.token_offset + n + 1);
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
  const float seed = carry ? carry[static_cast<long long>(b) * P + p] : 0.f;
  float run = seed;
  float own = 0.f;
  for (int i = 0; i < chunks; ++i) {
    const int c = reverse ? chunks - 1 - i : i;
    const float t = base[static_cast<long long>(c) * P];
    base[static_cast<long long>(c) * P] = run;
    run += t;
    own += t;
  }
  if (total) total[static_cast<long long>(b) * P + p] = own;
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                       const float* __restrict__ denom, float scale, int chunks, int P) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (p >= P) return;
  const float* base = partial + static_cast<long long>(b) * chunks * P + p;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int c = 0;
  for (; c + 4 <= chunks; c += 4) {
    s0 += base[static_cast<long long>(c) * P];
    s1 += base[static_cast<long long>(c + 1) * P];
    s2 += base[static_cast<long long>(c + 2) * P];
    s3 += base[static_cast<long long>(c + 3) * P];
  }
  for (; c < chunks; ++c) s0 += base[static_cast<long long>(c) * P];
  float s = (s0 + s1) + (s2 + s3);
  s *= scale;
  if (denom) {
    const float d = denom[b];
    s = d != 0.f ? s / d : 0.f;  // a sample with no valid token aggregates to zero
  }
  out[static_cast<long long>(b) * P + p] = s;
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
  pom_rope rope;
};

// Causal backward, pass 1: partial[b, c, :] = sum over the chunk of dout[b, n, :] / (n + 1 + offset).
template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads) causal_bwd_sum_kernel(const AggBwdDev a) {
  const int p = (blockIdx.x * kThreads + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  if (p >= a.P) return;
  const T* g = static_cast<const T*>(a.dout) + static_cast<long long>(b) * a.N * a.ld_dout + p;
  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
  const int n0 = c * kChunk, n1 = min(a.N, n0 + kChunk);
#pragma unroll 4
  for (int n = n0; n < n1; ++n) {
    float v[VEC];
    Vec<T, VEC>::ld(g + n * a.ld_dout, v);
    const float inv = 1.f / static_cast<float>(a.token_offset + n + 1);
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = fmaf(v[e], inv, acc[e]);
  }
  float* part = a.partial + (static_cast<long long>(b) * a.chunks + c) * a.P + p;
#pragma unroll
  for (int e = 0; e < VEC; ++e) part[e] = acc[e];
}

// CAUSAL == false: the gradient reaching every token is w[b,n] * dH[b, :].
// CAUSAL == true : walk the chunk backwards; W[n] = suffix + sum_{m >= n} dout[m]/(m+1+offset).
// Either way: un-rotate, then dx = g * poly'(a) * act'(x) and the coefficient gradient sums.
template <typename T, int VEC, int KR, bool CAUSAL>
__global__ void __launch_bounds__(kThreads) agg_bwd_kernel(const AggBwdDev a) {
  const int u = (blockIdx.x * kThreads + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  const bool rope = a.rope.kind != POM_ROPE_NONE;
  const ColMap m = map_unit(u, a.P, a.rope.kind);
  if (!m.valid) return;
  Coefs<VEC, KR> cf;
  cf.load(a.coeff, m, a.K, rope);
  const T* x = static_cast<const T*>(a.x) + static_cast<long long>(b) * a.N * a.ldx;
  T* dx = static_cast<T*>(a.dx) + static_cast<long long>(b) * a.N * a.ld_dx;
  const T* dout = CAUSAL ? static_cast<const T*>(a.dout) + static_cast<long long>(b) * a.N * a.ld_dout : nullptr;
  float g1[VEC], g2[VEC];
  float dc1[VEC][KR], dc2[VEC][KR];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    if (CAUSAL) {
      const float* part = a.partial + (static_cast<long long>(b) * a.chunks + c) * a.P;
      g1[e] = part[m.p1 + e];
      g2[e] = rope ? part[m.p2 + e] : 0.f;
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
#pragma unroll 2
  for (int i = 0; i < n1 - n0; ++i) {
    const int n = CAUSAL ? (n1 - 1 - i) : (n0 + i);
    float x1[VEC], x2[VEC];
    Vec<T, VEC>::ld(x + n * a.ldx + m.p1, x1);
    if (rope) Vec<T, VEC>::ld(x + n * a.ldx + m.p2, x2);
    float w = wb;
    if (CAUSAL) {
      const float inv = 1.f / static_cast<float>(a.token_offset + n + 1);
      float v[VEC];
      Vec<T, VEC>::ld(dout + n * a.ld_dout + m.p1, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) g1[e] = fmaf(v[e], inv, g1[e]);
      if (rope) {
        Vec<T, VEC>::ld(dout + n * a.ld_dout + m.p2, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) g2[e] = fmaf(v[e], inv, g2[e]);
      }
    } else if (a.row_weight) {
      w *= __ldg(a.row_weight + static_cast<long long>(b) * a.N + n);
    }
    float d1[VEC], d2[VEC];
    if (rope) {
      float cs[VEC], sn[VEC];
      rope_coeffs<VEC>(a.rope, m, n, cs, sn);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        d1[e] = w * (g1[e] * cs[e] + g2[e] * sn[e]);
        d2[e] = w * (g2[e] * cs[e] - g1[e] * sn[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) d1[e] = w * g1[e];
    }
    float o[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float av = pom_act(x1[e]);
      o[e] = d1[e] * poly_grad_reg<KR>(av, cf.c1[e], a.K) * pom_act_grad(x1[e]);
      float pw = av;
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        if (k < a.K) {
          dc1[e][k] = fmaf(d1[e], pw, dc1[e][k]);
          pw *= av;
        }
      }
    }
    Vec<T, VEC>::st(dx + n * a.ld_dx + m.p1, o);
    if (rope) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float av = pom_act(x2[e]);
        o[e] = d2[e] * poly_grad_reg<KR>(av, cf.c2[e], a.K) * pom_act_grad(x2[e]);
        float pw = av;
#pragma unroll
        for (int k = 0; k < KR; ++k) {
          if (k < a.K) {
            dc2[e][k] = fmaf(d2[e], pw, dc2[e][k]);
            pw *= av;
          }
        }
      }
      Vec<T, VEC>::st(dx + n * a.ld_dx + m.p2, o);
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
  pom_rope rope;
};

template <typename T, int VEC, bool BWD>
__global__ void __launch_bounds__(kThreads) select_kernel(const SelDev a) {
  const int u = (blockIdx.x * kThreads + threadIdx.x) * VEC;
  const int c = blockIdx.y, b = blockIdx.z;
  const bool rope = a.rope.kind != POM_ROPE_NONE;
  const ColMap m = map_unit(u, a.P, a.rope.kind);
  if (!m.valid) return;
  const long long rowb = static_cast<long long>(b) * a.T;
  const T* z = static_cast<const T*>(a.z) + rowb * a.ld_z;
  float b1[VEC], b2[VEC], h1[VEC], h2[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    b1[e] = a.activated ? 0.f : a.bias[m.p1 + e];
    b2[e] = (rope && !a.activated) ? a.bias[m.p2 + e] : 0.f;
    h1[e] = h2[e] = 0.f;
    if (!a.h_per_token) {
      const float* H = static_cast<const float*>(a.H) + static_cast<long long>(b) * a.P;
      h1[e] = H[m.p1 + e];
      if (rope) h2[e] = H[m.p2 + e];
    }
  }
  float accH1[VEC], accH2[VEC], accB1[VEC], accB2[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) accH1[e] = accH2[e] = accB1[e] = accB2[e] = 0.f;
  const int t0 = c * kChunk, t1 = min(a.T, t0 + kChunk);
#pragma unroll 2
  for (int t = t0; t < t1; ++t) {
    float z1[VEC], z2[VEC], s1[VEC], s2[VEC], cs[VEC], sn[VEC];
    Vec<T, VEC>::ld(z + t * a.ld_z + m.p1, z1);
    if (rope) {
      Vec<T, VEC>::ld(z + t * a.ld_z + m.p2, z2);
      rope_coeffs<VEC>(a.rope, m, t, cs, sn);
    }
    if (a.h_per_token) {
      const T* H = static_cast<const T*>(a.H) + (rowb + t) * a.ld_h;
      Vec<T, VEC>::ld(H + m.p1, h1);
      if (rope) Vec<T, VEC>::ld(H + m.p2, h2);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      z1[e] += b1[e];
      const float r1 = a.activated ? z1[e] : pom_hardsigmoid(z1[e]);
      if (rope) {
        z2[e] += b2[e];
        const float r2 = a.activated ? z2[e] : pom_hardsigmoid(z2[e]);
        s1[e] = r1 * cs[e] - r2 * sn[e];
        s2[e] = r2 * cs[e] + r1 * sn[e];
      } else {
        s1[e] = r1;
      }
    }
    if (!BWD) {
      float o[VEC];
      T* sh = static_cast<T*>(a.sh) + (rowb + t) * a.ld_sh;
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = s1[e] * h1[e];
      Vec<T, VEC>::st(sh + m.p1, o);
      if (rope) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = s2[e] * h2[e];
        Vec<T, VEC>::st(sh + m.p2, o);
      }
    } else {
      const T* dsh = static_cast<const T*>(a.dsh) + (rowb + t) * a.ld_dsh;
      T* dz = static_cast<T*>(a.dz) + (rowb + t) * a.ld_dz;
      float g1[VEC], g2[VEC], dh1[VEC], dh2[VEC], o[VEC];
      Vec<T, VEC>::ld(dsh + m.p1, g1);
      if (rope) Vec<T, VEC>::ld(dsh + m.p2, g2);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        dh1[e] = g1[e] * s1[e];
        accH1[e] += dh1[e];
        const float t1v = g1[e] * h1[e];  // gradient of the rotated gate
        float ds1 = t1v;
        if (rope) {
          dh2[e] = g2[e] * s2[e];
          accH2[e] += dh2[e];
          const float t2v = g2[e] * h2[e];
          ds1 = t1v * cs[e] + t2v * sn[e];
          const float ds2 = t2v * cs[e] - t1v * sn[e];
          g2[e] = a.activated ? ds2 : ds2 * pom_hardsigmoid_grad(z2[e]);
          accB2[e] += g2[e];
        }
        o[e] = a.activated ? ds1 : ds1 * pom_hardsigmoid_grad(z1[e]);
        accB1[e] += o[e];
      }
      Vec<T, VEC>::st(dz + m.p1, o);
      if (rope) Vec<T, VEC>::st(dz + m.p2, g2);
      if (a.h_per_token) {
        T* dh = static_cast<T*>(a.dh_tok) + (rowb + t) * a.ld_dh;
        Vec<T, VEC>::st(dh + m.p1, dh1);
        if (rope) Vec<T, VEC>::st(dh + m.p2, dh2);
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

// ------------------------------------------------------------------ small element-wise
__global__ void state_merge_kernel(const float* hp, const float* hc, float* hn, float n_past, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) hn[i] = (n_past * hp[i] + hc[i]) / (n_past + 1.f);
}
__global__ void cast_f32_bf16_kernel(const float* s, __nv_bfloat16* d, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) d[i] = __float2bfloat16_rn(s[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* s, float* d, long long count) {
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

// Two channels per thread when every access stays naturally aligned.
int pick_vec(int P, int rope_kind, int dtype, std::initializer_list<long long> lds,
             std::initializer_list<const void*> ptrs) {
  const int unit = rope_kind == POM_ROPE_2D ? P / 4 : rope_kind == POM_ROPE_1D ? P / 2 : P;
  if (unit % 2) return 1;
  for (long long ld : lds)
    if (ld % 2) return 1;
  const uintptr_t mask = dtype == POM_BF16 ? 3u : 7u;
  for (const void* p : ptrs)
    if (p && (reinterpret_cast<uintptr_t>(p) & mask)) return 1;
  return 2;
}

dim3 walk_grid(int P, int rope_kind, int vec, int chunks, int B) {
  const int units = static_cast<int>(ceil_div(first_channels(P, rope_kind), vec));
  return dim3(static_cast<unsigned>(ceil_div(units, kThreads)), static_cast<unsigned>(chunks),
              static_cast<unsigned>(B));
}

#define POM_DISPATCH_T_VEC(dtype, vec, CALL)                   \
  do {                                                         \
    if ((dtype) == POM_BF16) {                                 \
      if ((vec) == 2) { CALL(__nv_bfloat16, 2); } else { CALL(__nv_bfloat16, 1); } \
    } else {                                                   \
      if ((vec) == 2) { CALL(float, 2); } else { CALL(float, 1); }                 \
    }                                                          \
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
  dim3 grid(static_cast<unsigned>(ceil_div(P, 128)), static_cast<unsigned>(B));
  reduce_partials_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(partial, out, denom, scale, chunks,
                                                                             P);
  count_launch();
  return check_launch();
}

int pom_poly_agg_fwd(const pom_agg_args* a, void* stream) {
  if (!a || !a->x || !a->coeff || !a->partial) return POM_ERR_NULL;
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
  d.rope = a->rope;
  const int vec = pick_vec(a->P, a->rope.kind, a->dtype, {a->ldx, a->causal ? a->ld_out : 0},
                           {a->x, a->causal ? a->out : nullptr});
  const dim3 grid = walk_grid(a->P, a->rope.kind, vec, d.chunks, a->B);
#define CALL_SUM(T, V)                                                      \
  if (a->K <= 4) agg_fwd_kernel<T, V, 4, false><<<grid, kThreads, 0, st>>>(d); \
  else agg_fwd_kernel<T, V, kMaxDegree, false><<<grid, kThreads, 0, st>>>(d)
  POM_DISPATCH_T_VEC(a->dtype, vec, CALL_SUM);
#undef CALL_SUM
  count_launch();
  rc = check_launch();
  if (rc || !a->causal) return rc;
  dim3 sgrid(static_cast<unsigned>(ceil_div(a->P, 128)), static_cast<unsigned>(a->B));
  chunk_scan_kernel<<<sgrid, 128, 0, st>>>(a->partial, a->carry, a->total, d.chunks, a->P, 0);
  count_launch();
#define CALL_PFX(T, V)                                                     \
  if (a->K <= 4) agg_fwd_kernel<T, V, 4, true><<<grid, kThreads, 0, st>>>(d); \
  else agg_fwd_kernel<T, V, kMaxDegree, true><<<grid, kThreads, 0, st>>>(d)
  POM_DISPATCH_T_VEC(a->dtype, vec, CALL_PFX);
#undef CALL_PFX
  count_launch();
  return check_launch();
}

int pom_poly_agg_bwd(const pom_agg_bwd_args* a, void* stream) {
  if (!a || !a->x || !a->coeff || !a->dx || !a->dcoeff_partial) return POM_ERR_NULL;
  if (a->B <= 0 || a->N <= 0 || a->P <= 0 || a->K < 1) return POM_ERR_BAD_SHAPE;
  if (a->K > kMaxDegree) return POM_ERR_K_TOO_LARGE;
  if (a->B > 65535 || pom_agg_chunks(a->N) > 65535) return POM_ERR_TOO_LARGE;
  if (a->dtype != POM_BF16 && a->dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  if (a->ldx < a->P || a->ld_dx < a->P) return POM_ERR_BAD_STRIDE;
  if (a->causal ? (!a->dout || !a->partial || a->ld_dout < a->P) : !a->dH) return POM_ERR_NULL;
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
  d.rope = a->rope;
  const int vec = pick_vec(a->P, a->rope.kind, a->dtype, {a->ldx, a->ld_dx, a->causal ? a->ld_dout : 0},
                           {a->x, a->dx, a->causal ? a->dout : nullptr});
  const dim3 grid = walk_grid(a->P, a->rope.kind, vec, d.chunks, a->B);
  if (a->causal) {
    // Plain column walk (no channel pairing) for the scaled chunk sums.
    const int v2 = (a->P % 2 == 0) ? vec : 1;
    const dim3 g1 = walk_grid(a->P, POM_ROPE_NONE, v2, d.chunks, a->B);
#define CALL_CS(T, V) causal_bwd_sum_kernel<T, V><<<g1, kThreads, 0, st>>>(d)
    POM_DISPATCH_T_VEC(a->dtype, v2, CALL_CS);
#undef CALL_CS
    count_launch();
    dim3 sgrid(static_cast<unsigned>(ceil_div(a->P, 128)), static_cast<unsigned>(a->B));
    chunk_scan_kernel<<<sgrid, 128, 0, st>>>(a->partial, a->carry, a->total, d.chunks, a->P, 1);
    count_launch();
    if (a->phase == 1) return check_launch();  // totals only
#define CALL_BC(T, V)                                                     \
  if (a->K <= 4) agg_bwd_kernel<T, V, 4, true><<<grid, kThreads, 0, st>>>(d); \
  else agg_bwd_kernel<T, V, kMaxDegree, true><<<grid, kThreads, 0, st>>>(d)
    POM_DISPATCH_T_VEC(a->dtype, vec, CALL_BC);
#undef CALL_BC
  } else {
#define CALL_BN(T, V)                                                      \
  if (a->K <= 4) agg_bwd_kernel<T, V, 4, false><<<grid, kThreads, 0, st>>>(d); \
  else agg_bwd_kernel<T, V, kMaxDegree, false><<<grid, kThreads, 0, st>>>(d)
    POM_DISPATCH_T_VEC(a->dtype, vec, CALL_BN);
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
  const int vec = pick_vec(d.P, d.rope.kind, dtype, lds, ptrs);
  const dim3 grid = walk_grid(d.P, d.rope.kind, vec, d.chunks, d.B);
  if (bwd) {
#define CALL_SB(T, V) select_kernel<T, V, true><<<grid, kThreads, 0, st>>>(d)
    POM_DISPATCH_T_VEC(dtype, vec, CALL_SB);
#undef CALL_SB
  } else {
#define CALL_SF(T, V) select_kernel<T, V, false><<<grid, kThreads, 0, st>>>(d)
    POM_DISPATCH_T_VEC(dtype, vec, CALL_SF);
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
  d.rope = a->rope;
  return select_common(d, a->dtype, true,
                       {a->ld_z, a->ld_dsh, a->ld_dz, a->h_per_token ? a->ld_h : 0, a->h_per_token ? a->ld_dh : 0},
                       {a->z, a->dsh, a->dz, a->h_per_token ? a->H : nullptr, a->h_per_token ? a->dh_tok : nullptr},
                       static_cast<cudaStream_t>(stream));
}

int pom_state_merge(const float* h_past, const float* h_cur, float* h_new, float n_past, int64_t count, void* stream) {
  if (!h_past || !h_cur || !h_new) return POM_ERR_NULL;
  if (count <= 0) return POM_ERR_BAD_SHAPE;
  state_merge_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      h_past, h_cur, h_new, n_past, count);
  count_launch();
  return check_launch();
}

int pom_cast_f32_to_bf16(const float* src, void* dst, int64_t count, void* stream) {
  if (!src || !dst) return POM_ERR_NULL;
  if (count <= 0) return POM_ERR_BAD_SHAPE;
  cast_f32_bf16_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst), count);
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
