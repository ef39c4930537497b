// Multi-head scalar gating without the P-wide query side.
//
// With n_sel_heads > 1 the gate has one value per head, shared by the hd = P / heads channels of the head
// (reference pom/pom.py:119-122), so for a per-sample aggregate H (mask None or (B, N)) the output projection
// collapses:
//
//   y[b,t,d] = sum_p s[b,t,head(p)] * H[b,p] * Wo[d,p] = sum_h s[b,t,h] * Mb[b,h,d],
//   Mb[b,h,d] = sum_{p in head h} H[b,p] * Wo[d,p]
//
// The (B, T, P) tensor SH of the reference, the T x P x D output GEMM and their two backward GEMMs never exist:
// what remains is a (heads x D) matrix per sample and products with a 16-ish-wide inner dimension, all of which
// are bound by reading dy / writing y once.  Kernels here are plain SIMT (the inner dimension is far below a
// tensor-core tile); sums run in a fixed order.
#include <cuda_bf16.h>

#include "common.cuh"

using namespace pomh;

namespace {

constexpr int kMaxHeads = 64;

template <typename T>
__device__ __forceinline__ float ldf(const T* p) {
  if constexpr (sizeof(T) == 4) return *p;
  else return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void stf(T* p, float v) {
  if constexpr (sizeof(T) == 4) *p = v;
  else *p = __float2bfloat16_rn(v);
}

// Mb[b,h,d] = sum_j H[b, h*hd + j] * Wo[d, h*hd + j]; a thread owns one d and four samples.
template <typename T>
__global__ void __launch_bounds__(128) head_mix_kernel(const float* __restrict__ H, const T* __restrict__ Wo,
                                                       float* __restrict__ Mb, long long ldw, int B, int D, int P,
                                                       int heads) {
  const int d = blockIdx.x * 128 + threadIdx.x, h = blockIdx.y, b0 = blockIdx.z * 4;
  if (d >= D) return;
  const int hd = P / heads;
  const T* w = Wo + static_cast<long long>(d) * ldw + h * hd;
  const float* hb = H + static_cast<long long>(b0) * P + h * hd;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < hd; ++j) {
    const float wv = ldf(w + j);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (b0 + i < B) acc[i] = fmaf(hb[static_cast<long long>(i) * P + j], wv, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (b0 + i < B) Mb[(static_cast<long long>(b0 + i) * heads + h) * D + d] = acc[i];
}

// y[b,t,:] = sum_h s[b,t,h] * Mb[b,h,:] (+ residual).  CTA = 64 tokens of one sample; Mb[b] and the tokens' gate
// values sit in shared memory; a thread computes 4 tokens x 4 adjacent d at a time (one 16-byte read of Mb and four
// broadcast reads of s per 16 multiply-adds).  D % 4 == 0.
template <typename T>
__global__ void __launch_bounds__(256) heads_out_kernel(const float* __restrict__ s, const float* __restrict__ Mb,
                                                        const T* __restrict__ res, T* __restrict__ y, int Tn, int D,
                                                        int heads) {
  extern __shared__ __align__(16) float hs_smem[];
  float* mb = hs_smem;                 // [heads][D]
  float* st = hs_smem + heads * D;     // [64][heads], rows past the end zero
  const int b = blockIdx.y, t0 = blockIdx.x * 64;
  const int rows = min(64, Tn - t0);
  for (int i = threadIdx.x; i < heads * D; i += 256) mb[i] = Mb[static_cast<long long>(b) * heads * D + i];
  for (int i = threadIdx.x; i < 64 * heads; i += 256)
    st[i] = i < rows * heads ? s[(static_cast<long long>(b) * Tn + t0) * heads + i] : 0.f;
  __syncthreads();
  const int dq = D >> 2;  // groups of 4 columns
  const long long base = (static_cast<long long>(b) * Tn + t0) * D;
  for (int idx = threadIdx.x; idx < 16 * dq; idx += 256) {
    const int tg = idx / dq, d = (idx - tg * dq) * 4;  // consecutive threads: consecutive column groups, same tokens
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    for (int h = 0; h < heads; ++h) {
      const float4 m = *reinterpret_cast<const float4*>(mb + h * D + d);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float sv = st[(tg * 4 + i) * heads + h];
        acc[i][0] = fmaf(sv, m.x, acc[i][0]);
        acc[i][1] = fmaf(sv, m.y, acc[i][1]);
        acc[i][2] = fmaf(sv, m.z, acc[i][2]);
        acc[i][3] = fmaf(sv, m.w, acc[i][3]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = tg * 4 + i;
      if (t >= rows) break;
      const long long off = base + static_cast<long long>(t) * D + d;
      if constexpr (sizeof(T) == 2) {  // four bf16 values leave (and the residual arrives) as one 8-byte access
        if (res) {
          const uint2 q = *reinterpret_cast<const uint2*>(res + off);
          acc[i][0] += __uint_as_float(q.x << 16);
          acc[i][1] += __uint_as_float(q.x & 0xffff0000u);
          acc[i][2] += __uint_as_float(q.y << 16);
          acc[i][3] += __uint_as_float(q.y & 0xffff0000u);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[i][0], acc[i][1]);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[i][2], acc[i][3]);
        *reinterpret_cast<uint2*>(y + off) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      } else {
        float4 v = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        if (res) {
          const float4 q = *reinterpret_cast<const float4*>(res + off);
          v.x += q.x, v.y += q.y, v.z += q.z, v.w += q.w;
        }
        *reinterpret_cast<float4*>(y + off) = v;
      }
    }
  }
}

// ds[b,t,h] = sum_d dy[b,t,d] * Mb[b,h,d]: a warp takes 64 / HB tokens at a time, lanes stride over d and keep
// one accumulator per (token, head), so each shared-memory read of Mb feeds that many multiply-adds.
template <typename T, int HB>
__global__ void __launch_bounds__(256) heads_ds_kernel(const T* __restrict__ dy, const float* __restrict__ Mb,
                                                       float* __restrict__ ds, int Tn, int D, int heads) {
  extern __shared__ __align__(16) float hs_smem[];
  float* mb = hs_smem;  // [heads][D]
  const int b = blockIdx.y, t0 = blockIdx.x * 64;
  const int rows = min(64, Tn - t0);
  for (int i = threadIdx.x; i < heads * D; i += 256) mb[i] = Mb[static_cast<long long>(b) * heads * D + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int TW = 64 / HB;  // tokens per warp pass: 64 accumulators per lane whatever the head count
  for (int r0 = warp * TW; r0 < rows; r0 += 8 * TW) {
    const T* row = dy + (static_cast<long long>(b) * Tn + t0 + r0) * D;
    float acc[TW][HB];
#pragma unroll
    for (int i = 0; i < TW; ++i)
#pragma unroll
      for (int h = 0; h < HB; ++h) acc[i][h] = 0.f;
    for (int d = lane; d < D; d += 32) {
      float g[TW];
#pragma unroll
      for (int i = 0; i < TW; ++i) g[i] = r0 + i < rows ? ldf(row + static_cast<long long>(i) * D + d) : 0.f;
#pragma unroll
      for (int h = 0; h < HB; ++h) {
        if (h < heads) {
          const float m = mb[h * D + d];
#pragma unroll
          for (int i = 0; i < TW; ++i) acc[i][h] = fmaf(g[i], m, acc[i][h]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < TW; ++i)
#pragma unroll
      for (int h = 0; h < HB; ++h) {
        float v = acc[i][h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && h < heads && r0 + i < rows) ds[(static_cast<long long>(b) * Tn + t0 + r0 + i) * heads + h] = v;
      }
  }
}

// partial[(b, chunk), h, d] = sum over the chunk's 128 tokens of s[b,t,h] * dy[b,t,d]; a thread owns one d and reads
// a token's gate values as 16-byte broadcasts (rows padded to HB values with zeros).
template <typename T, int HB>
__global__ void __launch_bounds__(256) heads_dmb_kernel(const T* __restrict__ dy, const float* __restrict__ s,
                                                        float* __restrict__ partial, int Tn, int D, int heads) {
  __shared__ __align__(16) float st[64 * HB];  // [64][HB]
  const int b = blockIdx.y, c = blockIdx.x, t0 = c * 128;
  const int rows = min(128, Tn - t0);
  float* out = partial + (static_cast<long long>(b) * gridDim.x + c) * heads * D;
  // accumulators persist over the two 64-token halves of the chunk
  for (int dbase = 0; dbase < D; dbase += 256) {
    const int d = dbase + threadIdx.x;
    float acc[HB];
#pragma unroll
    for (int h = 0; h < HB; ++h) acc[h] = 0.f;
    for (int half = 0; half < 2; ++half) {
      const int r_lo = half * 64, r_hi = min(rows, r_lo + 64);
      __syncthreads();
      for (int i = threadIdx.x; i < 64 * HB; i += 256) {
        const int r = i / HB, h = i - r * HB;
        st[i] = (r_lo + r < r_hi && h < heads) ? s[(static_cast<long long>(b) * Tn + t0 + r_lo + r) * heads + h] : 0.f;
      }
      __syncthreads();
      if (d < D) {
        const T* col = dy + (static_cast<long long>(b) * Tn + t0 + r_lo) * D + d;
        for (int r = 0; r < r_hi - r_lo; ++r) {
          const float g = ldf(col + static_cast<long long>(r) * D);
#pragma unroll
          for (int q = 0; q < HB / 4; ++q) {
            const float4 sv = *reinterpret_cast<const float4*>(st + r * HB + 4 * q);
            acc[4 * q] = fmaf(sv.x, g, acc[4 * q]);
            acc[4 * q + 1] = fmaf(sv.y, g, acc[4 * q + 1]);
            acc[4 * q + 2] = fmaf(sv.z, g, acc[4 * q + 2]);
            acc[4 * q + 3] = fmaf(sv.w, g, acc[4 * q + 3]);
          }
        }
      }
    }
    if (d < D) {
#pragma unroll
      for (int h = 0; h < HB; ++h)
        if (h < heads) out[static_cast<long long>(h) * D + d] = acc[h];
    }
  }
}

// dH[b,p] = sum_d dMb[b,head(p),d] * Wo[d,p]; a thread owns one p and four samples.
template <typename T>
__global__ void __launch_bounds__(128) head_mix_dh_kernel(const float* __restrict__ dMb, const T* __restrict__ Wo,
                                                          float* __restrict__ dH, long long ldw, int B, int D, int P,
                                                          int heads) {
  const int p = blockIdx.x * 128 + threadIdx.x, b0 = blockIdx.y * 4;
  if (p >= P) return;
  const int h = p / (P / heads);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int d = 0; d < D; ++d) {
    const float wv = ldf(Wo + static_cast<long long>(d) * ldw + p);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (b0 + i < B) acc[i] = fmaf(dMb[(static_cast<long long>(b0 + i) * heads + h) * D + d], wv, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (b0 + i < B) dH[static_cast<long long>(b0 + i) * P + p] = acc[i];
}

// dWo[d,p] += sum_b dMb[b,head(p),d] * H[b,p]; a thread owns one p and eight rows d.
__global__ void __launch_bounds__(128) head_mix_dw_kernel(const float* __restrict__ dMb, const float* __restrict__ H,
                                                          float* __restrict__ dWo, int B, int D, int P, int heads) {
  const int p = blockIdx.x * 128 + threadIdx.x, d0 = blockIdx.y * 8;
  if (p >= P) return;
  const int h = p / (P / heads);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int b = 0; b < B; ++b) {
    const float hv = H[static_cast<long long>(b) * P + p];
    const float* m = dMb + (static_cast<long long>(b) * heads + h) * D + d0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (d0 + i < D) acc[i] = fmaf(m[i], hv, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (d0 + i < D) dWo[static_cast<long long>(d0 + i) * P + p] += acc[i];
}

int check(const pom_heads_args* a) {
  if (!a) return POM_ERR_NULL;
  if (a->B <= 0 || a->T <= 0 || a->D <= 0 || a->P <= 0 || a->heads < 2) return POM_ERR_BAD_SHAPE;
  if (a->heads > kMaxHeads || a->P % a->heads || a->D % 4) return POM_ERR_UNSUPPORTED;
  if (a->dtype != POM_BF16 && a->dtype != POM_F32) return POM_ERR_UNSUPPORTED;
  if (a->B > 65535) return POM_ERR_TOO_LARGE;
  return POM_OK;
}

size_t mb_smem(const pom_heads_args* a, int extra_floats) {
  return (static_cast<size_t>(a->heads) * a->D + extra_floats) * sizeof(float);
}

template <class Kern>
int allow_smem(Kern kern, size_t bytes) {
  if (bytes > 200 * 1024) return POM_ERR_TOO_LARGE;
  if (bytes > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) {
    (void)cudaGetLastError();
    return POM_ERR_CUDA;
  }
  return POM_OK;
}

}  // namespace

extern "C" {

int pom_heads_supported(int32_t heads, int32_t D, int32_t P) {
  return heads >= 2 && heads <= kMaxHeads && D > 0 && D % 4 == 0 && P > 0 && P % heads == 0 &&
         (static_cast<size_t>(heads) * D + 64 * heads) * sizeof(float) <= 200 * 1024;
}

int pom_heads_mix(const pom_heads_args* a, void* stream) {
  int rc = check(a);
  if (rc) return rc;
  if (!a->H || !a->Wo || !a->Mb) return POM_ERR_NULL;
  if (a->ldw < a->P) return POM_ERR_BAD_STRIDE;
  const dim3 grid(static_cast<unsigned>(ceil_div(a->D, 128)), static_cast<unsigned>(a->heads),
                  static_cast<unsigned>(ceil_div(a->B, 4)));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->dtype == POM_BF16)
    head_mix_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(a->H, static_cast<const __nv_bfloat16*>(a->Wo), a->Mb, a->ldw,
                                                         a->B, a->D, a->P, a->heads);
  else
    head_mix_kernel<float><<<grid, 128, 0, st>>>(a->H, static_cast<const float*>(a->Wo), a->Mb, a->ldw, a->B, a->D,
                                                 a->P, a->heads);
  count_launch();
  return check_launch();
}

int pom_heads_out_fwd(const pom_heads_args* a, void* stream) {
  int rc = check(a);
  if (rc) return rc;
  if (!a->s || !a->Mb || !a->y) return POM_ERR_NULL;
  const size_t smem = mb_smem(a, 64 * a->heads);
  const dim3 grid(static_cast<unsigned>(ceil_div(a->T, 64)), static_cast<unsigned>(a->B));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->dtype == POM_BF16) {
    if ((rc = allow_smem(heads_out_kernel<__nv_bfloat16>, smem))) return rc;
    heads_out_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(a->s, a->Mb, static_cast<const __nv_bfloat16*>(a->residual),
                                                             static_cast<__nv_bfloat16*>(a->y), a->T, a->D, a->heads);
  } else {
    if ((rc = allow_smem(heads_out_kernel<float>, smem))) return rc;
    heads_out_kernel<float><<<grid, 256, smem, st>>>(a->s, a->Mb, static_cast<const float*>(a->residual),
                                                     static_cast<float*>(a->y), a->T, a->D, a->heads);
  }
  count_launch();
  return check_launch();
}

#define POM_HEADS_BY_WIDTH(CALL)                 \
  do {                                           \
    if (a->heads <= 16) { CALL(16); }            \
    else if (a->heads <= 32) { CALL(32); }       \
    else { CALL(64); }                           \
  } while (0)

int pom_heads_out_bwd(const pom_heads_args* a, void* stream) {
  int rc = check(a);
  if (rc) return rc;
  if (!a->dy || !a->s || !a->Mb || !a->ds || !a->dMb_partial || !a->dMb) return POM_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = mb_smem(a, 0);
  const dim3 g1(static_cast<unsigned>(ceil_div(a->T, 64)), static_cast<unsigned>(a->B));
  const int chunks = static_cast<int>(ceil_div(a->T, 128));
  const dim3 g2(static_cast<unsigned>(chunks), static_cast<unsigned>(a->B));
#define CALL_DS(HB)                                                                                              \
  if (a->dtype == POM_BF16) {                                                                                    \
    if ((rc = allow_smem(heads_ds_kernel<__nv_bfloat16, HB>, smem))) return rc;                                  \
    heads_ds_kernel<__nv_bfloat16, HB><<<g1, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(a->dy), a->Mb,   \
                                                              a->ds, a->T, a->D, a->heads);                      \
    heads_dmb_kernel<__nv_bfloat16, HB><<<g2, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a->dy), a->s,      \
                                                            a->dMb_partial, a->T, a->D, a->heads);               \
  } else {                                                                                                       \
    if ((rc = allow_smem(heads_ds_kernel<float, HB>, smem))) return rc;                                          \
    heads_ds_kernel<float, HB><<<g1, 256, smem, st>>>(static_cast<const float*>(a->dy), a->Mb, a->ds, a->T,      \
                                                      a->D, a->heads);                                           \
    heads_dmb_kernel<float, HB><<<g2, 256, 0, st>>>(static_cast<const float*>(a->dy), a->s, a->dMb_partial,      \
                                                    a->T, a->D, a->heads);                                       \
  }
  POM_HEADS_BY_WIDTH(CALL_DS);
#undef CALL_DS
  count_launch(2);
  if ((rc = check_launch())) return rc;
  return pom_reduce_partials(a->dMb_partial, a->dMb, nullptr, 1.f, a->B, chunks, a->heads * a->D, stream);
}

int pom_heads_mix_bwd(const pom_heads_args* a, void* stream) {
  int rc = check(a);
  if (rc) return rc;
  if (!a->dMb || !a->H || !a->Wo || !a->dH || !a->dWo) return POM_ERR_NULL;
  if (a->ldw < a->P) return POM_ERR_BAD_STRIDE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 g1(static_cast<unsigned>(ceil_div(a->P, 128)), static_cast<unsigned>(ceil_div(a->B, 4)));
  if (a->dtype == POM_BF16)
    head_mix_dh_kernel<__nv_bfloat16><<<g1, 128, 0, st>>>(a->dMb, static_cast<const __nv_bfloat16*>(a->Wo), a->dH,
                                                          a->ldw, a->B, a->D, a->P, a->heads);
  else
    head_mix_dh_kernel<float><<<g1, 128, 0, st>>>(a->dMb, static_cast<const float*>(a->Wo), a->dH, a->ldw, a->B, a->D,
                                                  a->P, a->heads);
  const dim3 g2(static_cast<unsigned>(ceil_div(a->P, 128)), static_cast<unsigned>(ceil_div(a->D, 8)));
  head_mix_dw_kernel<<<g2, 128, 0, st>>>(a->dMb, a->H, a->dWo, a->B, a->D, a->P, a->heads);
  count_launch(2);
  return check_launch();
}

}  // extern "C"
