// Host launchers for the tcgen05 GEMM engine and its fused PoM epilogues, plus
// the fp32 SIMT GEMM of the high-precision mode.
#include <cudaTypedefs.h>
#include <mutex>
#include "common.cuh"
#include "epilogues.cuh"
#include "gemm_launch.cuh"

using namespace pomk;
using namespace pomh;

namespace pomh {
std::atomic<long long> g_launches{0};
// 0: automatic choice, 1: always the one-CTA kernel, 2: always the two-CTA (pair) kernel.
std::atomic<int> g_gemm_mode{0};
}

namespace {

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
  if (mode < 0 || mode % 10 > 2 || (mode / 10) % 10 > 3 || mode / 100 > 1) return POM_ERR_UNSUPPORTED;
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
  if (!a || !a->coeff || (!a->partial && !a->causal)) return POM_ERR_NULL;
  if (a->K < 1) return POM_ERR_BAD_SHAPE;
  if (a->causal) return ctx_gemm_causal(a, status, static_cast<cudaStream_t>(stream));
  if (a->rope.kind != POM_ROPE_NONE) return ctx_gemm_rope(a, status, static_cast<cudaStream_t>(stream));
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
  if (!a || !a->bias || (!a->H && !a->causal) || !a->sh_out) return POM_ERR_NULL;
  if (a->causal) return gate_gemm_causal(a, status, static_cast<cudaStream_t>(stream));
  if (a->rope.kind != POM_ROPE_NONE) return gate_gemm_rope(a, status, static_cast<cudaStream_t>(stream));
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
  if (!a || !a->bias || !a->z || !a->g_out || !a->db_partial) return POM_ERR_NULL;
  if (a->causal) return gate_bwd_gemm_causal(a, status, static_cast<cudaStream_t>(stream));
  if (!a->H || !a->dh_partial) return POM_ERR_NULL;
  if (a->rope.kind != POM_ROPE_NONE) return gate_bwd_gemm_rope(a, status, static_cast<cudaStream_t>(stream));
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
