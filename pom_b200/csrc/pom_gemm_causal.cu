// Token-causal forms of the fused tensor-core phases (epilogues_causal.cuh) behind pom_ctx_gemm / pom_gate_gemm /
// pom_gate_bwd_gemm with `causal` set, and the scan over 32-token groups that links them.
#include "common.cuh"
#include "epilogues_causal.cuh"
#include "gemm_launch.cuh"

using namespace pomk;
using namespace pomh;

namespace {

struct PairShape {
  int q, sections;
};

// Channel pairing of the tile: the rotary one when a rotation is asked for, else first half | second half.
int pair_shape(const pom_rope& r, int P, PairShape* s) {
  if (r.kind == POM_ROPE_2D) {
    if (P % 64) return POM_ERR_UNSUPPORTED;  // two sections: a 16-pair sub-unit never reaches over their border
    *s = PairShape{P / 4, 2};
  } else if (r.kind == POM_ROPE_1D || r.kind == POM_ROPE_NONE) {
    if (P % 16) return POM_ERR_UNSUPPORTED;
    *s = PairShape{P / 2, 1};
  } else {
    return POM_ERR_UNSUPPORTED;
  }
  return POM_OK;
}

int make_rope(const pom_rope& r, const PairShape& ps, RopeEpi* e, EpiMaps* maps) {
  *e = RopeEpi{};
  if (r.kind == POM_ROPE_NONE) {  // identity rotation: nothing is read
    e->rotate = 0;
    e->pos_stride = 1;
    e->len[0] = e->len[1] = 1;
    return POM_OK;
  }
  if (!r.pos || !r.cos0 || !r.sin0) return POM_ERR_NULL;
  if (ps.sections == 2 && (!r.cos1 || !r.sin1)) return POM_ERR_NULL;
  if (r.pos_stride != ps.sections) return POM_ERR_BAD_STRIDE;
  e->rotate = 1;
  e->cos[0] = r.cos0, e->sin[0] = r.sin0;
  e->cos[1] = ps.sections == 2 ? r.cos1 : r.cos0;
  e->sin[1] = ps.sections == 2 ? r.sin1 : r.sin0;
  e->pos = reinterpret_cast<const long long*>(r.pos);
  e->pos_stride = r.pos_stride;
  e->len[0] = r.len0, e->len[1] = ps.sections == 2 ? r.len1 : r.len0;
  e->step[0] = r.step0, e->step[1] = ps.sections == 2 ? r.step1 : r.step0;
  for (int s = 0; s < ps.sections; ++s) {
    if (e->len[s] < 1) return POM_ERR_BAD_SHAPE;
    if (e->step[s] != 0 && e->step[s] != 1) return POM_ERR_UNSUPPORTED;
    int rc;
    if ((rc = make_lane_table_map(&maps->lane[2 * s], e->cos[s], ps.q, e->len[s]))) return rc;
    if ((rc = make_lane_table_map(&maps->lane[2 * s + 1], e->sin[s], ps.q, e->len[s]))) return rc;
  }
  return POM_OK;
}

inline int groups_of(int rows) { return (rows + 31) / 32; }

// ---------------------------------------------------------------- scan over groups
// Three small launches, parallel over (sample, segment of 32 groups, channel):
//   1. segment sums               scratch[b, s, p] = sum of the segment's group totals
//   2. exclusive scan of segments (serial over at most a few hundred segments per (b, p)), seeded with carry_in
//   3. in-place exclusive scan inside every segment, seeded with its segment carry
constexpr int kSeg = 32;

__global__ void __launch_bounds__(128) seg_sum_kernel(const float* __restrict__ sums, float* __restrict__ seg,
                                                      int groups, int segs, int P) {
  griddep_wait();  // launched with programmatic stream serialization
  griddep_launch();
  const int p = blockIdx.x * 128 + threadIdx.x, s = blockIdx.y, b = blockIdx.z;
  if (p >= P) return;
  const int g0 = s * kSeg, g1 = min(groups, g0 + kSeg);
  const float* src = sums + (static_cast<long long>(b) * groups + g0) * P + p;
  float a0 = 0.f, a1 = 0.f;
  int g = g0;
  for (; g + 1 < g1; g += 2, src += 2ll * P) a0 += src[0], a1 += src[P];
  if (g < g1) a0 += src[0];
  seg[(static_cast<long long>(b) * segs + s) * P + p] = a0 + a1;
}

// Loads of a batch are issued together and only then replaced by their running sums: one memory latency per batch
// instead of one per element (the sums are formed in the same order either way).
__global__ void __launch_bounds__(128) seg_scan_kernel(float* __restrict__ seg, const float* __restrict__ carry_in,
                                                       float* __restrict__ total_out, int segs, int P, int reverse) {
  griddep_wait();  // launched with programmatic stream serialization
  griddep_launch();
  const int p = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
  if (p >= P) return;
  float* base = seg + static_cast<long long>(b) * segs * P + p;
  float run = carry_in ? carry_in[static_cast<long long>(b) * P + p] : 0.f;
  float own = 0.f;
  constexpr int kBatch = 16;
  for (int i0 = 0; i0 < segs; i0 += kBatch) {
    float v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + j;
      v[j] = i < segs ? base[static_cast<long long>(reverse ? segs - 1 - i : i) * P] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + j;
      if (i < segs) {
        base[static_cast<long long>(reverse ? segs - 1 - i : i) * P] = run;
        run += v[j];
        own += v[j];
      }
    }
  }
  if (total_out) total_out[static_cast<long long>(b) * P + p] = own;
}

__global__ void __launch_bounds__(128) seg_apply_kernel(float* __restrict__ sums, const float* __restrict__ seg,
                                                        int groups, int segs, int P, int reverse) {
  griddep_wait();  // launched with programmatic stream serialization
  griddep_launch();
  const int p = blockIdx.x * 128 + threadIdx.x, s = blockIdx.y, b = blockIdx.z;
  if (p >= P) return;
  const int g0 = s * kSeg, g1 = min(groups, g0 + kSeg);
  const int n = g1 - g0;
  float run = seg[(static_cast<long long>(b) * segs + s) * P + p];
  float* base = sums + static_cast<long long>(b) * groups * P + p;
  float v[kSeg];
#pragma unroll
  for (int i = 0; i < kSeg; ++i) v[i] = i < n ? base[static_cast<long long>(reverse ? g1 - 1 - i : g0 + i) * P] : 0.f;
#pragma unroll
  for (int i = 0; i < kSeg; ++i) {
    if (i < n) {
      base[static_cast<long long>(reverse ? g1 - 1 - i : g0 + i) * P] = run;
      run += v[i];
    }
  }
}

}  // namespace

namespace pomh {

int ctx_gemm_causal(const pom_ctx_args* a, int* status, cudaStream_t st) {
  if (!a->pre_out || !a->group_sums) return POM_ERR_NULL;
  if (a->K > EpiCtxCausal::kMaxK || a->row_weight) return POM_ERR_UNSUPPORTED;
  PairShape ps;
  int rc = pair_shape(a->rope, a->P, &ps);
  if (rc) return rc;
  Operands o{a->X, a->Wpo, a->N, a->P, a->D, a->ldx, a->ldw, a->B, false, false};
  o.pair_q = ps.q;
  o.pair_sections = ps.sections;
  if ((rc = check_operands(o))) return rc;
  if (a->hp_out && (a->ld_hp % 8 || a->ld_hp < a->P || !aligned16(a->hp_out))) return POM_ERR_BAD_ALIGN;
  if (a->ld_pre % 8 || a->ld_pre < a->P || !aligned16(a->pre_out)) return POM_ERR_BAD_ALIGN;
  EpiCtxCausal::Params ep{};
  ep.coeff = a->coeff;
  ep.K = a->K;
  ep.save_hp = a->hp_out != nullptr;
  ep.causal.group_sums = a->group_sums;
  ep.causal.groups = groups_of(a->N);
  ep.causal.P = a->P;
  EpiMaps maps{};
  if ((rc = make_rope(a->rope, ps, &ep.rope, &maps))) return rc;
  if (a->hp_out && (rc = make_io_map_paired(&maps.out0, a->hp_out, ps.q, 2 * ps.sections, a->N, a->B, a->ld_hp)))
    return rc;
  if ((rc = make_io_map_paired(&maps.out1, a->pre_out, ps.q, 2 * ps.sections, a->N, a->B, a->ld_pre))) return rc;
  return run_plan<false, false, EpiCtxCausal>(pick_plan(o, true), o, 1, maps, ep, status, st);
}

int gate_gemm_causal(const pom_gate_args* a, int* status, cudaStream_t st) {
  if (!a->pre || !a->carry) return POM_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(a->carry) % 16) return POM_ERR_BAD_STRIDE;  // staged four columns per load
  PairShape ps;
  int rc = pair_shape(a->rope, a->P, &ps);
  if (rc) return rc;
  Operands o{a->X, a->Wse, a->T, a->P, a->D, a->ldx, a->ldw, a->B, false, false};
  o.pair_q = ps.q;
  o.pair_sections = ps.sections;
  if ((rc = check_operands(o))) return rc;
  if (a->ld_sh % 8 || a->ld_sh < a->P || !aligned16(a->sh_out)) return POM_ERR_BAD_ALIGN;
  if (a->z_out && (a->ld_z % 8 || a->ld_z < a->P || !aligned16(a->z_out))) return POM_ERR_BAD_ALIGN;
  if (a->ld_pre % 8 || a->ld_pre < a->P || !aligned16(a->pre)) return POM_ERR_BAD_ALIGN;
  EpiGateCausal::Params ep{};
  ep.bias = a->bias;
  ep.save_z = a->z_out != nullptr;
  ep.causal.carry = a->carry;
  ep.causal.groups = groups_of(a->T);
  ep.causal.token_offset = a->token_offset;
  ep.causal.P = a->P;
  EpiMaps maps{};
  if ((rc = make_rope(a->rope, ps, &ep.rope, &maps))) return rc;
  if (a->z_out && (rc = make_io_map_paired(&maps.out0, a->z_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_z)))
    return rc;
  if ((rc = make_io_map_paired(&maps.out1, a->sh_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_sh))) return rc;
  if ((rc = make_io_map_paired(&maps.in0, a->pre, ps.q, 2 * ps.sections, a->T, a->B, a->ld_pre))) return rc;
  return run_plan<false, false, EpiGateCausal>(pick_plan(o, true), o, 1, maps, ep, status, st);
}

int gate_bwd_gemm_causal(const pom_gate_bwd_args* a, int* status, cudaStream_t st) {
  if (!a->WoT || !a->pre || !a->carry || !a->suf_out || !a->group_sums) return POM_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(a->carry) % 16) return POM_ERR_BAD_STRIDE;  // staged four columns per load
  PairShape ps;
  int rc = pair_shape(a->rope, a->P, &ps);
  if (rc) return rc;
  Operands o{a->dY, a->WoT, a->T, a->P, a->D, a->ld_dy, a->ldwt, a->B, false, false};
  o.pair_q = ps.q;
  o.pair_sections = ps.sections;
  if ((rc = check_operands(o))) return rc;
  if (a->ld_g % 8 || a->ld_g < a->P || !aligned16(a->g_out) || a->ld_z % 8 || a->ld_z < a->P || !aligned16(a->z))
    return POM_ERR_BAD_ALIGN;
  if (a->ld_pre % 8 || a->ld_pre < a->P || !aligned16(a->pre) || a->ld_suf % 8 || a->ld_suf < a->P ||
      !aligned16(a->suf_out))
    return POM_ERR_BAD_ALIGN;
  EpiGateBwdCausal::Params ep{};
  ep.bias = a->bias;
  ep.db_partial = a->db_partial;
  ep.causal.carry = a->carry;
  ep.causal.group_sums = a->group_sums;
  ep.causal.groups = groups_of(a->T);
  ep.causal.token_offset = a->token_offset;
  ep.causal.P = a->P;
  EpiMaps maps{};
  if ((rc = make_rope(a->rope, ps, &ep.rope, &maps))) return rc;
  if ((rc = make_io_map_paired(&maps.in0, a->z, ps.q, 2 * ps.sections, a->T, a->B, a->ld_z))) return rc;
  if ((rc = make_io_map_paired(&maps.in1, a->pre, ps.q, 2 * ps.sections, a->T, a->B, a->ld_pre))) return rc;
  if ((rc = make_io_map_paired(&maps.out0, a->g_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_g))) return rc;
  if ((rc = make_io_map_paired(&maps.out1, a->suf_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_suf))) return rc;
  return run_plan<false, false, EpiGateBwdCausal>(pick_plan(o, true), o, 1, maps, ep, status, st);
}

}  // namespace pomh

extern "C" {

int pom_group_scan(float* sums, const float* carry_in, float* total_out, float* scratch, int32_t B, int32_t groups,
                   int32_t P, int32_t reverse, void* stream) {
  if (!sums || !scratch) return POM_ERR_NULL;
  if (B <= 0 || groups <= 0 || P <= 0) return POM_ERR_BAD_SHAPE;
  const int segs = static_cast<int>(ceil_div(groups, kSeg));
  if (B > 65535 || segs > 65535) return POM_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned px = static_cast<unsigned>(ceil_div(P, 128));
  (void)launch_pdl(seg_sum_kernel, dim3(px, segs, B), dim3(128), 0, st, static_cast<const float*>(sums), scratch, groups,
                   segs, P);
  (void)launch_pdl(seg_scan_kernel, dim3(px, B), dim3(128), 0, st, scratch, carry_in, total_out, segs, P, reverse);
  (void)launch_pdl(seg_apply_kernel, dim3(px, segs, B), dim3(128), 0, st, sums, static_cast<const float*>(scratch), groups,
                   segs, P, reverse);
  count_launch(3);
  return check_launch();
}

}  // extern "C"
