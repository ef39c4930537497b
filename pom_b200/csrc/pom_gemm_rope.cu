// Fused tensor-core phases of the layer with rotary position embedding: host launchers of the paired-column
// GEMMs (epilogues_rope.cuh) behind pom_ctx_gemm / pom_gate_gemm / pom_gate_bwd_gemm, plus two small helpers:
// the position scan that tells the host which angle scheme the positions allow, and a bf16 transpose.
#include <climits>
#include "common.cuh"
#include "epilogues_rope.cuh"
#include "gemm_launch.cuh"

using namespace pomk;
using namespace pomh;

namespace {

struct PairShape {
  int q;         // first channels per section
  int sections;  // 1 (1-D) or 2 (2-D: row half, column half)
};

int pair_shape(const pom_rope& r, int P, PairShape* s) {
  if (r.kind == POM_ROPE_1D) {
    if (P % 16) return POM_ERR_UNSUPPORTED;
    *s = PairShape{P / 2, 1};
  } else if (r.kind == POM_ROPE_2D) {
    if (P % 64) return POM_ERR_UNSUPPORTED;  // two sections: a 16-pair sub-unit never reaches over their border
    *s = PairShape{P / 4, 2};
  } else {
    return POM_ERR_UNSUPPORTED;
  }
  return POM_OK;
}

// Fills the device-side rotary description and the lane-table tensor maps.
int make_rope(const pom_rope& r, const PairShape& ps, RopeEpi* e, EpiMaps* maps) {
  if (!r.pos || !r.cos0 || !r.sin0) return POM_ERR_NULL;
  if (ps.sections == 2 && (!r.cos1 || !r.sin1)) return POM_ERR_NULL;
  if (r.pos_stride != ps.sections) return POM_ERR_BAD_STRIDE;
  e->cos[0] = r.cos0, e->sin[0] = r.sin0;
  e->cos[1] = ps.sections == 2 ? r.cos1 : r.cos0;
  e->sin[1] = ps.sections == 2 ? r.sin1 : r.sin0;
  e->pos = reinterpret_cast<const long long*>(r.pos);
  e->pos_stride = r.pos_stride;
  e->rotate = 1;
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

// ---------------------------------------------------------------- position scan
// One CTA: per column of the positions, min / max and whether every aligned 32-token group is constant /
// consecutive.  Thread i owns tokens i, i + 1024, ... (a warp therefore always holds one aligned group).
__global__ void __launch_bounds__(1024) rope_pos_info_kernel(const long long* __restrict__ pos, long long n, int stride,
                                                             long long* __restrict__ info) {
  __shared__ long long s_min[2][32], s_max[2][32];
  __shared__ int s_flat[2][32], s_step[2][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c = 0; c < stride; ++c) {
    long long mn = LLONG_MAX, mx = LLONG_MIN;
    int flat = 1, step = 1;
    for (long long base = 0; base < n; base += 1024) {
      const long long i = base + threadIdx.x;
      const bool ok = i < n;
      const long long p = ok ? pos[i * stride + c] : 0;
      const long long p0 = __shfl_sync(0xffffffffu, p, 0);  // lane 0 of a group that has any token is valid
      if (ok) {
        mn = p < mn ? p : mn;
        mx = p > mx ? p : mx;
        if (p != p0) flat = 0;
        if (p != p0 + lane) step = 0;
      }
    }
    for (int off = 16; off; off >>= 1) {
      const long long omn = __shfl_xor_sync(0xffffffffu, mn, off), omx = __shfl_xor_sync(0xffffffffu, mx, off);
      mn = omn < mn ? omn : mn;
      mx = omx > mx ? omx : mx;
      flat &= __shfl_xor_sync(0xffffffffu, flat, off);
      step &= __shfl_xor_sync(0xffffffffu, step, off);
    }
    if (lane == 0) s_min[c][warp] = mn, s_max[c][warp] = mx, s_flat[c][warp] = flat, s_step[c][warp] = step;
  }
  __syncthreads();
  if (threadIdx.x < stride) {
    const int c = threadIdx.x;
    long long mn = LLONG_MAX, mx = LLONG_MIN;
    int flat = 1, step = 1;
    for (int w = 0; w < 32; ++w) {
      mn = s_min[c][w] < mn ? s_min[c][w] : mn;
      mx = s_max[c][w] > mx ? s_max[c][w] : mx;
      flat &= s_flat[c][w];
      step &= s_step[c][w];
    }
    info[4 * c + 0] = mn, info[4 * c + 1] = mx, info[4 * c + 2] = flat, info[4 * c + 3] = step;
  }
}

// 32 x 32 tiles through shared memory; rows / cols need no alignment.
__global__ void __launch_bounds__(256) transpose_bf16_kernel(const __nv_bfloat16* __restrict__ src,
                                                             __nv_bfloat16* __restrict__ dst, long long rows,
                                                             long long cols, long long ld_src, long long ld_dst) {
  __shared__ __nv_bfloat16 tile[32][34];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long c0 = static_cast<long long>(blockIdx.x) * 32, r0 = static_cast<long long>(blockIdx.y) * 32;
  for (int r = ty; r < 32; r += 8)
    if (r0 + r < rows && c0 + tx < cols) tile[r][tx] = src[(r0 + r) * ld_src + c0 + tx];
  __syncthreads();
  for (int c = ty; c < 32; c += 8)
    if (c0 + c < cols && r0 + tx < rows) dst[(c0 + c) * ld_dst + r0 + tx] = tile[tx][c];
}

}  // namespace

namespace pomh {

int ctx_gemm_rope(const pom_ctx_args* a, int* status, cudaStream_t st) {
  if (a->K > EpiCtxRope::kMaxK) return POM_ERR_UNSUPPORTED;
  PairShape ps;
  int rc = pair_shape(a->rope, a->P, &ps);
  if (rc) return rc;
  Operands o{a->X, a->Wpo, a->N, a->P, a->D, a->ldx, a->ldw, a->B, false, false};
  o.tile_weight = a->row_weight ? a->tile_weight : nullptr;
  o.pair_q = ps.q;
  o.pair_sections = ps.sections;
  if ((rc = check_operands(o))) return rc;
  if (a->hp_out && (a->ld_hp % 8 || a->ld_hp < a->P || !aligned16(a->hp_out))) return POM_ERR_BAD_ALIGN;
  EpiCtxRope::Params ep;
  ep.coeff = a->coeff;
  ep.K = a->K;
  ep.row_weight = a->row_weight;
  ep.save_hp = a->hp_out != nullptr;
  ep.partial = a->partial;
  ep.P = a->P;
  EpiMaps maps{};
  if ((rc = make_rope(a->rope, ps, &ep.rope, &maps))) return rc;
  if (a->hp_out && (rc = make_io_map_paired(&maps.out0, a->hp_out, ps.q, 2 * ps.sections, a->N, a->B, a->ld_hp)))
    return rc;
  return run_plan<false, false, EpiCtxRope>(pick_plan(o, true), o, 1, maps, ep, status, st);
}

int gate_gemm_rope(const pom_gate_args* a, int* status, cudaStream_t st) {
  PairShape ps;
  int rc = pair_shape(a->rope, a->P, &ps);
  if (rc) return rc;
  Operands o{a->X, a->Wse, a->T, a->P, a->D, a->ldx, a->ldw, a->B, false, false};
  o.pair_q = ps.q;
  o.pair_sections = ps.sections;
  if ((rc = check_operands(o))) return rc;
  if (a->h_row_stride != 0) return POM_ERR_UNSUPPORTED;
  if (a->ld_sh % 8 || a->ld_sh < a->P || !aligned16(a->sh_out)) return POM_ERR_BAD_ALIGN;
  if (a->z_out && (a->ld_z % 8 || a->ld_z < a->P || !aligned16(a->z_out))) return POM_ERR_BAD_ALIGN;
  EpiGateRope::Params ep;
  ep.bias = a->bias;
  ep.H = a->H;
  ep.h_batch_stride = a->h_batch_stride;
  ep.save_z = a->z_out != nullptr;
  EpiMaps maps{};
  if ((rc = make_rope(a->rope, ps, &ep.rope, &maps))) return rc;
  if (a->z_out && (rc = make_io_map_paired(&maps.out0, a->z_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_z)))
    return rc;
  if ((rc = make_io_map_paired(&maps.out1, a->sh_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_sh))) return rc;
  return run_plan<false, false, EpiGateRope>(pick_plan(o, true), o, 1, maps, ep, status, st);
}

int gate_bwd_gemm_rope(const pom_gate_bwd_args* a, int* status, cudaStream_t st) {
  if (!a->WoT) return POM_ERR_NULL;
  PairShape ps;
  int rc = pair_shape(a->rope, a->P, &ps);
  if (rc) return rc;
  // dSH[t, p] = sum_d dY[t, d] * WoT[p, d]
  Operands o{a->dY, a->WoT, a->T, a->P, a->D, a->ld_dy, a->ldwt, a->B, false, false};
  o.pair_q = ps.q;
  o.pair_sections = ps.sections;
  if ((rc = check_operands(o))) return rc;
  if (a->ld_g % 8 || a->ld_g < a->P || !aligned16(a->g_out) || a->ld_z % 8 || a->ld_z < a->P || !aligned16(a->z))
    return POM_ERR_BAD_ALIGN;
  EpiGateBwdRope::Params ep;
  ep.bias = a->bias;
  ep.H = a->H;
  ep.h_batch_stride = a->h_batch_stride;
  ep.dh_partial = a->dh_partial;
  ep.db_partial = a->db_partial;
  ep.P = a->P;
  EpiMaps maps{};
  if ((rc = make_rope(a->rope, ps, &ep.rope, &maps))) return rc;
  if ((rc = make_io_map_paired(&maps.in0, a->z, ps.q, 2 * ps.sections, a->T, a->B, a->ld_z))) return rc;
  if ((rc = make_io_map_paired(&maps.out0, a->g_out, ps.q, 2 * ps.sections, a->T, a->B, a->ld_g))) return rc;
  return run_plan<false, false, EpiGateBwdRope>(pick_plan(o, true), o, 1, maps, ep, status, st);
}

}  // namespace pomh

extern "C" {

int pom_rope_pos_info(const int64_t* pos, int64_t n, int32_t pos_stride, int64_t* info, void* stream) {
  if (!pos || !info) return POM_ERR_NULL;
  if (n <= 0 || (pos_stride != 1 && pos_stride != 2)) return POM_ERR_BAD_SHAPE;
  rope_pos_info_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(pos), n, pos_stride, reinterpret_cast<long long*>(info));
  count_launch();
  return check_launch();
}

int pom_transpose_bf16(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst,
                       void* stream) {
  if (!src || !dst) return POM_ERR_NULL;
  if (rows <= 0 || cols <= 0 || ld_src < cols || ld_dst < rows) return POM_ERR_BAD_SHAPE;
  if (ceil_div(rows, 32) > 65535) return POM_ERR_TOO_LARGE;
  dim3 grid(static_cast<unsigned>(ceil_div(cols, 32)), static_cast<unsigned>(ceil_div(rows, 32)));
  transpose_bf16_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols, ld_src, ld_dst);
  count_launch();
  return check_launch();
}

}  // extern "C"
