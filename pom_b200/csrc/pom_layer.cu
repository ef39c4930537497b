// Whole-layer entry points (bf16, fused path): the reference's PoM.forward / PoM.state_forward and their
// autograd as two calls, pom_layer_fwd and pom_layer_bwd, that enqueue the tensor-core phases, the small
// reductions between them and the streamed aggregation backward on one stream.  Host-side sequencing only: every
// kernel belongs to the phase entry points of this library, which stay available for hosts that need to put an
// exchange between the phases (token sharding) or that use the operator path (fp32, unusual positions).  Rotary
// embedding and the token-causal mask ride in the same phases (pom_layer_args::rope_c / rope_q / causal).
#include "common.cuh"
#include <cuda_bf16.h>

using namespace pomh;

namespace {

inline uint64_t align_up(uint64_t v) { return (v + 255u) & ~static_cast<uint64_t>(255u); }
inline int m_tiles(int rows) { return (rows + 127) / 128; }

struct Workspace {
  // forward
  uint64_t ctx_partial;   // (B, MT_N, P) fp32
  uint64_t h_tmp;         // (B, P) fp32: aggregate before the frame / state merge
  uint64_t tile_w;        // (B, MT_N) fp32: mask weight of every 128-token tile
  // backward
  uint64_t dh_partial;    // (B, MT_T, P)
  uint64_t db_partial;    // (B, MT_T, P)
  uint64_t dc_partial;    // (B * chunks_N, P * K)
  uint64_t dh;            // (B, P)
  uint64_t dh2;           // (B, P)
  // token-causal
  uint64_t scan;          // (B, ceil(groups/32), P) fp32: scratch of pom_group_scan (both calls)
  uint64_t suf;           // (B, N, P) bf16: running sums of the gradient of the prefix means (backward)
  uint64_t gsum;          // (B, groups, P) fp32: their group totals, then carries (backward)
  uint64_t total;
};

inline int groups_of(int rows) { return (rows + 31) / 32; }

Workspace carve(const pom_layer_args* a) {
  Workspace w;
  const uint64_t bp = static_cast<uint64_t>(a->B) * a->P * sizeof(float);
  uint64_t off = 0;
  w.ctx_partial = off;
  off = align_up(off + static_cast<uint64_t>(m_tiles(a->N)) * bp);
  w.h_tmp = off;
  off = align_up(off + bp);
  w.tile_w = off;
  off = align_up(off + static_cast<uint64_t>(a->B) * m_tiles(a->N) * sizeof(float));
  w.scan = off;
  if (a->causal) off = align_up(off + static_cast<uint64_t>((groups_of(a->N) + 31) / 32) * bp);
  const uint64_t fwd_end = off;
  // the backward regions reuse the buffer from its start (the scan scratch keeps its place: it is free again then)
  off = 0;
  w.dh_partial = off;
  off = align_up(off + static_cast<uint64_t>(m_tiles(a->T)) * bp);
  w.db_partial = off;
  off = align_up(off + static_cast<uint64_t>(m_tiles(a->T)) * bp);
  w.dc_partial = off;
  off = align_up(off + static_cast<uint64_t>(pom_agg_chunks(a->N)) * bp * a->K);
  w.dh = off;
  off = align_up(off + bp);
  w.dh2 = off;
  off = align_up(off + bp);
  w.suf = w.gsum = off;
  if (a->causal) {
    if (off < fwd_end) off = fwd_end;  // past the scan scratch
    w.suf = off;
    off = align_up(off + static_cast<uint64_t>(a->B) * a->N * a->P * 2);
    w.gsum = off;
    off = align_up(off + static_cast<uint64_t>(groups_of(a->N)) * bp);
  }
  w.total = off > fwd_end ? off : fwd_end;
  return w;
}

int check_common(const pom_layer_args* a) {
  if (!a || !a->xq || !a->w_qc || !a->w_ag || !a->se_bias || !a->coeff || !a->workspace) return POM_ERR_NULL;
  if (!a->causal && !a->H) return POM_ERR_NULL;
  if (a->B <= 0 || a->T <= 0 || a->N <= 0 || a->D <= 0 || a->P <= 0 || a->K < 1) return POM_ERR_BAD_SHAPE;
  if (a->K > 16) return POM_ERR_K_TOO_LARGE;
  if (a->D % 8 || a->P % 8) return POM_ERR_BAD_ALIGN;
  if (a->self_mixing && a->T != a->N) return POM_ERR_BAD_SHAPE;
  if (!a->self_mixing && !a->xc) return POM_ERR_NULL;
  if (a->frames < 1 || a->B % a->frames) return POM_ERR_BAD_SHAPE;
  if (a->frames > 1 && (a->mask || a->h_past)) return POM_ERR_UNSUPPORTED;
  if (a->mask && !a->denom) return POM_ERR_NULL;
  if (a->causal) {
    if (a->causal != 1 || a->T != a->N || a->mask || a->frames != 1 || a->h_past) return POM_ERR_UNSUPPORTED;
    if (!a->pre || !a->carry) return POM_ERR_NULL;
  }
  if (a->workspace_bytes < carve(a).total) return POM_ERR_TOO_LARGE;
  return POM_OK;
}

template <typename T>
T* at(const pom_layer_args* a, uint64_t off) {
  return reinterpret_cast<T*>(static_cast<char*>(a->workspace) + off);
}

const __nv_bfloat16* bf(const void* p) { return static_cast<const __nv_bfloat16*>(p); }

#define POM_TRY(expr)            \
  do {                           \
    const int rc_ = (expr);      \
    if (rc_ != POM_OK) return rc_; \
  } while (0)

int gemm(const void* A, const void* Bm, void* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
         bool a_mn, bool b_mn, int out_mode, const void* residual, int64_t ldr, int* status, void* stream) {
  pom_gemm_args g{};
  g.A = A;
  g.Bm = Bm;
  g.C = C;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = lda;
  g.ldb = ldb;
  g.ldc = ldc;
  g.batches = 1;
  g.a_mn_major = a_mn;
  g.b_mn_major = b_mn;
  g.out_mode = out_mode;
  g.split_k = 0;
  g.alpha = 1.f;
  g.residual = residual;
  g.ldr = ldr;
  return pom_gemm_bf16(&g, status, stream);
}

// dX (and dXc) = G·Wqc, dWqc += Gᵀ·X: the last launches of the backward call, whatever produced G = [dhp | dz].
int input_and_weight_grads(const pom_layer_args* a, __nv_bfloat16* G, __nv_bfloat16* g_hp, __nv_bfloat16* g_z,
                           float* d_wqc, int* status, void* stream) {
  const int D = a->D, P = a->P;
  const int64_t rows_q = static_cast<int64_t>(a->B) * a->T, rows_c = static_cast<int64_t>(a->B) * a->N;
  if (a->self_mixing) {
    POM_TRY(gemm(G, a->w_qc, a->dxq, rows_q, D, 2LL * P, 2LL * P, D, D, false, true, POM_OUT_BF16, nullptr, 0, status,
                 stream));
    return gemm(G, a->xq, d_wqc, 2LL * P, D, rows_q, 2LL * P, D, D, true, true, POM_OUT_F32_ACCUM, nullptr, 0, status,
                stream);
  }
  const __nv_bfloat16* w_se = bf(a->w_qc) + static_cast<int64_t>(P) * D;
  POM_TRY(gemm(g_hp, a->w_qc, a->dxc, rows_c, D, P, P, D, D, false, true, POM_OUT_BF16, nullptr, 0, status, stream));
  POM_TRY(gemm(g_z, w_se, a->dxq, rows_q, D, P, P, D, D, false, true, POM_OUT_BF16, nullptr, 0, status, stream));
  POM_TRY(gemm(g_hp, a->xc, d_wqc, P, D, rows_c, P, D, D, true, true, POM_OUT_F32_ACCUM, nullptr, 0, status, stream));
  return gemm(g_z, a->xq, d_wqc + static_cast<int64_t>(P) * D, P, D, rows_q, P, D, D, true, true, POM_OUT_F32_ACCUM,
              nullptr, 0, status, stream);
}

}  // namespace

extern "C" {

uint64_t pom_layer_workspace_bytes(const pom_layer_args* a) {
  if (!a || a->B <= 0 || a->T <= 0 || a->N <= 0 || a->P <= 0 || a->K < 1) return 0;
  return carve(a).total;
}

int pom_layer_fwd(const pom_layer_args* a, int* status, void* stream) {
  POM_TRY(check_common(a));
  if (!a->y || !a->sh) return POM_ERR_NULL;
  if (a->save && (!a->hp || !a->z)) return POM_ERR_NULL;
  const Workspace w = carve(a);
  const void* xc = a->self_mixing ? a->xq : a->xc;
  const __nv_bfloat16* w_po = bf(a->w_qc);
  const __nv_bfloat16* w_se = bf(a->w_qc) + static_cast<int64_t>(a->P) * a->D;
  const int64_t BP = static_cast<int64_t>(a->B) * a->P;

  if (a->mask) {  // denominators (valid context tokens per sample) and the weight of every 128-token tile
    POM_TRY(pom_reduce_partials(a->mask, a->denom, nullptr, 1.f, a->B, a->N, 1, stream));
    POM_TRY(pom_tile_weights(a->mask, at<float>(a, w.tile_w), a->B, a->N, stream));
  }

  pom_ctx_args c{};
  c.X = xc;
  c.Wpo = w_po;
  c.coeff = a->coeff;
  c.row_weight = a->mask;
  c.tile_weight = a->mask ? at<float>(a, w.tile_w) : nullptr;  // tiles that the mask empties are skipped
  c.hp_out = a->save ? a->hp : nullptr;
  c.partial = at<float>(a, w.ctx_partial);
  c.ldx = a->D;
  c.ldw = a->D;
  c.ld_hp = a->P;
  c.B = a->B;
  c.N = a->N;
  c.D = a->D;
  c.P = a->P;
  c.K = a->K;
  c.rope = a->rope_c;
  const int64_t rows = static_cast<int64_t>(a->B) * a->T;
  if (a->causal) {
    // running sums per 32-token group in the context epilogue, carries across groups, prefix means in the gate epilogue
    c.causal = 1;
    c.pre_out = a->pre;
    c.ld_pre = a->P;
    c.group_sums = a->carry;
    POM_TRY(pom_ctx_gemm(&c, status, stream));
    POM_TRY(pom_group_scan(a->carry, nullptr, nullptr, at<float>(a, w.scan), a->B, groups_of(a->N), a->P, 0, stream));
    pom_gate_args g{};
    g.X = a->xq;
    g.Wse = w_se;
    g.bias = a->se_bias;
    g.z_out = a->save ? a->z : nullptr;
    g.sh_out = a->sh;
    g.ldx = a->D;
    g.ldw = a->D;
    g.ld_z = a->P;
    g.ld_sh = a->P;
    g.B = a->B;
    g.T = a->T;
    g.D = a->D;
    g.P = a->P;
    g.rope = a->rope_q;
    g.causal = 1;
    g.pre = a->pre;
    g.ld_pre = a->P;
    g.carry = a->carry;
    g.token_offset = a->token_offset;
    POM_TRY(pom_gate_gemm(&g, status, stream));
    return gemm(a->sh, a->w_ag, a->y, rows, a->D, a->P, a->P, a->P, a->D, false, false, POM_OUT_BF16, a->residual,
                a->D, status, stream);
  }
  POM_TRY(pom_ctx_gemm(&c, status, stream));

  const bool post = a->frames > 1 || a->h_past;
  float* h_first = post ? at<float>(a, w.h_tmp) : a->H;
  POM_TRY(pom_reduce_partials(c.partial, h_first, a->mask ? a->denom : nullptr, a->mask ? 1.f : 1.f / a->N, a->B,
                              m_tiles(a->N), a->P, stream));
  if (a->frames > 1) POM_TRY(pom_frame_prefix_mean(h_first, a->H, a->B / a->frames, a->frames, a->P, 0, stream));
  if (a->h_past) POM_TRY(pom_state_merge(a->h_past, h_first, a->H, a->n_past, BP, stream));

  pom_gate_args g{};
  g.X = a->xq;
  g.Wse = w_se;
  g.bias = a->se_bias;
  g.H = a->H;
  g.z_out = a->save ? a->z : nullptr;
  g.sh_out = a->sh;
  g.ldx = a->D;
  g.ldw = a->D;
  g.ld_z = a->P;
  g.ld_sh = a->P;
  g.h_batch_stride = a->P;
  g.h_row_stride = 0;
  g.B = a->B;
  g.T = a->T;
  g.D = a->D;
  g.P = a->P;
  g.rope = a->rope_q;
  POM_TRY(pom_gate_gemm(&g, status, stream));

  return gemm(a->sh, a->w_ag, a->y, rows, a->D, a->P, a->P, a->P, a->D, false, false, POM_OUT_BF16, a->residual, a->D,
              status, stream);
}

int pom_layer_bwd(const pom_layer_args* a, int* status, void* stream) {
  POM_TRY(check_common(a));
  if (!a->dy || !a->hp || !a->z || !a->sh || !a->G || !a->dxq || !a->grads) return POM_ERR_NULL;
  if (!a->self_mixing && !a->dxc) return POM_ERR_NULL;
  const bool rot_q = a->rope_q.kind != POM_ROPE_NONE;
  if ((rot_q || a->causal) && !a->w_ag_t) return POM_ERR_NULL;
  const Workspace w = carve(a);
  const int B = a->B, T = a->T, N = a->N, D = a->D, P = a->P, K = a->K;
  const int64_t rows_q = static_cast<int64_t>(B) * T, rows_c = static_cast<int64_t>(B) * N;
  const int64_t n_qc = 2LL * P * D, n_ag = static_cast<int64_t>(D) * P;
  float* d_wqc = a->grads;
  float* d_wag = a->grads + n_qc;
  float* d_bias = d_wag + n_ag;
  float* d_coeff = d_bias + P;
  POM_TRY(pom_fill_zero(a->grads, (n_qc + n_ag + P + static_cast<int64_t>(P) * K) * sizeof(float), stream));

  // dWo[d, p] = sum_t dY[t, d] * SH[t, p]
  POM_TRY(gemm(a->dy, a->sh, d_wag, D, P, rows_q, D, P, P, true, true, POM_OUT_F32_ACCUM, nullptr, 0, status, stream));

  // G = [dhp | dz]: one (rows, 2P) matrix under self-mixing, two separate ones otherwise
  __nv_bfloat16* G = static_cast<__nv_bfloat16*>(a->G);
  __nv_bfloat16* g_hp = G;
  __nv_bfloat16* g_z = a->self_mixing ? G + P : G + rows_c * P;
  const int64_t ld_g = a->self_mixing ? 2LL * P : P;

  pom_gate_bwd_args gb{};
  gb.dY = a->dy;
  gb.Wo = a->w_ag;
  gb.bias = a->se_bias;
  gb.H = a->H;
  gb.z = a->z;
  gb.g_out = g_z;
  gb.dh_partial = at<float>(a, w.dh_partial);
  gb.db_partial = at<float>(a, w.db_partial);
  gb.ld_dy = D;
  gb.ldw = P;
  gb.ld_z = P;
  gb.ld_g = ld_g;
  gb.h_batch_stride = P;
  gb.B = B;
  gb.T = T;
  gb.D = D;
  gb.P = P;
  gb.rope = a->rope_q;
  gb.WoT = a->w_ag_t;
  gb.ldwt = D;
  pom_agg_bwd_args ab{};
  ab.x = a->hp;
  ab.coeff = a->coeff;
  ab.dx = g_hp;
  ab.dcoeff_partial = at<float>(a, w.dc_partial);
  ab.ldx = P;
  ab.ld_dx = ld_g;
  ab.B = B;
  ab.N = N;
  ab.P = P;
  ab.K = K;
  ab.dtype = POM_BF16;
  ab.rope = a->rope_c;
  if (a->causal) {
    gb.causal = 1;
    gb.pre = a->pre;
    gb.ld_pre = P;
    gb.carry = a->carry;
    gb.suf_out = at<void>(a, w.suf);
    gb.ld_suf = P;
    gb.group_sums = at<float>(a, w.gsum);
    gb.token_offset = a->token_offset;
    POM_TRY(pom_gate_bwd_gemm(&gb, status, stream));
    POM_TRY(pom_reduce_partials(gb.db_partial, d_bias, nullptr, 1.f, 1, B * m_tiles(T), P, stream));
    POM_TRY(pom_group_scan(gb.group_sums, nullptr, nullptr, at<float>(a, w.scan), B, groups_of(N), P, 1, stream));
    // gradient of token n's features: suf[n] + carry of the groups after its own
    ab.dout = gb.suf_out;
    ab.ld_dout = P;
    ab.partial = gb.group_sums;
    ab.scale = 1.f;
    ab.causal = 3;
    POM_TRY(pom_poly_agg_bwd(&ab, stream));
    POM_TRY(pom_reduce_partials(ab.dcoeff_partial, d_coeff, nullptr, 1.f, 1, pom_poly_agg_bwd_slots(&ab), P * K, stream));
    return input_and_weight_grads(a, G, g_hp, g_z, d_wqc, status, stream);
  }
  POM_TRY(pom_gate_bwd_gemm(&gb, status, stream));
  float* dH = at<float>(a, w.dh);
  float* dH2 = at<float>(a, w.dh2);
  POM_TRY(pom_reduce_partials(gb.dh_partial, dH, nullptr, 1.f, B, m_tiles(T), P, stream));
  POM_TRY(pom_reduce_partials(gb.db_partial, d_bias, nullptr, 1.f, 1, B * m_tiles(T), P, stream));

  const int64_t BP = static_cast<int64_t>(B) * P;
  if (a->dh_state) {  // gradient that reached the returned state: dH += dh_state   (two-term sum per element)
    // (B, 2, P) view is not available for two separate buffers: merge with weights 1 and 1 via the state kernel,
    // h_new = (n*h_past + h_cur) / (n + 1) with n = 1 gives the mean; scale back below through `scale`.
    POM_TRY(pom_state_merge(a->dh_state, dH, dH2, 1.f, BP, stream));  // (dh_state + dH) / 2
    POM_TRY(pom_reduce_partials(dH2, dH, nullptr, 2.f, B, 1, P, stream));
  }
  if (a->frames > 1) {
    POM_TRY(pom_frame_prefix_mean(dH, dH2, B / a->frames, a->frames, P, 1, stream));
    float* t = dH;
    dH = dH2;
    dH2 = t;
  }
  float scale = a->mask ? 1.f : 1.f / N;
  if (a->h_past) {  // H = (n_past * h_past + h_cur) / (n_past + 1)
    if (a->d_hpast)
      POM_TRY(pom_reduce_partials(dH, a->d_hpast, nullptr, a->n_past / (a->n_past + 1.f), B, 1, P, stream));
    scale /= (a->n_past + 1.f);
  }

  ab.row_weight = a->mask;
  ab.denom = a->mask ? a->denom : nullptr;
  ab.dH = dH;
  ab.scale = scale;
  ab.causal = 0;
  POM_TRY(pom_poly_agg_bwd(&ab, stream));
  POM_TRY(pom_reduce_partials(ab.dcoeff_partial, d_coeff, nullptr, 1.f, 1, pom_poly_agg_bwd_slots(&ab), P * K, stream));
  return input_and_weight_grads(a, G, g_hp, g_z, d_wqc, status, stream);
}

}  // extern "C"
