/*
 * pom_b200 — C ABI of the B200 (sm_100a) Polynomial-Mixer kernels.
 *
 * Every entry point
 *   - takes plain device pointers, sizes and strides (in elements) and a CUDA stream
 *     handle (`void*` == cudaStream_t); nothing in a signature depends on PyTorch;
 *   - only enqueues work on that stream: no allocation, no synchronisation, no host
 *     read of device memory, no retained pointer;
 *   - returns 0 on success or a negative POM_ERR_* code (see pom_strerror);
 *   - reports device-side problems (a bounded wait that expired) through the optional
 *     `status` word in device memory, which stays 0 when all is well.
 *
 * The caller owns all memory: inputs, outputs, saved activations, partial-sum
 * workspaces and the status word.
 *
 * Reference interface replaced (paths inside davidpicard/pom):
 *   pom/pom.py:52-100    polynomial_aggregation_      -> pom_poly_agg_fwd / pom_poly_agg_bwd
 *   pom/pom.py:103-122   polynomial_selection_        -> pom_select_fwd / pom_select_bwd
 *   pom/pom.py:193-231   PoM._get_h_s + PoM.forward   -> pom_ctx_gemm + pom_reduce_partials +
 *                                                        pom_gate_gemm + pom_gemm (output projection)
 *   pom/pom.py:233-262   PoM.state_forward            -> the same, with pom_state_merge in between
 *   pom/pom_rope.py:152-235, 443-526 (RoPE variants)  -> the `rope` member of the operator arguments
 *   pom/pom_triton*.py   poly_agg_*_triton            -> pom_poly_agg_fwd / pom_poly_agg_bwd
 */
#ifndef POM_B200_H_
#define POM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define POM_ABI_VERSION 3

enum {
  POM_OK = 0,
  POM_ERR_BAD_SHAPE = -1,
  POM_ERR_BAD_STRIDE = -2,
  POM_ERR_BAD_ALIGN = -3,
  POM_ERR_UNSUPPORTED = -4,
  POM_ERR_K_TOO_LARGE = -5,
  POM_ERR_CUDA = -6,
  POM_ERR_TIMEOUT = -7,
  POM_ERR_NULL = -8,
  POM_ERR_TOO_LARGE = -9
};

enum { POM_BF16 = 0, POM_F32 = 1 };
enum { POM_ROPE_NONE = 0, POM_ROPE_1D = 1, POM_ROPE_2D = 2 };
enum { POM_OUT_BF16 = 0, POM_OUT_F32 = 1, POM_OUT_F32_ACCUM = 2 };

int pom_abi_version(void);
const char* pom_strerror(int code);
/* 0 when the current device is an sm_100 part the kernels can run on. */
int pom_device_check(void);
/* Number of kernels this library has launched since load (all entry points). */
long long pom_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Rotary position description shared by the operators (reference pom/pom_rope.py:93-235).
 * 1-D: cos0/sin0 are (max_len, P/2) tables, pos is (N) int64, pos_stride 1.
 * 2-D: cos0/sin0 are the row tables (max_h, P/4), cos1/sin1 the column tables (max_w, P/4),
 *      pos is (N, 2) int64 (row, col), pos_stride 2.
 * len0 / len1 are the heights of the tables (rows).  The host validates positions against them
 * (pom_rope_pos_info gives min / max); on the device a position outside [0, len) is clamped into the
 * table, so a bad position gives a wrong rotation but never a read outside the tables (len 0 = unknown:
 * no clamp).
 * step0 / step1 describe the positions that section 0 (1-D, or the row half of 2-D) and section 1 (the
 * column half) use, per aligned group of 32 tokens:  0 = the tokens of a group share one position,
 * 1 = they hold consecutive positions (base, base + 1, ...), -1 = anything else.  The stand-alone
 * operators ignore it; the fused tensor-core phases (pom_ctx_gemm, pom_gate_gemm, pom_gate_bwd_gemm)
 * need 0 or 1 (they build every token's angle from its group's base angle and a lane offset) and return
 * POM_ERR_UNSUPPORTED otherwise.  pom_rope_pos_info computes both from the positions.
 * ------------------------------------------------------------------------------------------ */
typedef struct pom_rope {
  int32_t kind; /* POM_ROPE_* */
  int32_t pos_stride;
  const float* cos0;
  const float* sin0;
  const float* cos1;
  const float* sin1;
  const int64_t* pos;
  int32_t len0, len1;
  int32_t step0, step1;
} pom_rope;

/* Scans positions (n, pos_stride) int64 on the device and writes, for column c of the positions (c = 0, 1;
 * only c = 0 when pos_stride == 1), info[4c + 0] = min, info[4c + 1] = max, info[4c + 2] = 1 when every aligned
 * 32-token group is constant, info[4c + 3] = 1 when every aligned 32-token group is consecutive.  info is 8 int64
 * in device memory; the call only enqueues work.  (Host helper of the rotary epilogues: no reference counterpart,
 * the reference indexes its tables with the positions directly, pom/pom_rope.py:171-172.) */
int pom_rope_pos_info(const int64_t* pos, int64_t n, int32_t pos_stride, int64_t* info, void* stream);

/* ------------------------------------------------------------------------------------------
 * Tensor-core GEMM (tcgen05, bf16 inputs, fp32 accumulate):
 *     C[b, m, n] = alpha * sum_k A[b, m, k] * Bm[n, k]
 * A is (batches, M, K) with row stride lda (K-major) or, when a_mn_major, stored as (K, M)
 * with row stride lda (batches must be 1).  Bm is (N, K) row stride ldb, or when b_mn_major
 * stored as (K, N).  C is (batches*M, N) row stride ldc; out_mode selects bf16 store, fp32
 * store, or fp32 accumulate (the only mode in which split_k > 1 is allowed; C must be
 * zeroed or hold the value to accumulate onto).  split_k == 0 picks a split automatically
 * in accumulate mode.  All leading dimensions and base addresses must be multiples of
 * 8 elements / 16 bytes.
 * Strided batches: with b_batched the B operand has one matrix per batch as well (C[b] = A[b]·Bm[b]ᵀ); the
 * *_batch_stride fields give the element offset between consecutive batches of each tensor (0 = the matrices
 * follow one another; multiples of 8), so heads / frames / samples that sit side by side inside a wider matrix
 * run as one launch.  A transposed A may now have batches too.
 * Replaces: the cuBLAS calls behind nn.Linear in pom/pom.py:187,191,205,231 and their autograd.
 * ------------------------------------------------------------------------------------------ */
typedef struct pom_gemm_args {
  const void* A;
  const void* Bm;
  void* C;
  int64_t M, N, K;
  int64_t lda, ldb, ldc;
  int32_t batches;
  int32_t a_mn_major, b_mn_major;
  int32_t out_mode;
  int32_t split_k;
  float alpha;
  /* bf16 output only (the feed-forward block of the README's layer stack, README.md:28-35): */
  int32_t act;          /* 0 none, 1 exact GELU applied to alpha * sum */
  const void* residual; /* bf16 (batches*M, N) row stride ldr, added after the activation; NULL = none */
  int64_t ldr;
  int64_t a_batch_stride, b_batch_stride, c_batch_stride; /* elements; 0 = densely packed batches */
  int32_t b_batched;    /* 0: one B matrix for all batches; 1: one per batch */
} pom_gemm_args;
int pom_gemm_bf16(const pom_gemm_args* a, int* status, void* stream);

/* Diagnostic override for every tcgen05 GEMM entry point (tests and micro-benchmarks use it to reach each kernel
 * variant; production code leaves it at 0 = choose per problem).  Units digit: 1 = always the kernel that gives one
 * CTA a 128 x BN tile, 2 = always the kernel in which a cluster of two CTAs shares a 256 x BN tile (tcgen05
 * cta_group::2; each CTA loads half of the B tile).  Tens digit: 1 / 2 / 3 = 128 / 192 / 256 columns per tile where
 * the operands allow that width.  Hundreds digit 1 = the paired epilogues never get the column-stationary grid (every
 * CTA then changes its column block from tile to tile).  Process-wide, not thread-safe against concurrent launches. */
int pom_set_gemm_mode(int mode);

/* fp32 SIMT GEMM with the same meaning (fp32 A, Bm, C; out_mode F32 or F32_ACCUM); used by the
 * fp32 precision mode, where tensor-core inputs would not meet the 1e-4 bound. */
int pom_gemm_f32(const pom_gemm_args* a, void* stream);

/* ------------------------------------------------------------------------------------------
 * Context phase, fused (bf16): hp = X·Wpoᵀ on tensor cores; the epilogue rounds hp to bf16,
 * optionally saves it, applies act + polynomial (+ per-token weight) and reduces over each
 * 128-token tile.  partial is (B * ceil(N/128), P) fp32; reduce it with pom_reduce_partials.
 * With rope.kind != POM_ROPE_NONE the polynomial features of every token are rotated by its position before
 * the reduction (reference pom/pom_rope.py:513-515, pom_triton_rope.py:93-217): needs K <= 4, P % 16 == 0
 * (1-D) or P % 64 == 0 (2-D) and rope.step0/1 in {0, 1}; otherwise POM_ERR_UNSUPPORTED (use pom_poly_agg_fwd).
 * Replaces: pom/pom.py:205-206 + pom/pom.py:83-91 / 35-38 (and pom_triton.py:68-153).
 * ------------------------------------------------------------------------------------------ */
typedef struct pom_ctx_args {
  const void* X;       /* (B, N, D) bf16, row stride ldx */
  const void* Wpo;     /* (P, D) bf16, row stride ldw */
  const float* coeff;  /* (P, K) fp32 */
  const float* row_weight; /* (B, N) fp32 or NULL */
  void* hp_out;        /* (B*N, ld_hp) bf16 or NULL */
  float* partial;      /* (B * ceil(N/128), P) fp32 */
  int64_t ldx, ldw, ld_hp;
  int32_t B, N, D, P, K;
  const float* tile_weight; /* optional with row_weight: (B * ceil(N/128)) fp32 from pom_tile_weights; a 128-token
                               tile whose weights sum to 0 is skipped: no loads, no MMAs, partial = 0 and its rows of
                               hp_out are NOT written (pom_poly_agg_bwd never uses rows of weight 0) */
  pom_rope rope;       /* positions of the N context tokens (shared by all samples) */
  /* Token-causal form (causal != 0; reference pom/pom.py:92-95, pom_triton_causal.py:68-160): instead of per-tile
   * sums the epilogue writes, per aligned group of 32 tokens, the inclusive running sums of the (rotated)
   * polynomial features as bf16 `pre_out` (B*N, ld_pre) and the group totals `group_sums` (B, ceil(N/32), P) fp32;
   * `partial` and `row_weight` are not used.  pom_group_scan then turns the totals into carries for
   * pom_gate_gemm.  Works with and without rotary embedding (K <= 4, P % 16 == 0; 2-D rotary P % 64 == 0). */
  int32_t causal;
  void* pre_out;
  int64_t ld_pre;
  float* group_sums;
} pom_ctx_args;
int pom_ctx_gemm(const pom_ctx_args* a, int* status, void* stream);
/* out[b * ceil(N/128) + t] = sum of w[b, 128 t .. 128 t + 127] (w (B, N) fp32, key-padding weights >= 0). */
int pom_tile_weights(const float* w, float* out, int32_t B, int32_t N, void* stream);

/* out[b, p] = scale * sum_c partial[b, c, p] / denom[b]   (denom may be NULL = 1; a zero denominator
 * yields 0, the convention of pom/pom_triton_masked.py:166-167 for a sample with no valid token) */
int pom_reduce_partials(const float* partial, float* out, const float* denom, float scale, int32_t B,
                        int32_t chunks, int32_t P, void* stream);

/* ------------------------------------------------------------------------------------------
 * Query phase, fused (bf16): z = X·Wseᵀ; epilogue saves bf16 z (optional) and writes
 * SH = hardsigmoid(z + bias) ⊙ H as bf16.  H is fp32 with h_batch_stride / h_row_stride
 * (row stride 0: one vector per sample).  With rope.kind != POM_ROPE_NONE the gate is rotated by the query
 * token's position after the hardsigmoid (reference pom/pom_rope.py:522); same conditions as pom_ctx_gemm.
 * Replaces: pom/pom.py:207 + pom/pom.py:116-118.
 * ------------------------------------------------------------------------------------------ */
typedef struct pom_gate_args {
  const void* X;      /* (B, T, D) bf16 */
  const void* Wse;    /* (P, D) bf16 */
  const float* bias;  /* (P) fp32 */
  const float* H;     /* fp32 */
  void* z_out;        /* (B*T, ld_z) bf16 or NULL */
  void* sh_out;       /* (B*T, ld_sh) bf16 */
  int64_t ldx, ldw, ld_z, ld_sh;
  int64_t h_batch_stride, h_row_stride;
  int32_t B, T, D, P;
  pom_rope rope;      /* positions of the T query tokens */
  /* Token-causal form (causal != 0): H is not used; the epilogue re-reads `pre` (B*T, ld_pre) bf16 written by
   * the causal pom_ctx_gemm, adds the group carries `carry` (B, ceil(T/32), P) fp32 from pom_group_scan and
   * divides by (token_offset + t + 1): the prefix mean of pom/pom.py:92-95 for query token t. */
  int32_t causal;
  const void* pre;
  int64_t ld_pre;
  const float* carry;
  int64_t token_offset;
} pom_gate_args;
int pom_gate_gemm(const pom_gate_args* a, int* status, void* stream);

/* Backward of the query phase (bf16): dSH = dY·Wo on tensor cores; the epilogue re-reads z and
 * emits dz (bf16, written at g_out with row stride ld_g), and per-tile column sums of
 * dSH ⊙ s (-> dh_partial) and of dz (-> db_partial), both (B * ceil(T/128), P) fp32.
 * With rope.kind != POM_ROPE_NONE (rotated gate): dH sums dSH ⊙ R·s and dz is the transposed rotation of
 * dSH ⊙ H times hardsigmoid'; this form reads the output weight transposed, WoT (P, D) row stride ldwt (make it
 * with pom_transpose_bf16), so that the channel pairs of a tile are two row boxes of one K-major operand.
 * Replaces: autograd of pom/pom.py:207, 116-118, 231 (input-gradient half) and of pom/pom_rope.py:522. */
typedef struct pom_gate_bwd_args {
  const void* dY;     /* (B, T, D) bf16 */
  const void* Wo;     /* (D, P) bf16, row stride ldw */
  const float* bias;
  const float* H;     /* (B, P) fp32, h_batch_stride */
  const void* z;      /* (B*T, ld_z) bf16 */
  void* g_out;        /* (B*T, ld_g) bf16 */
  float* dh_partial;
  float* db_partial;
  int64_t ld_dy, ldw, ld_z, ld_g, h_batch_stride;
  int32_t B, T, D, P;
  const void* WoT;    /* rotary and causal forms: (P, D) bf16, row stride ldwt */
  int64_t ldwt;
  pom_rope rope;      /* positions of the T query tokens */
  /* Token-causal form (causal != 0; needs WoT): `pre` / `carry` as in pom_gate_args rebuild the prefix means for
   * dz; the gradient of the prefix means, dSH ⊙ R·s / (token_offset + t + 1), is summed UP the rows of every
   * 32-token group and written as bf16 `suf_out` (B*T, ld_suf) plus group totals `group_sums`
   * (B, ceil(T/32), P) fp32 (reverse pom_group_scan, then pom_poly_agg_bwd with causal == 3).  dh_partial and H are
   * not used.  Backward halves of pom_triton_causal.py:176-344 / pom_triton_rope.py:618-873. */
  int32_t causal;
  const void* pre;
  int64_t ld_pre;
  const float* carry;
  void* suf_out;
  int64_t ld_suf;
  float* group_sums;
  int64_t token_offset;
} pom_gate_bwd_args;

/* In-place exclusive scan over the 32-token groups of (B, groups, P) fp32 group totals:
 *   reverse == 0:  sums[b, g, :] <- carry_in[b, :] + sum_{g' < g} sums[b, g', :]
 *   reverse != 0:  sums[b, g, :] <- carry_in[b, :] + sum_{g' > g} sums[b, g', :]
 * carry_in (B, P) may be NULL (token sharding: the totals of the ranks before / after this one); total_out (B, P),
 * optional, receives the sum over this call's groups (without carry_in).  scratch: B * ceil(groups / 32) * P floats.
 * Replaces the serial token loops of pom_triton_causal.py:107-160 / 233-325 at group granularity. */
int pom_group_scan(float* sums, const float* carry_in, float* total_out, float* scratch, int32_t B, int32_t groups,
                   int32_t P, int32_t reverse, void* stream);
int pom_gate_bwd_gemm(const pom_gate_bwd_args* a, int* status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Stand-alone aggregation operator (any dtype, optional rotary embedding):
 *   poly[b,n,:] = R_n · polynomial(act(x[b,n,:]))
 *   causal == 0 : out[b, :]    = sum_n w[b,n] * poly[b,n,:]             -> `partial` then reduce
 *   causal == 1 : out[b, n, :] = (carry[b,:] + sum_{m<=n} poly[b,m,:]) / (n + 1 + token_offset)
 *   causal == 2 : out[b, n, :] = poly[b,n,:]     (per-token features, no reduction; `partial` unused; the
 *                 input of the (B, M, N)-mask product, reference pom/pom.py:41-45, 98-99)
 * Non-causal: the kernel writes per-chunk sums into partial (B, chunks, P); call
 * pom_reduce_partials.  Causal: `partial` (B, chunks, P) is scratch; out is (B, N, P) of dtype.
 * chunks = pom_agg_chunks(N).
 * Replaces: pom/pom.py:83-100 and the kernels of pom/pom_triton.py, pom_triton_causal.py,
 * pom_triton_masked.py, pom_triton_rope.py (forward halves).
 * ------------------------------------------------------------------------------------------ */
int32_t pom_agg_chunks(int32_t N);

typedef struct pom_agg_args {
  const void* x;        /* (B, N, P) dtype, row stride ldx */
  const float* coeff;   /* (P, K) fp32 */
  const float* row_weight; /* (B, N) fp32 or NULL; non-causal only */
  const float* carry;   /* (B, P) fp32 or NULL; causal only: sum over tokens of earlier shards */
  float* partial;       /* (B, chunks, P) fp32 */
  void* out;            /* causal only: (B, N, P) dtype, row stride ld_out */
  float* total;         /* causal only, optional: (B, P) fp32 sum over this call's tokens */
  int64_t ldx, ld_out;
  int64_t token_offset; /* global index of token 0 (causal) */
  int32_t B, N, P, K;
  int32_t dtype, causal;
  pom_rope rope;
} pom_agg_args;
int pom_poly_agg_fwd(const pom_agg_args* a, void* stream);

/* Mean / weighted-mean aggregation for callers that must not allocate.  (No counterpart in the
 * reference: it exists for hosts of this library, not to mirror one of its functions.)
 *
 * Some programs that embed these kernels hand out every byte of device memory when they start and
 * then forbid cudaMalloc for good: serving processes with a fixed memory plan, plug-in hosts whose
 * worker threads may not enter the allocator because an allocation can stall the whole device or
 * fail long after start-up.  Such a caller has no place to get the (B, chunks, P) partial-sum buffer
 * that pom_poly_agg_fwd needs.  This entry point computes
 *     out[b, :] = scale * sum_n w[b,n] * R_n·polynomial(act(x[b,n,:])) / denom[b]
 * (non-causal pom_poly_agg_fwd followed by pom_reduce_partials, bit for bit) with the partial sums
 * held in a workspace that is part of the library image: 4 Mi floats (16 MiB) per GPU, resident from
 * the moment the library is loaded on that GPU until the process ends.  a->partial, a->out, a->total,
 * a->carry and a->causal (must be 0) are not used; `denom` may be NULL (= 1); `out` is (B, P) fp32.
 *
 * Limits and rules:
 *   - B * pom_agg_chunks(N) * P must not exceed 4 194 304, else POM_ERR_TOO_LARGE and nothing runs.
 *   - No cudaMalloc / cudaFree or allocating library call is made, on any call.  The first call on
 *     each device looks up the workspace address (a host-side runtime query, no device work); make
 *     that first call before starting any stream capture.
 *   - All calls on one GPU share the one workspace.  Calls whose kernels could overlap on the GPU
 *     (different streams without ordering between them) race on it; keep them on one stream or
 *     order them yourself.  Nothing needs clearing between calls: each call overwrites every slot
 *     it later reads. */
int pom_poly_agg_mean_noalloc(const pom_agg_args* a, const float* denom, float scale, float* out, void* stream);

/* Backward of the aggregation operator.
 *   causal == 0 : dH (B, P) fp32 is the gradient of out; token weight = row_weight[b,n] / denom[b]
 *                 (either may be NULL = 1); `scale` multiplies everything (1/N for a plain mean).
 *   causal == 1 : dout (B, N, P) dtype; `carry` (B, P) fp32 optional = suffix sum from later shards;
 *                 `total` optional output (B, P): this shard's sum of dout[n]/(n+1+offset).
 *   causal == 2 : dout (B, N, P) dtype is the gradient of each token's own features (no suffix sum).
 *   causal == 3 : fused token-causal path (bf16, K <= 4): the gradient of token n's features is
 *                 suf[b, n, :] + carry_b[b, n / 32, :] with `suf` = dout (bf16 running sums written by the causal
 *                 pom_gate_bwd_gemm) and carry_b = `partial` after the reverse pom_group_scan.
 *                 phase == 1 stops after the totals (used to obtain `total` before the cross-shard
 *                 exchange that produces `carry`); phase == 0 runs everything.
 * Outputs: dx (B, N, P) dtype row stride ld_dx; dcoeff_partial (B*chunks, P, K) fp32, to be
 * reduced with pom_reduce_partials(B=1, chunks=B*chunks, P=P*K).
 * Replaces: backward halves of the kernels named above. */
typedef struct pom_agg_bwd_args {
  const void* x;
  const float* coeff;
  const float* row_weight;
  const float* denom;
  const float* dH;      /* non-causal */
  const void* dout;     /* causal */
  const float* carry;
  float* partial;       /* causal scratch (B, chunks, P) */
  float* total;
  void* dx;
  float* dcoeff_partial;
  int64_t ldx, ld_dx, ld_dout;
  int64_t token_offset;
  float scale;
  int32_t B, N, P, K;
  int32_t dtype, causal, phase;
  pom_rope rope;
} pom_agg_bwd_args;
int pom_poly_agg_bwd(const pom_agg_bwd_args* a, void* stream);
/* Number of (P, K) slots of dcoeff_partial that pom_poly_agg_bwd writes for these arguments (the caller sums
 * exactly that many); never more than B * pom_agg_chunks(N), which is the capacity to allocate. */
int32_t pom_poly_agg_bwd_slots(const pom_agg_bwd_args* a);
/* Synchronous read of this device's operator status word: 0, or the code of the first bounded wait inside an
 * operator kernel (a shared-memory staging barrier) that expired; results of that launch are then incomplete. */
int pom_ops_status(int32_t* value_out);

/* ------------------------------------------------------------------------------------------
 * Selection operator: SH[b,t,:] = R_t·hardsigmoid(z[b,t,:] + bias) ⊙ H[b, t or 0, :]
 * H is fp32 (B, P) when h_per_token == 0, else (B, T, P) of dtype with row stride ld_h.
 * Replaces: pom/pom.py:207 (+ se_bias), pom/pom_rope.py:522, pom/pom.py:116-118.
 * ------------------------------------------------------------------------------------------ */
typedef struct pom_select_args {
  const void* z;       /* (B, T, P) dtype, row stride ld_z */
  const float* bias;   /* (P) fp32 */
  const void* H;
  void* sh;            /* (B, T, P) dtype, row stride ld_sh */
  int64_t ld_z, ld_h, ld_sh;
  int32_t B, T, P;
  int32_t dtype, h_per_token;
  int32_t activated;   /* nonzero: z already holds the gate s (bias and hardsigmoid are skipped) */
  const float* row_denom; /* optional, per-token H only: H[b,t,:] is divided by row_denom[b*T+t] (a zero divisor
                             makes the row 0); the row sums of a (B, M, N) mask (reference pom/pom.py:41-45) */
  pom_rope rope;
} pom_select_args;
int pom_select_fwd(const pom_select_args* a, void* stream);

/* Backward: given dSH, emits dz (dtype, row stride ld_dz), dbias partial sums
 * (B*chunks, P) and either dH partial sums (B, chunks, P) fp32 (h_per_token == 0) or the
 * per-token dH (B, T, P) dtype row stride ld_dh. */
typedef struct pom_select_bwd_args {
  const void* dsh;
  const void* z;
  const float* bias;
  const void* H;
  void* dz;
  float* dbias_partial;
  float* dh_partial;
  void* dh_tok;
  int64_t ld_dsh, ld_z, ld_h, ld_dz, ld_dh;
  int32_t B, T, P;
  int32_t dtype, h_per_token;
  int32_t activated;   /* as in pom_select_args; dz is then the gradient of s itself */
  const float* row_denom; /* as in pom_select_args; dh_tok is then the gradient of the un-divided H */
  pom_rope rope;
} pom_select_bwd_args;
int pom_select_bwd(const pom_select_bwd_args* a, void* stream);

/* Multi-head scalar gating (reference pom/pom.py:119-122): one gate value per (token, head) multiplies the
 * P / heads channels of that head.  `s` is the activated (and, with rotary embedding, rotated) gate, fp32
 * (B, T, heads).  Forward: sh[b,t,p] = s[b,t,p / head_dim] * H[b, t or 0, p].  Backward: gradient of H (per-chunk
 * partial sums (B, chunks, P) fp32, or per token in dtype) and gradient of s, accumulated into `ds` (B, T, heads)
 * fp32, which the caller zeroes first.  H as in pom_select_args. */
typedef struct pom_select_heads_args {
  const float* s;
  const void* H;
  const void* dsh;     /* backward only */
  void* sh;            /* forward only */
  float* ds;           /* backward only */
  float* dh_partial;   /* backward, h_per_token == 0 */
  void* dh_tok;        /* backward, h_per_token != 0 */
  int64_t ld_h, ld_sh, ld_dsh, ld_dh;
  int32_t B, T, P, heads;
  int32_t dtype, h_per_token;
} pom_select_heads_args;
int pom_select_heads_fwd(const pom_select_heads_args* a, void* stream);
int pom_select_heads_bwd(const pom_select_heads_args* a, void* stream);

/* Multi-head gating (n_sel_heads > 1, reference pom/pom.py:119-122) with a per-sample aggregate H: the gate has
 * one value per head, so  y[b,t,:] = sum_h s[b,t,h] * Mb[b,h,:]  with  Mb[b,h,d] = sum_{p in head h} H[b,p] Wo[d,p].
 * These four calls replace pom_select_heads_* plus the output projection and its two backward GEMMs
 * (pom/pom.py:231 and autograd) by products whose inner dimension is the head count:
 *   pom_heads_mix      Mb from H and Wo
 *   pom_heads_out_fwd  y = s·Mb (+ residual)
 *   pom_heads_out_bwd  ds[b,t,h] = sum_d dy·Mb ;  dMb[b,h,d] = sum_t s·dy   (dMb_partial: scratch)
 *   pom_heads_mix_bwd  dH[b,p] = sum_d dMb[b,head(p),d] Wo[d,p] ;  dWo[d,p] += sum_b dMb[b,head(p),d] H[b,p]
 * dtype (POM_BF16 / POM_F32) is that of Wo, y, residual and dy; everything else is fp32.  heads <= 64, P % heads == 0,
 * D % 4 == 0 and heads * D fp32 must fit in shared memory (pom_heads_supported). */
typedef struct pom_heads_args {
  const float* H;        /* (B, P) */
  const void* Wo;        /* (D, P), row stride ldw */
  const float* s;        /* (B, T, heads) gate values */
  float* Mb;             /* (B, heads, D) */
  void* y;               /* (B, T, D) */
  const void* residual;  /* (B, T, D) or NULL */
  const void* dy;        /* (B, T, D) */
  float* ds;             /* (B, T, heads) */
  float* dMb_partial;    /* (B, ceil(T/128), heads, D) scratch */
  float* dMb;            /* (B, heads, D) */
  float* dH;             /* (B, P) */
  float* dWo;            /* (D, P) contiguous, accumulated into */
  int64_t ldw;
  int32_t B, T, D, P, heads, dtype;
} pom_heads_args;
int pom_heads_supported(int32_t heads, int32_t D, int32_t P);
int pom_heads_mix(const pom_heads_args* a, void* stream);
int pom_heads_out_fwd(const pom_heads_args* a, void* stream);
int pom_heads_out_bwd(const pom_heads_args* a, void* stream);
int pom_heads_mix_bwd(const pom_heads_args* a, void* stream);

/* Running-mean state update of state_forward (reference pom/pom.py:255-259):
 *   h_new[b,:] = (n_past * h_past[b,:] + h_cur[b,:]) / (n_past + 1)        (fp32, B*P elements) */
int pom_state_merge(const float* h_past, const float* h_cur, float* h_new, float n_past, int64_t count, void* stream);

/* Block-causal aggregate over equal frames: the single-pass form of calling state_forward once per frame
 * (reference pom/pom.py:251-259, where every call weighs equally) and of a block-lower-triangular (B, N, N) mask
 * (pom/pom.py:41-45, 98-99).  in/out (B, F, P) fp32, in = per-frame means.
 *   adjoint == 0:  out[b,f,:] = (1/(f+1)) * sum_{g<=f} in[b,g,:]
 *   adjoint != 0:  out[b,g,:] = sum_{f>=g} in[b,f,:] / (f+1)          (gradient of the above)
 * in and out may be the same buffer. */
int pom_frame_prefix_mean(const float* in, float* out, int32_t B, int32_t F, int32_t P, int32_t adjoint, void* stream);

/* Asynchronous zero fill of `bytes` bytes (cudaMemsetAsync on the stream); used for split-K accumulators. */
int pom_fill_zero(void* dst, int64_t bytes, void* stream);

/* dst (cols, rows) bf16 row stride ld_dst  <-  transpose of src (rows, cols) bf16 row stride ld_src. */
int pom_transpose_bf16(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst,
                       void* stream);

/* Element conversion helpers (count elements): fp32 -> bf16, bf16 -> fp32. */
int pom_cast_f32_to_bf16(const float* src, void* dst, int64_t count, void* stream);
int pom_cast_bf16_to_f32(const void* src, float* dst, int64_t count, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Whole layer in two calls (bf16, one GPU, no rotary embedding, mask none or (B, N)): everything
 * PoM.forward / PoM.state_forward (reference pom/pom.py:216-262) and their autograd do, sequenced on `stream`
 * from the phase entry points above.  All tensors contiguous; the caller owns every buffer.
 *
 *   forward : [denom = sum_n mask] -> pom_ctx_gemm -> H = mean (or masked mean) [-> running mean over frames]
 *             [-> merge with h_past] -> pom_gate_gemm -> y = SH·Woᵀ (+ residual)
 *   backward: grads := 0; dWo; pom_gate_bwd_gemm; dH, dbias [+ dh_state] [-> adjoint of the frame mean]
 *             [-> d_hpast]; streamed aggregation backward; dX and dWqc (one GEMM each under self-mixing)
 *
 * `frames` > 1 folds a block-causal sequence: batch rows are (sample, frame) pairs, B % frames == 0 (see
 * pom_frame_prefix_mean).  h_past / n_past: the running-mean state of state_forward.  Hosts that need an exchange
 * between the phases (token sharding) call the phase entry points themselves. */
typedef struct pom_layer_args {
  int32_t B, T, N, D, P, K;   /* T query tokens, N context tokens per batch row; P = expand * D; K = degree */
  int32_t self_mixing;        /* context == queries (T == N, xc ignored) */
  int32_t frames;             /* >= 1 */
  int32_t save;               /* forward: keep hp and z for backward */
  float n_past;               /* weight of h_past (calls so far) */
  const void* xq;             /* (B, T, D) bf16 */
  const void* xc;             /* (B, N, D) bf16 or NULL */
  const void* w_qc;           /* (2P, D) bf16: rows [0, P) polynomial projection, [P, 2P) gate projection */
  const void* w_ag;           /* (D, P) bf16 */
  const float* se_bias;       /* (P) */
  const float* coeff;         /* (P, K) */
  const float* mask;          /* (B, N) fp32 weights or NULL */
  const float* h_past;        /* (B, P) fp32 or NULL */
  const void* residual;       /* (B, T, D) bf16 or NULL: added to y */
  void* y;                    /* (B, T, D) bf16, forward output */
  void* hp;                   /* (B, N, P) bf16, saved projection (forward out when save, backward in) */
  void* z;                    /* (B, T, P) bf16, saved gate pre-activation */
  void* sh;                   /* (B, T, P) bf16, gated state (operand of the output projection) */
  float* H;                   /* (B, P) fp32 aggregate (forward out, backward in) */
  float* denom;               /* (B) fp32 mask sums (forward out, backward in); required with mask */
  const void* dy;             /* backward: (B, T, D) bf16 */
  const float* dh_state;      /* backward: (B, P) fp32 gradient of the returned state, or NULL */
  void* G;                    /* backward scratch, bf16: (B*T, 2P) under self-mixing, else (B*N + B*T) * P */
  void* dxq;                  /* (B, T, D) bf16 */
  void* dxc;                  /* (B, N, D) bf16 (cross-mixing only) */
  float* grads;               /* fp32, zeroed by the call: [dWqc (2P*D) | dWo (D*P) | dbias (P) | dcoeff (P*K)] */
  float* d_hpast;             /* (B, P) fp32 or NULL */
  void* workspace;            /* pom_layer_workspace_bytes() bytes, 256-byte aligned, shared by both calls */
  uint64_t workspace_bytes;
  /* Rotary embedding (pom/pom_rope.py:487-522) and the token-causal mask (pom/pom.py:92-95) inside the same two
   * calls, under the conditions of pom_ctx_gemm / pom_gate_gemm (degree <= 4, P % 16 == 0, 2-D: P % 64 == 0,
   * positions constant or consecutive inside aligned 32-token groups); otherwise POM_ERR_UNSUPPORTED. */
  pom_rope rope_c;            /* positions of the N context tokens (kind POM_ROPE_NONE: no rotation) */
  pom_rope rope_q;            /* positions of the T query tokens */
  const void* w_ag_t;         /* backward with rope_q or causal: (P, D) bf16, the output weight transposed
                                 (pom_transpose_bf16) */
  int32_t causal;             /* 1: token-causal prefix mean; needs T == N, no mask, frames == 1, no state */
  int32_t reserved0;
  int64_t token_offset;       /* causal: global index of token 0 */
  void* pre;                  /* causal: (B, N, P) bf16 running sums per 32-token group (forward out, backward in) */
  float* carry;               /* causal: (B, ceil(N/32), P) fp32 group carries (forward out, backward in); H is
                                 not used */
} pom_layer_args;
uint64_t pom_layer_workspace_bytes(const pom_layer_args* a);
int pom_layer_fwd(const pom_layer_args* a, int* status, void* stream);
int pom_layer_bwd(const pom_layer_args* a, int* status, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Token-sharding exchanges over NVLink peer memory (no counterpart in the reference, which is single-GPU;
 * they carry the cross-rank sums that a token-sharded PoM.forward needs: the (B, P) aggregate of
 * pom/pom.py:90-96 split over ranks, its gradient, the causal prefix/suffix carries, and the sum of
 * the parameter gradients).
 *
 * Every rank owns one exchange buffer of pom_peer_layout()[2] bytes, zero-filled before first use, which all
 * ranks of the node map: the owner exports it (pom_peer_export: CUDA IPC handle of the enclosing allocation +
 * byte offset of the buffer inside it), the handle travels by any host channel, the others open it
 * (pom_peer_open, returns the allocation's base in this process; add the offset).  Layout:
 *   [0, POM_PEER_HEADER_BYTES)  epoch counters and flags
 *   [layout[0], layout[1])      message slots: 2 epochs x world writers x slot_floats fp32
 *   [layout[1], layout[2])      parameter-gradient region: flat_floats fp32 accumulators (reduced in place by
 *                               pom_peer_allreduce_flat), then at layout[1] + 4 * flat_floats a bf16 staging image and
 *                               at layout[1] + 6 * flat_floats the bf16 result image of pom_peer_allreduce_flat_bf16
 * The library allocates nothing; the caller owns the buffers and must keep them alive, and mapped by the
 * peers, until all ranks have finished their last exchange.  All ranks must issue the same sequence of
 * exchange calls.  Waits on other ranks are bounded (pom_peer_comm::wait_ns, 2 s when 0): on expiry
 * POM_ERR_TIMEOUT is stored in *status (device int, zero before the first call; once non-zero, later exchanges do
 * not wait) and the results are undefined.  Recovery: the epoch counters of the rank that gave up have moved on,
 * so the group must drop its buffers, zero-fill new ones, exchange handles again and clear the status word before
 * the next exchange; a comm is not usable again after a timeout.  The calls only enqueue work on `stream` and can be captured into CUDA graphs (the epochs
 * are device-side counters).  Kernels of different ranks wait on each other, so every rank must run on its
 * own GPU. */
#define POM_PEER_MAX_RANKS 16
#define POM_PEER_FLAT_CTAS 128
#define POM_PEER_HEADER_BYTES 65536
#define POM_PEER_HANDLE_BYTES 64

typedef struct pom_peer_comm {
  void* base[POM_PEER_MAX_RANKS];   /* base[r]: rank r's exchange buffer as addressable from this process */
  int32_t rank, world;
  unsigned long long slot_floats;   /* capacity of one message (multiple of 4) */
  unsigned long long flat_floats;   /* capacity of the gradient region (multiple of 4, may be 0) */
  unsigned long long wait_ns;       /* limit of every wait on another rank, in nanoseconds; 0 = 2 s */
} pom_peer_comm;

/* out[0] = byte offset of the slots, out[1] = of the gradient region, out[2] = total bytes. */
int pom_peer_layout(int world, unsigned long long slot_floats, unsigned long long flat_floats,
                    unsigned long long out[3]);
int pom_peer_export(const void* dev_ptr, void* handle_out /* POM_PEER_HANDLE_BYTES */, unsigned long long* offset_out);
int pom_peer_open(const void* handle, void** base_out);
int pom_peer_close(void* base);

enum { POM_PEER_SUM_ALL = 0, POM_PEER_SUM_BEFORE = 1, POM_PEER_SUM_AFTER = 2 };

/* out[b, p] = scale * sum_{r in range} sum_c partial_r[b, c, p] / denom[b]   (denom optional; 0 -> 0)
 * range = all ranks, the ranks before this one, or the ranks after it (rank order, so every rank of an
 * all-reduce gets bitwise the same result).  B * P <= slot_floats.  out may alias partial when chunks == 1. */
typedef struct pom_peer_xchg_args {
  const float* partial;
  float* out;
  const float* denom;
  float scale;
  int32_t B, chunks, P;
  int32_t mode;
} pom_peer_xchg_args;
int pom_peer_exchange(const pom_peer_comm* c, const pom_peer_xchg_args* a, int* status, void* stream);

/* In-place sum over ranks of the first n_floats (multiple of 4) of every rank's gradient region: rank r adds
 * slice r of all ranks in rank order and stores the result to all ranks. */
int pom_peer_allreduce_flat(const pom_peer_comm* c, unsigned long long n_floats, int* status, void* stream);

/* The same sum with bf16 on the wire, for gradients that end up in bf16 anyway: every rank rounds its fp32
 * accumulators to bf16 (staging image, local), rank r adds slice r of all ranks in fp32 in rank order and stores the
 * bf16 result into every rank's result image (byte offset layout[1] + 6 * flat_floats of its buffer).  n_floats and
 * flat_floats multiples of 8.  The fp32 accumulators are left as they were. */
int pom_peer_allreduce_flat_bf16(const pom_peer_comm* c, unsigned long long n_floats, int* status, void* stream);

/* Asynchronous device-to-device copy of `bytes` bytes on the stream (cudaMemcpyAsync; no kernel). */
int pom_copy_bytes(void* dst, const void* src, int64_t bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* POM_B200_H_ */
