"""Thin tensor-level wrappers over the C ABI (no autograd here).

Each function validates devices/dtypes, allocates outputs with PyTorch's caching
allocator, and enqueues the kernel(s) on the current CUDA stream.  Nothing in this
module computes on the CPU or with PyTorch operators.
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _abi
from ._abi import (AggArgs, AggBwdArgs, CtxArgs, GateArgs, GateBwdArgs, GemmArgs, Rope, SelectArgs, SelectBwdArgs,
                   SelectHeadsArgs, ptr)


def _require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("pom_b200 runs on CUDA tensors only (no CPU fallback)")
        dev = dev or t.device
        if t.device != dev:
            raise RuntimeError("all tensors of one call must live on the same GPU")
    return dev


def _ld(t: torch.Tensor, dim: int) -> int:
    """Stride of ``dim``.  A dimension of size 1 may report any stride: it is kept when it is a usable leading
    dimension (at least a row long, a multiple of 8 elements), else replaced by the row length rounded up to 8."""
    s = t.stride(dim)
    if t.shape[dim] > 1:
        return s
    w = t.shape[-1]
    return s if (s >= w and s % 8 == 0) else (w + 7) // 8 * 8


def _row_stride(t: torch.Tensor) -> int:
    """Leading dimension of a 2-D or 3-D tensor whose last dim is contiguous and whose
    leading dims collapse to one row index.  PyTorch leaves the stride of a dimension of size 1 arbitrary (a slice
    of a (B, 1, W) tensor may report any value there), so such a dimension never decides the answer."""
    if t.stride(-1) != 1:
        raise ValueError("last dimension must be contiguous")
    if t.dim() == 2:
        return t.stride(0) if t.shape[0] > 1 else t.shape[1]
    if t.dim() == 3:
        B, N = t.shape[0], t.shape[1]
        if N == 1:
            return t.stride(0) if B > 1 else t.shape[2]
        if B > 1 and t.stride(0) != t.stride(1) * N:
            raise ValueError("batch and token dimensions must collapse to one row stride")
        return t.stride(1)
    raise ValueError("expected a 2-D or 3-D tensor")


@dataclass
class RopeSpec:
    """Rotary tables and positions for one side (context or query) of the layer."""
    kind: int
    cos0: torch.Tensor
    sin0: torch.Tensor
    pos: torch.Tensor  # int64, (N,) or (N, 2), contiguous
    cos1: Optional[torch.Tensor] = None
    sin1: Optional[torch.Tensor] = None
    # per position column, how the positions of every aligned group of 32 tokens look: 0 = one shared position,
    # 1 = consecutive positions, -1 = anything else / unknown (see rope_pos_info); the fused tensor-core phases
    # need 0 or 1, the stand-alone operators take any positions
    steps: Tuple[int, int] = (-1, -1)

    def to_c(self) -> Rope:
        r = Rope()
        r.kind = self.kind
        r.pos_stride = 2 if self.kind == _abi.ROPE_2D else 1
        r.cos0, r.sin0 = ptr(self.cos0), ptr(self.sin0)
        r.cos1, r.sin1 = ptr(self.cos1), ptr(self.sin1)
        r.pos = ptr(self.pos)
        r.len0 = self.cos0.shape[0]
        r.len1 = self.cos1.shape[0] if self.cos1 is not None else 0
        r.step0, r.step1 = self.steps
        return r

    def fusable(self, p: int) -> bool:
        """Whether the rotary GEMM epilogues can take this description for p channels."""
        if self.kind == _abi.ROPE_1D:
            return p % 16 == 0 and self.cos0.shape[1] == p // 2 and self.steps[0] in (0, 1)
        return (p % 64 == 0 and self.cos0.shape[1] == p // 4 and self.cos1.shape[1] == p // 4
                and self.steps[0] in (0, 1) and self.steps[1] in (0, 1))


_pos_info_cache = {}


def rope_pos_info(pos: torch.Tensor):
    """Per column of ``pos`` ((N,) or (N, 2) int64, CUDA, contiguous): (min, max, step) with step as in
    :class:`RopeSpec`.  One small kernel plus a synchronising read the first time a given tensor (object and
    version) is seen; later calls are answered from a cache, so a training loop that reuses its position tensor
    never synchronises (and may be captured into a CUDA graph after its first step)."""
    _require_cuda(pos)
    if pos.dtype != torch.int64 or not pos.is_contiguous():
        raise TypeError("positions must be a contiguous int64 tensor")
    key = id(pos)
    # a tensor made under torch.inference_mode() has no version counter: it is scanned on every call
    cacheable = not pos.is_inference()
    ent = _pos_info_cache.get(key) if cacheable else None
    if ent is not None and ent[0]() is pos and ent[1] == pos._version:
        return ent[2]
    for k in [k for k, e in _pos_info_cache.items() if e[0]() is None]:
        del _pos_info_cache[k]
    stride = 1 if pos.dim() == 1 else pos.shape[1]
    info = torch.empty((8,), dtype=torch.int64, device=pos.device)
    _abi.check(_abi.lib().pom_rope_pos_info(ptr(pos), pos.shape[0], stride, ptr(info), _abi.stream_ptr()),
               "pom_rope_pos_info")
    vals = info.cpu().tolist()
    out = tuple((vals[4 * c], vals[4 * c + 1], 0 if vals[4 * c + 2] else (1 if vals[4 * c + 3] else -1))
                for c in range(stride))
    if cacheable:
        _pos_info_cache[key] = (weakref.ref(pos), pos._version, out)
    return out


def transpose_bf16(src: torch.Tensor) -> torch.Tensor:
    """(rows, cols) bf16 -> its (cols, rows) transpose as a new contiguous tensor."""
    _require_cuda(src)
    if src.dim() != 2 or src.dtype != torch.bfloat16 or src.stride(1) != 1:
        raise ValueError("expected a 2-D bfloat16 tensor with a contiguous last dimension")
    rows, cols = src.shape
    dst = torch.empty((cols, rows), dtype=torch.bfloat16, device=src.device)
    _abi.check(_abi.lib().pom_transpose_bf16(ptr(src), ptr(dst), rows, cols, src.stride(0), rows, _abi.stream_ptr()),
               "pom_transpose_bf16")
    return dst


def _rope_c(spec: Optional[RopeSpec]) -> Rope:
    if spec is None:
        r = Rope()
        r.kind = _abi.ROPE_NONE
        r.pos_stride = 1
        return r
    return spec.to_c()


# ---------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         accumulate: bool = False, split_k: int = 0, alpha: float = 1.0, act: Optional[str] = None,
         residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[m, n] = alpha * sum_k A[m, k] * B[n, k].

    ``a`` is (M, K) — or (K, M) when ``a_mn`` — and ``b`` is (N, K) — or (K, N) when ``b_mn``;
    both row-major with a contiguous last dimension.  bf16 inputs run on the tcgen05 kernel,
    fp32 inputs on the SIMT kernel.  ``accumulate`` adds into a fp32 ``out``.  For bf16 outputs the epilogue can
    apply ``act="gelu"`` and add a bf16 ``residual`` of the output's shape.
    """
    dev = _require_cuda(a, b, out)
    if a.dtype != b.dtype:
        raise TypeError("operand dtypes differ")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"reduction dims differ: {K} vs {Kb}")
    is_bf16 = a.dtype == torch.bfloat16
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an output tensor")
        odt = out_dtype or (torch.bfloat16 if is_bf16 else torch.float32)
        out = torch.empty((M, N), dtype=odt, device=dev)
    if out.shape != (M, N):
        raise ValueError("output shape mismatch")
    if accumulate and out.dtype != torch.float32:
        raise TypeError("accumulate needs a float32 output")
    g = GemmArgs()
    g.A, g.Bm, g.C = ptr(a), ptr(b), ptr(out)
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb, g.ldc = _row_stride(a), _row_stride(b), _row_stride(out)
    g.batches = 1
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.out_mode = _abi.OUT_F32_ACCUM if accumulate else (_abi.OUT_BF16 if out.dtype == torch.bfloat16 else _abi.OUT_F32)
    g.split_k = split_k if accumulate else 1
    g.alpha = alpha
    if act not in (None, "gelu"):
        raise ValueError("act must be None or 'gelu'")
    g.act = 1 if act == "gelu" else 0
    if residual is not None:
        if residual.shape != (M, N) or residual.dtype != torch.bfloat16:
            raise ValueError("residual must be a bfloat16 tensor of the output's shape")
        g.residual, g.ldr = ptr(residual), _row_stride(residual)
    if (g.act or residual is not None) and not (is_bf16 and out.dtype == torch.bfloat16):
        raise TypeError("activation / residual epilogue needs bfloat16 operands and output")
    L = _abi.lib()
    if is_bf16:
        _abi.check(L.pom_gemm_bf16(C.byref(g), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_gemm_bf16")
    else:
        if a.dtype != torch.float32 or out.dtype != torch.float32:
            raise TypeError("fp32 GEMM needs float32 operands and output")
        _abi.check(L.pom_gemm_f32(C.byref(g), _abi.stream_ptr()), "pom_gemm_f32")
    return out


def gemm_batched(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
                 out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                 accumulate: bool = False, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = A[i]·B[i]ᵀ on the tcgen05 kernel, one launch for all batches.

    ``a`` is (batch, M, K) — or (batch, K, M) with ``a_mn`` —, ``b`` is (batch, N, K) — or (batch, K, N) with ``b_mn`` —
    or 2-D (shared by all batches); bf16, last dimension contiguous, any row and batch strides that are multiples of
    8 elements, so heads or samples that sit side by side inside a wider matrix can be passed as strided views.
    ``out`` (batch, M, N) may be such a view too (bf16, fp32, or fp32 accumulate)."""
    dev = _require_cuda(a, b, out, residual)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_batched needs bfloat16 operands")
    nb = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mn else (a.shape[1], a.shape[2])
    bb = b.dim() == 3
    bs = b.shape[1:] if bb else b.shape
    N, Kb = (bs[1], bs[0]) if b_mn else (bs[0], bs[1])
    if K != Kb or (bb and b.shape[0] != nb):
        raise ValueError("operand shapes do not match")
    if a.stride(2) != 1 or b.stride(-1) != 1:
        raise ValueError("last dimensions must be contiguous")
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an output tensor")
        out = torch.empty((nb, M, N), dtype=out_dtype or torch.bfloat16, device=dev)
    if out.shape != (nb, M, N) or out.stride(2) != 1:
        raise ValueError("output shape mismatch")
    g = GemmArgs()
    g.A, g.Bm, g.C = ptr(a), ptr(b), ptr(out)
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb, g.ldc = _ld(a, 1), _ld(b, -2), _ld(out, 1)
    g.batches = nb
    g.a_batch_stride, g.c_batch_stride = a.stride(0), out.stride(0)
    g.b_batched, g.b_batch_stride = int(bb), (b.stride(0) if bb else 0)
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.out_mode = _abi.OUT_F32_ACCUM if accumulate else (_abi.OUT_BF16 if out.dtype == torch.bfloat16 else _abi.OUT_F32)
    g.split_k, g.alpha = 1, 1.0
    if residual is not None:
        if residual.shape != out.shape or residual.dtype != torch.bfloat16 or not residual.is_contiguous() \
                or not out.is_contiguous():
            raise ValueError("residual must be a contiguous bfloat16 tensor of the (contiguous) output's shape")
        g.residual, g.ldr = ptr(residual), _ld(residual, 1)
        g.c_batch_stride = 0
    _abi.check(_abi.lib().pom_gemm_bf16(C.byref(g), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_gemm_bf16")
    return out


def reduce_partials(partial: torch.Tensor, *, denom: Optional[torch.Tensor] = None, scale: float = 1.0,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(B, chunks, P) fp32 -> (B, P): scale * (sum over chunks, in a fixed order) / denom[b]."""
    _require_cuda(partial, denom, out)
    B, chunks, P = partial.shape
    assert partial.dtype == torch.float32 and partial.is_contiguous()
    if out is None:
        out = torch.empty((B, P), dtype=torch.float32, device=partial.device)
    # Few samples and many chunks (one long sequence): the kernel's grid is (P/32, B), so first fold groups of
    # chunks into (B*G, P) with G times as many CTAs, then finish over the G group sums.
    if chunks >= 128 and B * ((P + 31) // 32) < 256:
        G = next((g for g in (32, 16, 8, 4) if chunks % g == 0), 0)
        if G:
            part = torch.empty((B * G, P), dtype=torch.float32, device=partial.device)
            _abi.check(_abi.lib().pom_reduce_partials(ptr(partial), ptr(part), None, 1.0, B * G, chunks // G, P,
                                                      _abi.stream_ptr()), "pom_reduce_partials")
            partial, chunks = part, G
    _abi.check(_abi.lib().pom_reduce_partials(ptr(partial), ptr(out), ptr(denom), scale, B, chunks, P,
                                              _abi.stream_ptr()), "pom_reduce_partials")
    return out


def m_tiles(n_rows: int) -> int:
    return (n_rows + 127) // 128


# ---------------------------------------------------------------------------- fused GEMM phases (bf16)
def tile_weights(mask: torch.Tensor) -> torch.Tensor:
    """(B, N) fp32 key-padding weights -> (B, ceil(N/128)) sums per 128-token tile."""
    _require_cuda(mask)
    B, N = mask.shape
    out = torch.empty((B, m_tiles(N)), dtype=torch.float32, device=mask.device)
    _abi.check(_abi.lib().pom_tile_weights(ptr(mask), ptr(out), B, N, _abi.stream_ptr()), "pom_tile_weights")
    return out


def token_groups(n: int) -> int:
    """Aligned groups of 32 tokens in a sequence of n tokens (the granularity of the fused token-causal path)."""
    return (n + 31) // 32


def ctx_gemm(x: torch.Tensor, w_po: torch.Tensor, coeff: torch.Tensor, *, row_weight: Optional[torch.Tensor] = None,
             save_hp: bool = True, tile_weight: Optional[torch.Tensor] = None, rope: Optional[RopeSpec] = None,
             causal: bool = False):
    """Context phase: returns (partial (B, MT, P) fp32, hp (B, N, P) bf16 or None).  With ``tile_weight``
    (from :func:`tile_weights`) tiles that the mask empties are skipped and their rows of hp stay unwritten.
    ``rope`` (fusable, degree <= 4): the polynomial features are rotated by the token positions before the sum.
    ``causal``: returns (group totals (B, ceil(N/32), P) fp32, hp, pre (B, N, P) bf16) instead — per 32-token group
    the running sums of the features and their totals; :func:`group_scan` turns the totals into carries."""
    dev = _require_cuda(x, w_po, coeff, row_weight)
    B, N, D = x.shape
    P, K = coeff.shape
    hp = torch.empty((B, N, P), dtype=torch.bfloat16, device=dev) if save_hp else None
    a = CtxArgs()
    a.X, a.Wpo, a.coeff, a.row_weight = ptr(x), ptr(w_po), ptr(coeff), ptr(row_weight)
    if causal:
        sums = torch.empty((B, token_groups(N), P), dtype=torch.float32, device=dev)
        pre = torch.empty((B, N, P), dtype=torch.bfloat16, device=dev)
        a.hp_out, a.causal, a.pre_out, a.ld_pre, a.group_sums = ptr(hp), 1, ptr(pre), P, ptr(sums)
        a.ldx, a.ldw, a.ld_hp = _row_stride(x), _row_stride(w_po), P
        a.B, a.N, a.D, a.P, a.K = B, N, D, P, K
        a.rope = _rope_c(rope)
        _abi.check(_abi.lib().pom_ctx_gemm(C.byref(a), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_ctx_gemm")
        return sums, hp, pre
    partial = torch.empty((B, m_tiles(N), P), dtype=torch.float32, device=dev)
    a.hp_out, a.partial = ptr(hp), ptr(partial)
    a.tile_weight = ptr(tile_weight)
    a.ldx, a.ldw, a.ld_hp = _row_stride(x), _row_stride(w_po), P
    a.B, a.N, a.D, a.P, a.K = B, N, D, P, K
    a.rope = _rope_c(rope)
    _abi.check(_abi.lib().pom_ctx_gemm(C.byref(a), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_ctx_gemm")
    return partial, hp


def group_scan(sums: torch.Tensor, carry_in: Optional[torch.Tensor] = None, *, reverse: bool = False,
               want_total: bool = False) -> Optional[torch.Tensor]:
    """In-place exclusive scan over the 32-token groups of (B, groups, P) fp32 totals (forward: prefix, reverse:
    suffix), seeded with ``carry_in`` (B, P).  Returns the (B, P) sum over the groups when ``want_total``."""
    _require_cuda(sums, carry_in)
    B, G, P = sums.shape
    assert sums.dtype == torch.float32 and sums.is_contiguous()
    scratch = torch.empty((B * ((G + 31) // 32) * P,), dtype=torch.float32, device=sums.device)
    total = torch.empty((B, P), dtype=torch.float32, device=sums.device) if want_total else None
    _abi.check(_abi.lib().pom_group_scan(ptr(sums), ptr(carry_in), ptr(total), ptr(scratch), B, G, P, int(reverse),
                                         _abi.stream_ptr()), "pom_group_scan")
    return total


def gate_gemm(x: torch.Tensor, w_se: torch.Tensor, bias: torch.Tensor, h: Optional[torch.Tensor], *,
              save_z: bool = True, rope: Optional[RopeSpec] = None, causal=None):
    """Query phase: returns (SH (B, T, P) bf16, z (B, T, P) bf16 or None). ``h`` is (B, P) fp32.  ``rope``: the
    gate is rotated by the query positions after the hardsigmoid.  ``causal`` = (pre, carry, token_offset): the
    per-token prefix mean (pre + carry[group]) / (token_offset + t + 1) takes the place of ``h``."""
    dev = _require_cuda(x, w_se, bias, h)
    B, T, D = x.shape
    P = w_se.shape[0]
    sh = torch.empty((B, T, P), dtype=torch.bfloat16, device=dev)
    z = torch.empty((B, T, P), dtype=torch.bfloat16, device=dev) if save_z else None
    a = GateArgs()
    a.X, a.Wse, a.bias, a.H = ptr(x), ptr(w_se), ptr(bias), ptr(h)
    a.z_out, a.sh_out = ptr(z), ptr(sh)
    a.ldx, a.ldw, a.ld_z, a.ld_sh = _row_stride(x), _row_stride(w_se), P, P
    a.h_batch_stride, a.h_row_stride = (h.stride(0) if h is not None else 0), 0
    a.B, a.T, a.D, a.P = B, T, D, P
    a.rope = _rope_c(rope)
    if causal is not None:
        pre, carry, offset = causal
        if tuple(pre.shape) != (B, T, P) or tuple(carry.shape) != (B, token_groups(T), P):
            raise ValueError("pre must be (B, T, P) and carry (B, ceil(T/32), P)")
        a.causal, a.pre, a.ld_pre, a.carry, a.token_offset = 1, ptr(pre), P, ptr(carry), int(offset)
    _abi.check(_abi.lib().pom_gate_gemm(C.byref(a), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_gate_gemm")
    return sh, z


def gate_bwd_gemm(dy: torch.Tensor, w_o: torch.Tensor, bias: torch.Tensor, h: Optional[torch.Tensor], z: torch.Tensor,
                  g_out: torch.Tensor, *, rope: Optional[RopeSpec] = None, w_o_t: Optional[torch.Tensor] = None,
                  causal=None):
    """Backward of the query phase. Writes dz into ``g_out`` (a (B*T, P) view with its own row
    stride) and returns (dh_partial, dbias_partial), both (B, MT, P) fp32.  ``rope``: backward of the rotated
    gate; this form reads the output weight transposed: ``w_o_t`` (P, D), or a copy made here when it is None.
    ``causal`` = (pre, carry, token_offset): returns (dbias_partial, suf (B, T, P) bf16, group totals
    (B, ceil(T/32), P) fp32) instead — the running sums, up the rows of every 32-token group, of the gradient of the
    prefix means, for :func:`group_scan` (reverse) and :func:`poly_agg_bwd` (``fused_causal``)."""
    dev = _require_cuda(dy, w_o, bias, h, z, g_out)
    B, T, D = dy.shape
    P = w_o.shape[1]
    dh_p = None if causal is not None else torch.empty((B, m_tiles(T), P), dtype=torch.float32, device=dev)
    db_p = torch.empty((B, m_tiles(T), P), dtype=torch.float32, device=dev)
    a = GateBwdArgs()
    a.dY, a.Wo, a.bias, a.H, a.z = ptr(dy), ptr(w_o), ptr(bias), ptr(h), ptr(z)
    a.g_out, a.dh_partial, a.db_partial = ptr(g_out), ptr(dh_p), ptr(db_p)
    a.ld_dy, a.ldw, a.ld_z, a.ld_g = _row_stride(dy), _row_stride(w_o), _row_stride(z), _row_stride(g_out)
    a.h_batch_stride = h.stride(0) if h is not None else 0
    a.B, a.T, a.D, a.P = B, T, D, P
    a.rope = _rope_c(rope)
    suf = sums = None
    if causal is not None:
        pre, carry, offset = causal
        suf = torch.empty((B, T, P), dtype=torch.bfloat16, device=dev)
        sums = torch.empty((B, token_groups(T), P), dtype=torch.float32, device=dev)
        a.causal, a.pre, a.ld_pre, a.carry, a.token_offset = 1, ptr(pre), P, ptr(carry), int(offset)
        a.suf_out, a.ld_suf, a.group_sums = ptr(suf), P, ptr(sums)
    if rope is not None or causal is not None:
        w_t = w_o_t if w_o_t is not None else transpose_bf16(w_o)
        if tuple(w_t.shape) != (P, D) or w_t.dtype != torch.bfloat16 or not w_t.is_contiguous():
            raise ValueError(f"w_o_t must be a contiguous bfloat16 ({P}, {D}) tensor")
        a.WoT, a.ldwt = ptr(w_t), D
    _abi.check(_abi.lib().pom_gate_bwd_gemm(C.byref(a), ptr(_abi.status_word(dev)), _abi.stream_ptr()),
               "pom_gate_bwd_gemm")
    if causal is not None:
        return db_p, suf, sums
    return dh_p, db_p


# ---------------------------------------------------------------------------- whole layer (bf16, fused path)
def _layer_args(xq, xc, w_qc, w_ag, bias, coeff, mask, h_past, n_past, frames, rope_c=None, rope_q=None,
                causal=False, token_offset=0):
    B, T, D = xq.shape
    N = T if xc is None else xc.shape[1]
    P, K = coeff.shape
    a = _abi.LayerArgs()
    a.B, a.T, a.N, a.D, a.P, a.K = B, T, N, D, P, K
    a.self_mixing, a.frames, a.n_past = int(xc is None), int(frames), float(n_past or 0.0)
    a.xq, a.xc, a.w_qc, a.w_ag = ptr(xq), ptr(xc), ptr(w_qc), ptr(w_ag)
    a.se_bias, a.coeff, a.mask, a.h_past = ptr(bias), ptr(coeff), ptr(mask), ptr(h_past)
    a.rope_c, a.rope_q = _rope_c(rope_c), _rope_c(rope_q)
    a.causal, a.token_offset = int(bool(causal)), int(token_offset)
    nbytes = int(_abi.lib().pom_layer_workspace_bytes(C.byref(a)))
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=xq.device)
    a.workspace, a.workspace_bytes = ptr(ws), nbytes
    return a, ws


def layer_fwd(xq, xc, w_qc, w_ag, bias, coeff, *, mask=None, h_past=None, n_past=0.0, residual=None, frames=1,
              save=True, rope_c: Optional[RopeSpec] = None, rope_q: Optional[RopeSpec] = None, causal=False,
              token_offset=0):
    """Whole fused forward (``xc`` None = self-mixing), optionally with rotary embedding of the context features
    (``rope_c``) and of the gate (``rope_q``).  Returns (y, hp, z, sh, H, denom); hp and z are None unless ``save``;
    denom is None without a mask.  ``causal``: the token-causal prefix mean; H is then the (B, ceil(N/32), P) group
    carries and the seventh return value the (B, N, P) bf16 running sums ``pre`` (both needed by :func:`layer_bwd`)."""
    dev = _require_cuda(xq, xc, w_qc, w_ag, bias, coeff, mask, h_past, residual)
    a, ws = _layer_args(xq, xc, w_qc, w_ag, bias, coeff, mask, h_past, n_past, frames, rope_c, rope_q, causal,
                        token_offset)
    B, T, N, D, P = a.B, a.T, a.N, a.D, a.P
    bf = dict(dtype=torch.bfloat16, device=dev)
    y, sh = torch.empty((B, T, D), **bf), torch.empty((B, T, P), **bf)
    hp = torch.empty((B, N, P), **bf) if save else None
    z = torch.empty((B, T, P), **bf) if save else None
    denom = torch.empty((B,), dtype=torch.float32, device=dev) if mask is not None else None
    a.save, a.residual = int(save), ptr(residual)
    a.y, a.hp, a.z, a.sh, a.denom = ptr(y), ptr(hp), ptr(z), ptr(sh), ptr(denom)
    pre = None
    if causal:
        pre = torch.empty((B, N, P), **bf)
        H = torch.empty((B, token_groups(N), P), dtype=torch.float32, device=dev)
        a.pre, a.carry = ptr(pre), ptr(H)
    else:
        H = torch.empty((B, P), dtype=torch.float32, device=dev)
        a.H = ptr(H)
    _abi.check(_abi.lib().pom_layer_fwd(C.byref(a), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_layer_fwd")
    if causal:
        return y, hp, z, sh, H, denom, pre
    return y, hp, z, sh, H, denom


def layer_bwd(dy, xq, xc, w_qc, w_ag, bias, coeff, hp, z, sh, H, *, mask=None, denom=None, h_past=None, n_past=0.0,
              dh_state=None, frames=1, want_d_hpast=False, rope_c: Optional[RopeSpec] = None,
              rope_q: Optional[RopeSpec] = None, w_ag_t: Optional[torch.Tensor] = None, causal=None, token_offset=0,
              flat_out: Optional[torch.Tensor] = None):
    """Whole fused backward.  Returns (dxq, dxc or None, flat fp32 parameter gradients
    [dWqc | dWo | dbias | dcoeff], d_hpast (B, P) fp32 or None).  With ``rope_q`` or ``causal`` the transposed output
    weight ``w_ag_t`` (P, D) is required; ``causal`` = the running sums ``pre`` of the forward call, whose carries
    come in ``H``.  The flat buffer is zero-filled by the call."""
    dev = _require_cuda(dy, xq, xc, w_qc, w_ag, bias, coeff, hp, z, sh, H, mask, denom, h_past, dh_state, w_ag_t, causal)
    a, ws = _layer_args(xq, xc, w_qc, w_ag, bias, coeff, mask, h_past, n_past, frames, rope_c, rope_q,
                        causal is not None, token_offset)
    a.w_ag_t = ptr(w_ag_t)
    B, T, N, D, P, K = a.B, a.T, a.N, a.D, a.P, a.K
    bf = dict(dtype=torch.bfloat16, device=dev)
    G = torch.empty((B * T * 2 * P if xc is None else (B * N + B * T) * P,), **bf)
    dxq = torch.empty((B, T, D), **bf)
    dxc = None if xc is None else torch.empty((B, N, D), **bf)
    n_flat = 2 * P * D + D * P + P + P * K
    flat = flat_out  # ``flat_out``: caller-owned fp32 accumulators (e.g. the gradient region of a peer exchange)
    if flat is None:
        flat = torch.empty((n_flat,), dtype=torch.float32, device=dev)
    elif flat.dtype != torch.float32 or flat.numel() < n_flat or not flat.is_contiguous() or flat.device != dev:
        raise ValueError(f"flat_out must be a contiguous float32 tensor of at least {n_flat} elements on {dev}")
    d_hpast = torch.empty((B, P), dtype=torch.float32, device=dev) if (want_d_hpast and h_past is not None) else None
    a.hp, a.z, a.sh, a.denom = ptr(hp), ptr(z), ptr(sh), ptr(denom)
    if causal is not None:
        a.pre, a.carry = ptr(causal), ptr(H)
    else:
        a.H = ptr(H)
    a.dy, a.dh_state, a.G, a.dxq, a.dxc = ptr(dy), ptr(dh_state), ptr(G), ptr(dxq), ptr(dxc)
    a.grads, a.d_hpast = ptr(flat), ptr(d_hpast)
    _abi.check(_abi.lib().pom_layer_bwd(C.byref(a), ptr(_abi.status_word(dev)), _abi.stream_ptr()), "pom_layer_bwd")
    return dxq, dxc, flat, d_hpast


# ---------------------------------------------------------------------------- stand-alone operators
def agg_chunks(n: int) -> int:
    return int(_abi.lib().pom_agg_chunks(n))


def poly_agg_fwd(x: torch.Tensor, coeff: torch.Tensor, *, row_weight: Optional[torch.Tensor] = None,
                 causal: bool = False, rope: Optional[RopeSpec] = None, carry: Optional[torch.Tensor] = None,
                 token_offset: int = 0, want_total: bool = False, per_token: bool = False):
    """Non-causal: returns partial sums (B, chunks, P) fp32 (finish with reduce_partials).
    Causal: returns (out (B, N, P) of x.dtype, total (B, P) fp32 or None).
    ``per_token``: returns each token's own rotated polynomial features (B, N, P), no reduction."""
    dev = _require_cuda(x, coeff, row_weight, carry)
    B, N, P = x.shape
    K = coeff.shape[1]
    chunks = agg_chunks(N)
    causal = causal or per_token
    partial = None if per_token else torch.empty((B, chunks, P), dtype=torch.float32, device=dev)
    out = torch.empty((B, N, P), dtype=x.dtype, device=dev) if causal else None
    total = torch.empty((B, P), dtype=torch.float32, device=dev) if (causal and want_total) else None
    a = AggArgs()
    a.x, a.coeff, a.row_weight, a.carry = ptr(x), ptr(coeff), ptr(row_weight), ptr(carry)
    a.partial, a.out, a.total = ptr(partial), ptr(out), ptr(total)
    a.ldx, a.ld_out, a.token_offset = _row_stride(x), P, token_offset
    a.B, a.N, a.P, a.K = B, N, P, K
    a.dtype, a.causal = _abi.dtype_code(x.dtype), (2 if per_token else int(causal))
    a.rope = _rope_c(rope)
    _abi.check(_abi.lib().pom_poly_agg_fwd(C.byref(a), _abi.stream_ptr()), "pom_poly_agg_fwd")
    if per_token:
        return out
    if causal:
        return out, total
    return partial


def poly_agg_bwd(x: torch.Tensor, coeff: torch.Tensor, *, dx_out: torch.Tensor, dH: Optional[torch.Tensor] = None,
                 dout: Optional[torch.Tensor] = None, row_weight: Optional[torch.Tensor] = None,
                 denom: Optional[torch.Tensor] = None, scale: float = 1.0, causal: bool = False,
                 rope: Optional[RopeSpec] = None, carry: Optional[torch.Tensor] = None, token_offset: int = 0,
                 want_total: bool = False, totals_only: bool = False, dcoeff_out: Optional[torch.Tensor] = None,
                 per_token: bool = False, fused_causal=None):
    """Writes dx into ``dx_out`` (a (B, N, P) view, own row stride) and returns
    (dcoeff (P, K) fp32, total (B, P) fp32 or None).  ``fused_causal`` = (suf, carry): the gradient of token n's
    features is suf[b, n] + carry[b, n // 32] (outputs of the causal :func:`gate_bwd_gemm` and :func:`group_scan`)."""
    dev = _require_cuda(x, coeff, dx_out, dH, dout, row_weight, denom, carry)
    B, N, P = x.shape
    K = coeff.shape[1]
    chunks = agg_chunks(N)
    dcp = torch.empty((1, B * chunks, P * K), dtype=torch.float32, device=dev)
    causal = causal or per_token
    partial = torch.empty((B, chunks, P), dtype=torch.float32, device=dev) if (causal and not per_token) else None
    total = torch.empty((B, P), dtype=torch.float32, device=dev) if (causal and want_total) else None
    if fused_causal is not None:
        dout, partial = fused_causal
        if tuple(dout.shape) != (B, N, P) or tuple(partial.shape) != (B, token_groups(N), P):
            raise ValueError("fused_causal needs suf (B, N, P) and carry (B, ceil(N/32), P)")
    a = AggBwdArgs()
    a.x, a.coeff, a.row_weight, a.denom = ptr(x), ptr(coeff), ptr(row_weight), ptr(denom)
    a.dH, a.dout, a.carry, a.partial, a.total = ptr(dH), ptr(dout), ptr(carry), ptr(partial), ptr(total)
    a.dx, a.dcoeff_partial = ptr(dx_out), ptr(dcp)
    a.ldx, a.ld_dx = _row_stride(x), _row_stride(dx_out)
    a.ld_dout = _row_stride(dout) if dout is not None else 0
    a.token_offset, a.scale = token_offset, scale
    a.B, a.N, a.P, a.K = B, N, P, K
    a.dtype, a.causal, a.phase = _abi.dtype_code(x.dtype), (2 if per_token else int(causal)), int(totals_only)
    if fused_causal is not None:
        a.causal = 3
    a.rope = _rope_c(rope)
    _abi.check(_abi.lib().pom_poly_agg_bwd(C.byref(a), _abi.stream_ptr()), "pom_poly_agg_bwd")
    if totals_only:
        return None, total
    slots = int(_abi.lib().pom_poly_agg_bwd_slots(C.byref(a)))
    dcoeff = reduce_partials(dcp[:, :slots], out=None if dcoeff_out is None else dcoeff_out.view(1, P * K)).view(P, K)
    return dcoeff, total


def _check_h(h: torch.Tensor, per_tok: bool, B: int, T: int, P: int, dtype: torch.dtype) -> None:
    """The selection kernels index a per-token H with the query token: its shape must be that of z."""
    if per_tok:
        if h.dtype != dtype:
            raise TypeError("per-token H must have the dtype of z")
        if tuple(h.shape) != (B, T, P):
            raise ValueError(f"per-token H must have shape {(B, T, P)}, got {tuple(h.shape)}")
    else:
        if h.dtype != torch.float32:
            raise TypeError("broadcast H must be float32")
        if tuple(h.shape) != (B, P):
            raise ValueError(f"broadcast H must have shape {(B, P)}, got {tuple(h.shape)}")


def select_fwd(z: torch.Tensor, bias: Optional[torch.Tensor], h: torch.Tensor, *, rope: Optional[RopeSpec] = None,
               activated: bool = False, row_denom: Optional[torch.Tensor] = None) -> torch.Tensor:
    """SH = R·hardsigmoid(z + bias) ⊙ H.  ``h`` is (B, P) fp32 (one vector per sample) or (B, T, P) of z.dtype."""
    dev = _require_cuda(z, bias, h)
    B, T, P = z.shape
    per_tok = h.dim() == 3
    _check_h(h, per_tok, B, T, P, z.dtype)
    sh = torch.empty((B, T, P), dtype=z.dtype, device=dev)
    a = SelectArgs()
    a.z, a.bias, a.H, a.sh = ptr(z), ptr(bias), ptr(h), ptr(sh)
    a.ld_z, a.ld_h, a.ld_sh = _row_stride(z), (_row_stride(h) if per_tok else 0), P
    a.B, a.T, a.P = B, T, P
    a.dtype, a.h_per_token, a.activated = _abi.dtype_code(z.dtype), int(per_tok), int(activated)
    a.row_denom = ptr(row_denom)
    a.rope = _rope_c(rope)
    _abi.check(_abi.lib().pom_select_fwd(C.byref(a), _abi.stream_ptr()), "pom_select_fwd")
    return sh


def select_bwd(dsh: torch.Tensor, z: torch.Tensor, bias: Optional[torch.Tensor], h: torch.Tensor, dz_out: torch.Tensor,
               *, rope: Optional[RopeSpec] = None, activated: bool = False, dbias_out: Optional[torch.Tensor] = None,
               row_denom: Optional[torch.Tensor] = None):
    """Returns (dH, dbias): dH is (B, P) fp32 un-normalised sum over tokens when ``h`` is per-sample,
    else the per-token (B, T, P) gradient in z.dtype.  dz is written into ``dz_out``."""
    dev = _require_cuda(dsh, z, bias, h, dz_out)
    B, T, P = z.shape
    per_tok = h.dim() == 3
    _check_h(h, per_tok, B, T, P, z.dtype)
    if tuple(dsh.shape) != (B, T, P):
        raise ValueError(f"dsh must have the shape of z {(B, T, P)}, got {tuple(dsh.shape)}")
    chunks = agg_chunks(T)
    db_p = torch.empty((1, B * chunks, P), dtype=torch.float32, device=dev)
    dh_p = None if per_tok else torch.empty((B, chunks, P), dtype=torch.float32, device=dev)
    dh_tok = torch.empty((B, T, P), dtype=z.dtype, device=dev) if per_tok else None
    a = SelectBwdArgs()
    a.dsh, a.z, a.bias, a.H = ptr(dsh), ptr(z), ptr(bias), ptr(h)
    a.dz, a.dbias_partial, a.dh_partial, a.dh_tok = ptr(dz_out), ptr(db_p), ptr(dh_p), ptr(dh_tok)
    a.ld_dsh, a.ld_z, a.ld_dz = _row_stride(dsh), _row_stride(z), _row_stride(dz_out)
    a.ld_h, a.ld_dh = (_row_stride(h) if per_tok else 0), P
    a.B, a.T, a.P = B, T, P
    a.dtype, a.h_per_token, a.activated = _abi.dtype_code(z.dtype), int(per_tok), int(activated)
    a.row_denom = ptr(row_denom)
    a.rope = _rope_c(rope)
    _abi.check(_abi.lib().pom_select_bwd(C.byref(a), _abi.stream_ptr()), "pom_select_bwd")
    dbias = reduce_partials(db_p, out=None if dbias_out is None else dbias_out.view(1, P)).view(P)
    dH = dh_tok if per_tok else reduce_partials(dh_p)
    return dH, dbias


def _heads_args(s: torch.Tensor, h: torch.Tensor, dtype: torch.dtype) -> SelectHeadsArgs:
    B, T, heads = s.shape
    per_tok = h.dim() == 3
    P = h.shape[-1]
    if s.dtype != torch.float32 or not s.is_contiguous():
        raise TypeError("the per-head gate must be a contiguous float32 tensor")
    _check_h(h, per_tok, B, T, P, dtype)
    a = SelectHeadsArgs()
    a.s, a.H = ptr(s), ptr(h)
    a.ld_h = _row_stride(h) if per_tok else 0
    a.B, a.T, a.P, a.heads = B, T, P, heads
    a.dtype, a.h_per_token = _abi.dtype_code(dtype), int(per_tok)
    return a


def select_heads_fwd(s: torch.Tensor, h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """SH[b,t,p] = s[b,t,head(p)] * H: s (B, T, heads) fp32; H (B, P) fp32 or (B, T, P) of ``dtype``."""
    dev = _require_cuda(s, h)
    a = _heads_args(s, h, dtype)
    sh = torch.empty((a.B, a.T, a.P), dtype=dtype, device=dev)
    a.sh, a.ld_sh = ptr(sh), a.P
    _abi.check(_abi.lib().pom_select_heads_fwd(C.byref(a), _abi.stream_ptr()), "pom_select_heads_fwd")
    return sh


def select_heads_bwd(dsh: torch.Tensor, s: torch.Tensor, h: torch.Tensor, ds_out: torch.Tensor) -> torch.Tensor:
    """Adds the gate gradient into ``ds_out`` (B, T, heads) fp32 (zeroed by the caller) and returns dH:
    (B, P) fp32 summed over tokens when H is per sample, else per token in dsh.dtype."""
    dev = _require_cuda(dsh, s, h, ds_out)
    a = _heads_args(s, h, dsh.dtype)
    per_tok = bool(a.h_per_token)
    chunks = agg_chunks(a.T)
    dh_p = None if per_tok else torch.empty((a.B, chunks, a.P), dtype=torch.float32, device=dev)
    dh_tok = torch.empty((a.B, a.T, a.P), dtype=dsh.dtype, device=dev) if per_tok else None
    a.dsh, a.ld_dsh, a.ds = ptr(dsh), _row_stride(dsh), ptr(ds_out)
    a.dh_partial, a.dh_tok, a.ld_dh = ptr(dh_p), ptr(dh_tok), a.P
    _abi.check(_abi.lib().pom_select_heads_bwd(C.byref(a), _abi.stream_ptr()), "pom_select_heads_bwd")
    return dh_tok if per_tok else reduce_partials(dh_p)


# ---------------------------------------------------------------------------- multi-head gate, collapsed output side
def heads_supported(heads: int, D: int, P: int) -> bool:
    return bool(_abi.lib().pom_heads_supported(heads, D, P))


def _heads_common(B, T, D, P, heads, dtype):
    a = _abi.HeadsArgs()
    a.B, a.T, a.D, a.P, a.heads, a.dtype = B, T, D, P, heads, _abi.dtype_code(dtype)
    return a


def heads_mix(H: torch.Tensor, w_ag: torch.Tensor, heads: int) -> torch.Tensor:
    """Mb[b, h, d] = sum over the channels p of head h of H[b, p] * Wo[d, p]  ->  (B, heads, D) fp32."""
    dev = _require_cuda(H, w_ag)
    B, P = H.shape
    D = w_ag.shape[0]
    if w_ag.dtype == torch.bfloat16:  # one strided-batched tensor-core launch over the heads; Mb in bf16
        hd = P // heads
        Mb = torch.empty((B, heads, D), dtype=torch.bfloat16, device=dev)
        gemm_batched(to_bf16(H).view(B, heads, hd).transpose(0, 1), w_ag.view(D, heads, hd).transpose(0, 1),
                     out=Mb.transpose(0, 1))
        return Mb
    Mb = torch.empty((B, heads, D), dtype=torch.float32, device=dev)
    a = _heads_common(B, 1, D, P, heads, w_ag.dtype)
    a.H, a.Wo, a.Mb, a.ldw = ptr(H), ptr(w_ag), ptr(Mb), _row_stride(w_ag)
    _abi.check(_abi.lib().pom_heads_mix(C.byref(a), _abi.stream_ptr()), "pom_heads_mix")
    return Mb


def heads_out_fwd(s: torch.Tensor, Mb: torch.Tensor, dtype: torch.dtype, residual: Optional[torch.Tensor] = None):
    """y[b, t, :] = sum_h s[b, t, h] * Mb[b, h, :] (+ residual): s (B, T, heads) fp32 -> (B, T, D) of ``dtype``."""
    dev = _require_cuda(s, Mb, residual)
    B, T, heads = s.shape
    D = Mb.shape[2]
    if dtype == torch.bfloat16:  # per sample: (T x heads) · (heads x D), the inner dimension zero-padded by TMA
        return gemm_batched(to_bf16(s), Mb, b_mn=True, residual=residual)
    y = torch.empty((B, T, D), dtype=dtype, device=dev)
    a = _heads_common(B, T, D, heads, heads, dtype)  # P is not used by this call; any multiple of heads
    a.s, a.Mb, a.y, a.residual = ptr(s), ptr(Mb), ptr(y), ptr(residual)
    _abi.check(_abi.lib().pom_heads_out_fwd(C.byref(a), _abi.stream_ptr()), "pom_heads_out_fwd")
    return y


def heads_out_bwd(dy: torch.Tensor, s: torch.Tensor, Mb: torch.Tensor):
    """Returns (ds (B, T, heads) fp32, dMb (B, heads, D) fp32)."""
    dev = _require_cuda(dy, s, Mb)
    B, T, heads = s.shape
    D = Mb.shape[2]
    if dy.dtype == torch.bfloat16:
        ds = gemm_batched(dy, Mb, out_dtype=torch.float32)                              # (B, T, heads)
        dMb = gemm_batched(to_bf16(s), dy, a_mn=True, b_mn=True, out_dtype=torch.float32)  # (B, heads, D)
        return ds, dMb
    ds = torch.empty((B, T, heads), dtype=torch.float32, device=dev)
    dMb = torch.empty((B, heads, D), dtype=torch.float32, device=dev)
    part = torch.empty((B, (T + 127) // 128, heads, D), dtype=torch.float32, device=dev)
    a = _heads_common(B, T, D, heads, heads, dy.dtype)
    a.dy, a.s, a.Mb, a.ds, a.dMb_partial, a.dMb = ptr(dy), ptr(s), ptr(Mb), ptr(ds), ptr(part), ptr(dMb)
    _abi.check(_abi.lib().pom_heads_out_bwd(C.byref(a), _abi.stream_ptr()), "pom_heads_out_bwd")
    return ds, dMb


def heads_mix_bwd(dMb: torch.Tensor, H: torch.Tensor, w_ag: torch.Tensor, dwo_accum: torch.Tensor) -> torch.Tensor:
    """Returns dH (B, P) fp32 and adds the output-projection gradient into ``dwo_accum`` ((D, P) fp32, contiguous)."""
    dev = _require_cuda(dMb, H, w_ag, dwo_accum)
    B, heads, D = dMb.shape
    P = H.shape[1]
    assert dwo_accum.is_contiguous() and dwo_accum.dtype == torch.float32 and dwo_accum.shape == (D, P)
    dH = torch.empty((B, P), dtype=torch.float32, device=dev)
    if w_ag.dtype == torch.bfloat16:
        hd = P // heads
        g16 = to_bf16(dMb).transpose(0, 1)                       # (heads, B, D) view
        w3 = w_ag.view(D, heads, hd).transpose(0, 1)             # (heads, D, hd) view
        gemm_batched(g16, w3, b_mn=True, out=dH.view(B, heads, hd).transpose(0, 1))
        gemm_batched(g16, to_bf16(H).view(B, heads, hd).transpose(0, 1), a_mn=True, b_mn=True,
                     out=dwo_accum.view(D, heads, hd).transpose(0, 1), accumulate=True)
        return dH
    a = _heads_common(B, 1, D, P, heads, w_ag.dtype)
    a.dMb, a.H, a.Wo, a.dH, a.dWo, a.ldw = ptr(dMb), ptr(H), ptr(w_ag), ptr(dH), ptr(dwo_accum), _row_stride(w_ag)
    _abi.check(_abi.lib().pom_heads_mix_bwd(C.byref(a), _abi.stream_ptr()), "pom_heads_mix_bwd")
    return dH


def state_merge(h_past: torch.Tensor, h_cur: torch.Tensor, n_past: float) -> torch.Tensor:
    _require_cuda(h_past, h_cur)
    out = torch.empty_like(h_cur)
    _abi.check(_abi.lib().pom_state_merge(ptr(h_past), ptr(h_cur), ptr(out), float(n_past), h_cur.numel(),
                                          _abi.stream_ptr()), "pom_state_merge")
    return out


def frame_prefix_mean(h: torch.Tensor, frames: int, adjoint: bool = False) -> torch.Tensor:
    """(B·F, P) fp32 per-frame means -> running mean over the frames of each sample (or its adjoint)."""
    _require_cuda(h)
    rows, P = h.shape
    if h.dtype != torch.float32 or not h.is_contiguous() or rows % frames:
        raise ValueError("expected a contiguous fp32 (B*F, P) tensor")
    out = torch.empty_like(h)
    _abi.check(_abi.lib().pom_frame_prefix_mean(ptr(h), ptr(out), rows // frames, frames, P, int(adjoint),
                                                _abi.stream_ptr()), "pom_frame_prefix_mean")
    return out


def zeros_f32(n: int, device) -> torch.Tensor:
    """Flat fp32 buffer of n zeros (allocation by PyTorch, fill by cudaMemsetAsync on the current stream)."""
    out = torch.empty((n,), dtype=torch.float32, device=device)
    _abi.check(_abi.lib().pom_fill_zero(ptr(out), out.numel() * 4, _abi.stream_ptr()), "pom_fill_zero")
    return out


def fill_zero(t: torch.Tensor) -> torch.Tensor:
    """Zero an existing contiguous tensor in place on the current stream."""
    _require_cuda(t)
    _abi.check(_abi.lib().pom_fill_zero(ptr(t), t.numel() * t.element_size(), _abi.stream_ptr()), "pom_fill_zero")
    return t


def clone(src: torch.Tensor) -> torch.Tensor:
    """Copy of a contiguous CUDA tensor (asynchronous device-to-device copy on the current stream)."""
    _require_cuda(src)
    if not src.is_contiguous():
        raise ValueError("expected a contiguous tensor")
    out = torch.empty_like(src)
    _abi.check(_abi.lib().pom_copy_bytes(ptr(out), ptr(src), src.numel() * src.element_size(), _abi.stream_ptr()),
               "pom_copy_bytes")
    return out


def to_bf16(src: torch.Tensor) -> torch.Tensor:
    _require_cuda(src)
    src = src.contiguous()
    out = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    _abi.check(_abi.lib().pom_cast_f32_to_bf16(ptr(src), ptr(out), src.numel(), _abi.stream_ptr()), "pom_cast")
    return out


def to_f32(src: torch.Tensor) -> torch.Tensor:
    _require_cuda(src)
    src = src.contiguous()
    out = torch.empty(src.shape, dtype=torch.float32, device=src.device)
    _abi.check(_abi.lib().pom_cast_bf16_to_f32(ptr(src), ptr(out), src.numel(), _abi.stream_ptr()), "pom_cast")
    return out


def launch_count() -> int:
    return int(_abi.lib().pom_launch_count())
