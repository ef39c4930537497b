"""Operator-level entry points under the reference's own names.

The reference exposes its fused kernels as functions that its tests and benchmarks call directly
(``poly_agg_mean_triton`` pom/pom_triton.py:383, ``poly_agg_causal_triton`` pom/pom_triton_causal.py:400,
``poly_agg_masked_triton`` pom/pom_triton_masked.py:402, ``poly_agg_rope_mean_triton`` /
``poly_agg_rope_causal_triton`` pom/pom_triton_rope.py:985, 1020) next to the PyTorch helpers ``pom_activation``
(pom/pom.py:27), ``apply_rope_1d`` / ``apply_rope_2d`` (pom/pom_rope.py:152, 183) and ``_poly_features``
(pom/pom_rope.py:242).  The functions below take the same arguments in the same order, return the same shapes
and raise the same errors; all of them run on the CUDA operators of this package (there is no CPU path) and
are differentiable.  The ``*_triton`` names and the ``TRITON_*_AVAILABLE`` flags are kept as aliases so that a
script written against the reference's modules needs only its import lines changed.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _abi, ops
from .functional import MAX_BATCH, _batch_slices, _f32, _ones, eager_only, on_tensor_device, polynomial_aggregation_
from .ops import RopeSpec

__all__ = [
    "pom_activation", "poly_features", "apply_rope_1d", "apply_rope_2d",
    "poly_agg_mean", "poly_agg_causal", "poly_agg_masked", "poly_agg_rope_mean", "poly_agg_rope_causal",
    "poly_agg_mean_triton", "poly_agg_causal_triton", "poly_agg_masked_triton", "poly_agg_rope_mean_triton",
    "poly_agg_rope_causal_triton", "TRITON_AVAILABLE", "TRITON_CAUSAL_AVAILABLE", "TRITON_MASKED_AVAILABLE",
    "TRITON_ROPE_AVAILABLE",
]


def _check_degree(coeff: torch.Tensor, k: int) -> None:
    if k > 16:
        raise NotImplementedError(f"k ≤ 16 supported (got {k})")
    if coeff.shape[1] != k:
        raise ValueError(f"coeff has {coeff.shape[1]} columns but k={k}")


def _rows(x: torch.Tensor) -> torch.Tensor:
    """(B, N, P) with unit stride along P and the samples laid end to end."""
    if not x.is_cuda:
        raise RuntimeError("pom_b200 has no CPU path: pass CUDA tensors")
    if x.dim() != 3:
        raise ValueError(f"expected a (B, N, D) tensor, got {tuple(x.shape)}")
    B, N, _ = x.shape
    if x.stride(-1) != 1 or (B > 1 and x.stride(0) != x.stride(1) * N):
        x = x.contiguous()
    return x


def _table(t: torch.Tensor, device, width: int, name: str) -> torch.Tensor:
    t = t.to(device=device, dtype=torch.float32).contiguous()
    if t.dim() != 2 or t.shape[1] != width:
        raise ValueError(f"{name} must have shape (positions, {width}), got {tuple(t.shape)}")
    return t


def _positions(pos: Optional[torch.Tensor], n: int, cols: int, device, heights) -> torch.Tensor:
    """int64 positions on the device, checked against the table heights (the reference's table lookup raises
    an IndexError for a position outside its tables, pom/pom_rope.py:171-172)."""
    if pos is None:
        pos = torch.arange(n, device=device, dtype=torch.int64)
    pos = pos.to(device=device, dtype=torch.int64).contiguous()
    want = (n,) if cols == 1 else (n, 2)
    if tuple(pos.shape) != want:
        raise ValueError(f"positions must have shape {want}, got {tuple(pos.shape)}")
    for (lo, hi, _), height in zip(ops.rope_pos_info(pos), heights):
        if lo < 0 or hi >= height:
            raise IndexError(f"positions span [{lo}, {hi}] but the rotary table has {height} rows")
    return pos


def _spec_1d(x: torch.Tensor, positions, freqs_cos, freqs_sin) -> RopeSpec:
    B, N, D = x.shape
    if D % 2 != 0:
        raise ValueError(f"D must be even for RoPE (got {D})")
    cos = _table(freqs_cos, x.device, D // 2, "freqs_cos")
    sin = _table(freqs_sin, x.device, D // 2, "freqs_sin")
    pos = _positions(positions, N, 1, x.device, (cos.shape[0],))
    return RopeSpec(_abi.ROPE_1D, cos, sin, pos)


def _spec_2d(x: torch.Tensor, positions_hw, row_cos, row_sin, col_cos, col_sin) -> RopeSpec:
    B, N, D = x.shape
    if D % 4 != 0:
        raise ValueError(f"D must be divisible by 4 for 2-D RoPE (got {D})")
    tabs = [_table(t, x.device, D // 4, n) for t, n in ((row_cos, "row_cos"), (row_sin, "row_sin"),
                                                        (col_cos, "col_cos"), (col_sin, "col_sin"))]
    if positions_hw is None:
        raise ValueError("positions_hw (N, 2) must be provided for 2-D RoPE")
    pos = _positions(positions_hw, N, 2, x.device, (tabs[0].shape[0], tabs[2].shape[0]))
    return RopeSpec(_abi.ROPE_2D, tabs[0], tabs[1], pos, tabs[2], tabs[3])


def _in_batch_slices(fn, x: torch.Tensor, *shared):
    """``fn(x, *shared)``, in runs of at most MAX_BATCH samples when x has more (the kernels put the sample index in
    a grid dimension; the samples are independent)."""
    if x.dim() != 3 or x.shape[0] <= MAX_BATCH:
        return fn(x, *shared)
    return torch.cat([fn(x[sl], *shared) for sl in _batch_slices(x.shape[0])], dim=0)


# --------------------------------------------------------------------------- rotation alone
class _Rotate(torch.autograd.Function):
    """y = R(positions) · x and dx = Rᵀ · dy: the selection operator with the gate taken as given (no
    hardsigmoid, no bias) and the constant 1 as the aggregate."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, x, spec: RopeSpec):
        x = _rows(x)
        ctx.spec = spec
        ctx.shape = x.shape
        return ops.select_fwd(x, None, _ones(x.shape[0], x.shape[2], x.device), rope=spec, activated=True)

    @staticmethod
    @on_tensor_device
    def backward(ctx, g):
        B, N, P = ctx.shape
        g = _rows(g)
        dx = torch.empty((B, N, P), dtype=g.dtype, device=g.device)
        # the operator never reads the gate values in this mode, so the gradient stands in for them
        ops.select_bwd(g, g, None, _ones(B, P, g.device), dx, rope=ctx.spec, activated=True)
        return dx, None


@eager_only
@on_tensor_device
def apply_rope_1d(x: torch.Tensor, positions: torch.Tensor, freqs_cos: torch.Tensor,
                  freqs_sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half 1-D rotary embedding: channel k pairs with k + D/2 (reference pom/pom_rope.py:152-180).
    x (B, N, D); positions (N,) int64; freqs_cos / freqs_sin (max_len, D // 2).  Returns (B, N, D)."""
    x = _rows(x)
    return _in_batch_slices(_Rotate.apply, x, _spec_1d(x, positions, freqs_cos, freqs_sin))


@eager_only
@on_tensor_device
def apply_rope_2d(x: torch.Tensor, positions_hw: torch.Tensor, row_cos: torch.Tensor, row_sin: torch.Tensor,
                  col_cos: torch.Tensor, col_sin: torch.Tensor) -> torch.Tensor:
    """2-D rotary embedding: the first half of the channels rotates with the row position, the second half with
    the column position, each half pairing k with k + D/4 (reference pom/pom_rope.py:183-235).
    x (B, N, D); positions_hw (N, 2) int64; row_* (max_h, D // 4); col_* (max_w, D // 4)."""
    x = _rows(x)
    return _in_batch_slices(_Rotate.apply, x, _spec_2d(x, positions_hw, row_cos, row_sin, col_cos, col_sin))


# --------------------------------------------------------------------------- per-token polynomial features
class _Features(torch.autograd.Function):
    """f[b, n, p] = sum_k coeff[p, k] act(x[b, n, p])^(k+1) (reference pom/pom_rope.py:242-265, pom/pom.py:83-89)."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, x, coeff):
        x = _rows(x)
        coeff32 = _f32(coeff.contiguous())
        ctx.save_for_backward(x, coeff32)
        ctx.cdt = coeff.dtype
        return ops.poly_agg_fwd(x, coeff32, per_token=True)

    @staticmethod
    @on_tensor_device
    def backward(ctx, g):
        x, coeff32 = ctx.saved_tensors
        dx = torch.empty_like(x)
        dc, _ = ops.poly_agg_bwd(x, coeff32, dx_out=dx, dout=_rows(g), per_token=True)
        dc = dc.contiguous()
        return dx, (dc if ctx.cdt == torch.float32 else ops.to_bf16(dc))


@eager_only
def poly_features(x: torch.Tensor, coeff: torch.Tensor, k: int) -> torch.Tensor:
    """Per-token polynomial features (B, N, D) before any aggregation (the reference's ``_poly_features``)."""
    _check_degree(coeff, k)
    return _in_batch_slices(_Features.apply, x, coeff)


@eager_only
def pom_activation(x: torch.Tensor) -> torch.Tensor:
    """clamp(leaky_relu(x, 0.01), -0.1, 6) (reference pom/pom.py:27-28) for a (B, N, D) tensor: the degree-1
    feature with coefficient 1."""
    one = torch.ones((x.shape[-1], 1), dtype=torch.float32, device=x.device)
    shape = x.shape
    if x.dim() != 3:  # any shape with the channels last
        x = x.reshape(1, -1, shape[-1]) if x.dim() < 3 else x.reshape(-1, shape[-2], shape[-1])
    return _in_batch_slices(_Features.apply, x, one).view(shape)


# --------------------------------------------------------------------------- fused aggregations
def poly_agg_mean(x: torch.Tensor, coeff: torch.Tensor, k: int) -> torch.Tensor:
    """Polynomial features averaged over the tokens: (B, N, D), (D, K) -> (B, 1, D)
    (reference pom/pom_triton.py:383-403)."""
    _check_degree(coeff, k)
    return polynomial_aggregation_(x, coeff, k, None)


def poly_agg_causal(x: torch.Tensor, coeff: torch.Tensor, k: int) -> torch.Tensor:
    """out[b, m] = mean over n <= m of the features: (B, N, D) -> (B, N, D)
    (reference pom/pom_triton_causal.py:400-423)."""
    _check_degree(coeff, k)
    return polynomial_aggregation_(x, coeff, k, "causal")


def poly_agg_masked(x: torch.Tensor, mask: torch.Tensor, coeff: torch.Tensor, k: int) -> torch.Tensor:
    """Mask-weighted mean over the tokens, mask (B, N) of 0/1 or continuous weights: -> (B, 1, D)
    (reference pom/pom_triton_masked.py:402-428)."""
    _check_degree(coeff, k)
    if mask.dim() != 2:
        raise ValueError(f"expected a (B, N) mask, got {tuple(mask.shape)}")
    return polynomial_aggregation_(x, coeff, k, mask)


@eager_only
@on_tensor_device
def poly_agg_rope_mean(x: torch.Tensor, coeff: torch.Tensor, k: int, freqs_cos: torch.Tensor,
                       freqs_sin: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Features, 1-D rotation by position, mean over the tokens: -> (B, 1, D); positions default to 0..N-1
    (reference pom/pom_triton_rope.py:985-1018)."""
    _check_degree(coeff, k)
    x = _rows(x)
    return polynomial_aggregation_(x, coeff, k, None, rope=_spec_1d(x, positions, freqs_cos, freqs_sin))


@eager_only
@on_tensor_device
def poly_agg_rope_causal(x: torch.Tensor, coeff: torch.Tensor, k: int, freqs_cos: torch.Tensor,
                         freqs_sin: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Features, 1-D rotation by position, causal prefix mean: -> (B, N, D)
    (reference pom/pom_triton_rope.py:1020-1053)."""
    _check_degree(coeff, k)
    x = _rows(x)
    return polynomial_aggregation_(x, coeff, k, "causal", rope=_spec_1d(x, positions, freqs_cos, freqs_sin))


# the reference's names for the same entry points
poly_agg_mean_triton = poly_agg_mean
poly_agg_causal_triton = poly_agg_causal
poly_agg_masked_triton = poly_agg_masked
poly_agg_rope_mean_triton = poly_agg_rope_mean
poly_agg_rope_causal_triton = poly_agg_rope_causal
TRITON_AVAILABLE = TRITON_CAUSAL_AVAILABLE = TRITON_MASKED_AVAILABLE = TRITON_ROPE_AVAILABLE = True
