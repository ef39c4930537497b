"""``PoMRoPE`` — drop-in for the reference's ``pom.PoMRoPE`` (reference pom/pom_rope.py:303-526).

The polynomial features of each context token are rotated by that token's position before
aggregation, and the hardsigmoid gate of each query token is rotated by the query position
before gating.  1-D positions pair channel p with p + P/2; 2-D (row, col) positions rotate the
first half of the channels by the row index and the second half by the column index.
Table buffers keep the reference names (``freqs_cos``/``freqs_sin`` or ``row_cos``/``row_sin``/
``col_cos``/``col_sin``) so state dicts interchange.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _abi, ops
from .functional import LayerSpec, SeqShard, _derived_of, _mask_kind, eager_only, on_tensor_device, pom_layer
from .ops import RopeSpec
from .operators import apply_rope_1d, apply_rope_2d  # noqa: F401  (the reference defines them in this module)
from .pom import PoM


def precompute_freqs_1d(dim: int, max_seq_len: int, base: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables (max_seq_len, dim // 2) with theta_k = base^(-k / (dim/2))  (reference pom/pom_rope.py:93-118)."""
    assert dim % 2 == 0, f"dim must be even for 1-D RoPE, got {dim}"
    half = dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), inv_freq)
    return ang.cos(), ang.sin()


def precompute_freqs_2d(dim: int, max_h: int, max_w: int, base: float = 10000.0):
    """Row and column cos/sin tables, each (max, dim // 4)  (reference pom/pom_rope.py:121-149)."""
    assert dim % 4 == 0, f"dim must be divisible by 4 for 2-D RoPE, got {dim}"
    quarter = dim // 4
    inv_freq = 1.0 / (base ** (torch.arange(0, quarter, dtype=torch.float32) / quarter))
    ra = torch.outer(torch.arange(max_h, dtype=torch.float32), inv_freq)
    ca = torch.outer(torch.arange(max_w, dtype=torch.float32), inv_freq)
    return ra.cos(), ra.sin(), ca.cos(), ca.sin()


class PoMRoPE(PoM):
    """Polynomial Mixer with rotary position embedding.

    Extra arguments: ``max_seq_len`` (1-D table length), ``max_h`` / ``max_w`` (2-D table sizes),
    ``rope_base``, ``rope_2d``.
    """

    def __init__(self, dim: int, degree: int, expand: int, n_groups: int = 1, n_sel_heads: int = 1, bias: bool = False,
                 max_seq_len: int = 4096, max_h: int = 64, max_w: int = 64, rope_base: float = 10000.0,
                 rope_2d: bool = False):
        super().__init__(dim, degree, expand, n_groups, n_sel_heads, bias)
        self.rope_2d = rope_2d
        rope_dim = dim * expand
        if n_sel_heads > 1:  # same constraints as the reference (pom/pom_rope.py:343-359)
            hd = rope_dim // n_sel_heads
            if rope_2d:
                assert n_sel_heads % 4 == 0, f"n_sel_heads ({n_sel_heads}) must be divisible by 4 for 2-D RoPE"
                assert hd >= 4, f"head_dim ({hd}) must be >= 4 for 2-D RoPE with n_sel_heads > 1"
            else:
                assert n_sel_heads % 2 == 0, f"n_sel_heads ({n_sel_heads}) must be even for 1-D RoPE"
                assert hd >= 2, f"head_dim ({hd}) must be >= 2 for 1-D RoPE with n_sel_heads > 1"
        if rope_2d:
            assert rope_dim % 4 == 0, f"dim * expand ({rope_dim}) must be divisible by 4 for 2-D RoPE"
            rc, rs, cc, cs = precompute_freqs_2d(rope_dim, max_h, max_w, rope_base)
            self.register_buffer("row_cos", rc)
            self.register_buffer("row_sin", rs)
            self.register_buffer("col_cos", cc)
            self.register_buffer("col_sin", cs)
        else:
            assert rope_dim % 2 == 0, f"dim * expand ({rope_dim}) must be even for 1-D RoPE"
            fc, fs = precompute_freqs_1d(rope_dim, max_seq_len, rope_base)
            self.register_buffer("freqs_cos", fc)
            self.register_buffer("freqs_sin", fs)

    def _tables(self, for_gate: bool):
        """fp32 tables; for the per-head gate the columns are sub-sampled so that gate pair k rotates at the
        leading frequency of head k (reference pom/pom_rope.py:417-437).  Derived tables (an fp32 copy of buffers
        that were cast with the module, the sub-sampled gate tables) are kept until their buffer changes."""
        names = ("row_cos", "row_sin", "col_cos", "col_sin") if self.rope_2d else ("freqs_cos", "freqs_sin")
        sub = for_gate and self.n_sel_heads > 1
        r = self._head_copies() if sub else 1
        if self.rope_2d:
            stride, keep = self.head_dim, self.n_sel_heads // 4
        else:
            stride, keep = self.head_dim // 2, self.n_sel_heads // 2

        def make(t: torch.Tensor) -> torch.Tensor:
            t = t.float()
            if sub:
                t = t[:, ::stride][:, :keep]
                if r > 1:  # repeated gate heads: pair k of the r * heads wide gate is copy k % r of pair k // r
                    t = t.repeat_interleave(r, dim=1)
            return t.contiguous()

        what = f"rope_table/{int(sub)}/{r}"
        return [_derived_of(getattr(self, n), what, make) for n in names]

    def _default_positions(self, n_tokens: int, device) -> torch.Tensor:
        """0..n-1 on ``device``, one tensor per (length, device) so that its position scan is cached."""
        cache = self.__dict__.setdefault("_arange_cache", {})
        key = (n_tokens, str(device))
        if key not in cache:
            if len(cache) >= 16:  # many distinct lengths (variable-length batches): do not let them pile up
                cache.clear()
            with torch.inference_mode(False):  # an ordinary tensor, so that its position scan can be cached
                cache[key] = torch.arange(n_tokens, device=device, dtype=torch.int64)
        return cache[key]

    @staticmethod
    def _checked_steps(pos: torch.Tensor, heights) -> Tuple[int, ...]:
        """Validates the positions against the table heights (the reference's table lookup raises an index
        error for a position outside its tables, pom/pom_rope.py:171-172) and returns their group structure."""
        info = ops.rope_pos_info(pos)
        for (lo, hi, _), height, name in zip(info, heights, ("row / sequence", "column")):
            if lo < 0 or hi >= height:
                raise IndexError(f"{name} positions span [{lo}, {hi}] but the rotary table has {height} rows "
                                 "(raise max_seq_len / max_h / max_w)")
        return tuple(step for _, _, step in info)

    def _rope_spec(self, n_tokens: int, positions, positions_hw, device, for_gate: bool = False) -> RopeSpec:
        tabs = self._tables(for_gate)
        if self.rope_2d:
            if positions_hw is None:
                raise ValueError("positions_hw (N, 2) must be provided when rope_2d=True")
            pos = positions_hw.to(device=device, dtype=torch.int64).contiguous()
            if pos.shape != (n_tokens, 2):
                raise ValueError(f"positions_hw must have shape ({n_tokens}, 2)")
            steps = self._checked_steps(pos, (tabs[0].shape[0], tabs[2].shape[0]))
            return RopeSpec(_abi.ROPE_2D, tabs[0], tabs[1], pos, tabs[2], tabs[3], steps=steps)
        if positions is None:
            positions = self._default_positions(n_tokens, device)
        pos = positions.to(device=device, dtype=torch.int64).contiguous()
        if pos.shape != (n_tokens,):
            raise ValueError(f"positions must have shape ({n_tokens},)")
        steps = self._checked_steps(pos, (tabs[0].shape[0],))
        return RopeSpec(_abi.ROPE_1D, tabs[0], tabs[1], pos, steps=(steps[0], -1))

    @eager_only
    @on_tensor_device
    def forward(self, xq: torch.Tensor, xc: Optional[torch.Tensor] = None, mask=None,
                positions: Optional[torch.Tensor] = None, ctx_positions: Optional[torch.Tensor] = None,
                positions_hw: Optional[torch.Tensor] = None, ctx_positions_hw: Optional[torch.Tensor] = None,
                shard: Optional[SeqShard] = None, grad_peer=None) -> torch.Tensor:
        """As ``PoM.forward`` plus token positions: ``positions`` (T,) / ``ctx_positions`` (N,) int64 for
        1-D tables (default 0..T-1; the context defaults to the query positions under self-mixing, else
        0..N-1), ``positions_hw`` (T, 2) / ``ctx_positions_hw`` (N, 2) for 2-D tables.  ``shard`` and ``grad_peer``
        (extensions) as in ``PoM.forward``."""
        self_mixing = xc is None or xc is xq
        kind = _mask_kind(mask)
        if kind == "block":
            raise NotImplementedError("BlockCausal is not combined with rotary embedding")
        T = xq.shape[1]
        N = T if self_mixing else xc.shape[1]
        cpos = ctx_positions if ctx_positions is not None else (positions if self_mixing else None)
        cpos_hw = ctx_positions_hw if ctx_positions_hw is not None else (positions_hw if self_mixing else None)
        rope_q = self._rope_spec(T, positions, positions_hw, xq.device, for_gate=True)
        same = self_mixing and ctx_positions is None and ctx_positions_hw is None and self.n_sel_heads <= 1
        rope_c = rope_q if same else self._rope_spec(N, cpos, cpos_hw, xq.device)
        spec = LayerSpec(degree=self.order, mask_kind=kind, self_mixing=self_mixing, rope_ctx=rope_c, rope_qry=rope_q,
                         shard=shard, n_sel_heads=self._heads(), grad_peer=grad_peer)
        w_qc, se_bias = self._weights()
        xq, xc = self._tokens(self._cast(xq)), (None if self_mixing else self._tokens(self._cast(xc)))
        y, _ = pom_layer(xq, xc, self._cast(w_qc), se_bias, self.po_coeff, self._out_weight(),
                         mask if kind in ("keypad", "full") else None, None, spec)
        return self._finish(y)
