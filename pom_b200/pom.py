"""``PoM`` — drop-in module for the reference's ``pom.PoM`` (reference pom/pom.py:142-280)
running on the B200 kernels of this package.

Constructor arguments, parameter names (``qc_proj.weight``, ``se_bias``, ``po_coeff``,
``ag_proj.weight``; with ``n_groups > 1``: ``po_proj.weight``, ``se_proj.weight``, ``se_proj.bias``) and their
creation order are those of the reference, so a given ``torch.manual_seed`` produces the same weights and
checkpoints interchange.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .functional import LayerSpec, SeqShard, _derived_of, _f32, _mask_kind, _ones, eager_only, on_tensor_device, pom_layer
from .functional import polynomial_aggregation_, polynomial_selection_, pom  # noqa: F401  (defined here in the reference)
from .operators import pom_activation  # noqa: F401


class PoM(nn.Module):
    """Polynomial Mixer layer.

    Args:
        dim:         input/output feature dimension D.
        degree:      polynomial degree K (1..16).
        expand:      channel expansion; the polynomial features have P = expand * dim channels.
        n_groups:    > 1: the polynomial projection is a grouped 1x1 convolution (input slice i feeds output
                     slice i) and the gate projection a separate biased Linear, as in the reference.  The layer
                     runs the grouped projection as one dense tensor-core GEMM on the block-diagonal weight
                     assembled per call (a copy; no arithmetic).
        n_sel_heads: 0 or 1: one gate value per channel; > 1: one gate value per head, shared by the
                     dim*expand / n_sel_heads channels of that head.
        bias:        add a bias to the output projection (and, with n_groups > 1, to the grouped projection).
    """

    def __init__(self, dim: int, degree: int, expand: int, n_groups: int = 1, n_sel_heads: int = 1, bias: bool = False):
        super().__init__()
        assert dim % n_groups == 0, "dim must be divisible by n_groups"
        assert n_sel_heads <= 1 or dim * expand % n_sel_heads == 0, "dim * expand must be divisible by n_sel_heads"
        self.dim = dim
        self.order = degree
        self.order_expand = expand
        self.n_groups = n_groups
        self.n_sel_heads = n_sel_heads
        self.head_dim = dim * expand // max(n_sel_heads, 1)
        self._po_dim = expand * dim
        self._grouped_cache = None  # (key, assembled grouped projection) for calls without autograd
        self._se_dim = n_sel_heads if n_sel_heads > 1 else expand * dim
        # creation order matters for seeded initialisation: (qc_proj, se_bias | po_proj, se_proj), po_coeff, ag_proj
        if n_groups > 1:
            self.po_proj = nn.Conv1d(dim, expand * dim, kernel_size=1, bias=bias, groups=n_groups)
            self.se_proj = nn.Linear(dim, self._se_dim, bias=True)
        else:
            self.qc_proj = nn.Linear(dim, self._po_dim + self._se_dim, bias=False)
            self.se_bias = nn.Parameter(torch.zeros(self._se_dim))
        self.po_coeff = nn.Parameter(torch.randn(dim * expand, degree).clamp(-0.001, 0.001))
        self.ag_proj = nn.Linear(expand * dim, dim, bias=bias)

    # ------------------------------------------------------------------ helpers
    def _spec(self, xq, xc, mask, shard: Optional[SeqShard]) -> Tuple[LayerSpec, Optional[torch.Tensor]]:
        kind = _mask_kind(mask)
        frames = 1
        if kind == "block":
            if mask.frame_len <= 0 or xq.shape[1] % mask.frame_len:
                raise ValueError(f"sequence length {xq.shape[1]} is not a multiple of frame_len {mask.frame_len}")
            kind, frames = "none", xq.shape[1] // mask.frame_len
        spec = LayerSpec(degree=self.order, mask_kind=kind, self_mixing=(xc is None or xc is xq), shard=shard,
                         n_sel_heads=self._heads(), frames=frames)
        return spec, (mask if kind in ("keypad", "full") else None)

    # A bias of the grouped projection (reference pom/pom.py:182, nn.Conv1d(..., bias=bias)) travels as one more
    # input column: the tokens get _BIAS_COLS extra channels (1, 0, ..., 0) and the projection weight as many extra
    # columns, the first of which holds the bias for the polynomial rows and 0 for the gate rows.  Eight columns
    # keep the rows of both operands 16-byte aligned in bf16.
    _BIAS_COLS = 8

    def _tokens(self, x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """The tokens as the projection reads them: unchanged, or with the bias channels appended."""
        if x is None or not self._has_bias_cols():
            return x
        one = x.new_zeros(self._BIAS_COLS)
        one[0] = 1
        return torch.cat([x, one.expand(*x.shape[:-1], self._BIAS_COLS)], dim=-1)

    @staticmethod
    def _autocast_dtype() -> Optional[torch.dtype]:
        """bfloat16 while CUDA autocast to bfloat16 is active, else None.  Under autocast the reference's Linear
        layers compute in bf16 from fp32 master weights; so does this layer (tokens and projection weights are cast
        on the way in, gradients come back in the parameters' own dtype)."""
        try:
            on, dt = torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")
        except TypeError:  # older signature
            on, dt = torch.is_autocast_enabled(), torch.get_autocast_gpu_dtype()
        return dt if on and dt == torch.bfloat16 else None

    def _cast(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """A token tensor or projection weight in the autocast dtype (unchanged outside autocast).  The cast of a
        weight that needs no gradient is kept until the weight changes."""
        dt = self._autocast_dtype()
        if t is None or dt is None or t.dtype == dt or not t.is_floating_point():
            return t
        if isinstance(t, nn.Parameter) and not (torch.is_grad_enabled() and t.requires_grad):
            return _derived_of(t, "autocast", lambda w: w.detach().to(dt))
        return t.to(dt)

    def _head_copies(self) -> int:
        """How many adjacent copies of every gate head the CUDA path works with.  A bf16 gate projection needs
        rows of 16 bytes, that is a multiple of 8 heads; other head counts are brought there by repeating each row
        of the gate weight (and bias, and rotary column) r times: r * heads heads of head_dim / r channels gate
        exactly as heads heads of head_dim channels, and autograd sums the copies' gradients."""
        h = self.n_sel_heads
        ws = self.qc_proj.weight if self.n_groups == 1 else self.se_proj.weight
        if h <= 1 or (self._autocast_dtype() or ws.dtype) != torch.bfloat16 or h % 8 == 0:
            return 1
        r = 8 // math.gcd(h, 8)
        if self._po_dim % (h * r):
            raise NotImplementedError("bf16 multi-head gating needs dim * expand to be a multiple of 8")
        return r

    def _heads(self) -> int:
        """Gate heads as the CUDA path sees them (see ``_head_copies``)."""
        return self.n_sel_heads * self._head_copies() if self.n_sel_heads > 1 else self.n_sel_heads

    def _weights(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(P + S, D) projection weight and (S,) gate bias.  Grouped: the (P, D/g, 1) convolution weight is laid
        out as its block-diagonal (P, D) matrix (reference pom/pom.py:180-183, 203-205); gradients flow back
        through the copy to the blocks.  With a bias on the grouped projection the matrix is (P + S, D + 8)
        (see ``_tokens``); with repeated gate heads S = r * heads (see ``_head_copies``)."""
        r = self._head_copies()
        if self.n_groups == 1 and r == 1:
            return self.qc_proj.weight, self.se_bias
        P = self._po_dim
        if self.n_groups == 1:
            src = (self.qc_proj.weight, self.se_bias)
        else:
            src = tuple(t for t in (self.po_proj.weight, self.se_proj.weight, self.se_proj.bias, self.po_proj.bias)
                        if t is not None)
        # Without autograd the assembled tensors are kept per parameter version (in-place updates and .data swaps
        # change the key); with autograd they are rebuilt per call, which is once per version in a training loop.
        track = torch.is_grad_enabled() and any(t.requires_grad for t in src)
        # parameters made under torch.inference_mode() have no version counter: assembled on every call
        keep = not track and not any(t.is_inference() for t in src)
        key = tuple((t._version, t.data_ptr(), t.dtype, t.device) for t in src) + (r,) if keep else None
        if keep and self._grouped_cache is not None and self._grouped_cache[0] == key:
            return self._grouped_cache[1]
        if keep and torch.is_inference_mode_enabled():
            with torch.inference_mode(False), torch.no_grad():  # what is cached must stay usable by a later backward
                return self._weights()
        if self.n_groups == 1:
            w_po, ws, bias = self.qc_proj.weight[:P], self.qc_proj.weight[P:], self.se_bias
        else:
            g = self.n_groups
            w = self.po_proj.weight.squeeze(-1)
            w_po = torch.block_diag(*w.view(g, P // g, self.dim // g).unbind(0))
            ws, bias = self.se_proj.weight, self.se_proj.bias
        if r > 1:
            ws, bias = ws.repeat_interleave(r, dim=0), bias.repeat_interleave(r)
        w_qc = torch.cat([w_po, ws], dim=0)
        bp = None if self.n_groups == 1 else self.po_proj.bias
        if bp is not None:
            extra = w_qc.new_zeros(w_qc.shape[0], self._BIAS_COLS - 1)
            first = torch.cat([bp.to(w_qc.dtype), w_qc.new_zeros(ws.shape[0])])
            w_qc = torch.cat([w_qc, first[:, None], extra], dim=1)
        if keep:
            self._grouped_cache = (key, (w_qc, bias))
        return w_qc, bias

    def _has_bias_cols(self) -> bool:
        return self.n_groups > 1 and self.po_proj.bias is not None

    def _out_weight(self) -> torch.Tensor:
        """(D, P) output projection; with the bias channels, as many zero rows below it, so that the layer keeps
        one width on both sides (the extra outputs are 0 and ``_finish`` drops them)."""
        w = self._cast(self.ag_proj.weight)
        return torch.cat([w, w.new_zeros(self._BIAS_COLS, w.shape[1])], dim=0) if self._has_bias_cols() else w

    def _residual(self, r: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if r is None or not self._has_bias_cols():
            return r
        return torch.cat([r, r.new_zeros(*r.shape[:-1], self._BIAS_COLS)], dim=-1)

    def _finish(self, y: torch.Tensor) -> torch.Tensor:
        if self._has_bias_cols():
            y = y[..., :self.dim]
        return y if self.ag_proj.bias is None else y + self.ag_proj.bias.to(y.dtype)

    # ------------------------------------------------------------------ API
    @eager_only
    @on_tensor_device
    def forward(self, xq: torch.Tensor, xc: Optional[torch.Tensor] = None, mask=None,
                shard: Optional[SeqShard] = None, residual: Optional[torch.Tensor] = None,
                grad_peer=None) -> torch.Tensor:
        """xq (B, T, D) queries; xc (B, N, D) context (None: self-mixing); mask None, "causal", (B, N), (B, T, N) or ``BlockCausal(frame_len)`` (extension).

        ``shard`` (extension) declares that xq/xc are this rank's token slice of a longer sequence;
        ``residual`` (extension, bf16) is added to the output inside the output projection's epilogue;
        ``grad_peer`` (extension): a ``peer.PeerExchange`` over data-parallel replicas — the backward pass sums the
        parameter gradients over its ranks itself (bf16 on the wire), so no all-reduce is needed afterwards.
        """
        spec, m = self._spec(xq, xc, mask, shard)
        spec.grad_peer = grad_peer
        w_qc, se_bias = self._weights()
        xq, xc = self._tokens(self._cast(xq)), (None if spec.self_mixing else self._tokens(self._cast(xc)))
        y, _ = pom_layer(xq, xc, self._cast(w_qc), se_bias, self.po_coeff, self._out_weight(), m, None, spec,
                         self._residual(self._cast(residual)))
        return self._finish(y)

    @eager_only
    @on_tensor_device
    def state_forward(self, xq: torch.Tensor, xc: Optional[torch.Tensor] = None,
                      state: Optional[Dict[str, Any]] = None,
                      residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, Any]]:
        """Incremental forward with a running-mean state {'h': (B, 1, P) fp32, 'n': calls so far}.

        As in the reference (pom/pom.py:251-262) the counter advances by one per call, so every
        call weighs equally whatever its token count.  ``residual`` (extension, bf16): a (B, T, D) tensor added
        to the output inside the output projection's epilogue.
        """
        spec = LayerSpec(degree=self.order, self_mixing=(xc is None or xc is xq), want_state=True,
                         n_sel_heads=self._heads())
        h_past = None
        n_past = 0
        if state is not None:
            n_past = state["n"]
            h_past = state["h"]
            if not torch.is_tensor(h_past):  # after reset(): h == 0.0
                h_past = None if n_past == 0 else torch.full((xq.shape[0], 1, self._po_dim), float(h_past),
                                                             device=xq.device, dtype=torch.float32)
        if h_past is not None and n_past > 0:
            spec.n_past = float(n_past)
        else:
            h_past = None
        w_qc, se_bias = self._weights()
        xq, xc = self._tokens(self._cast(xq)), (None if spec.self_mixing else self._tokens(self._cast(xc)))
        y, h = pom_layer(xq, xc, self._cast(w_qc), se_bias, self.po_coeff, self._out_weight(), None, h_past, spec,
                         self._residual(self._cast(residual)))
        return self._finish(y), {"h": h, "n": n_past + 1}

    @eager_only
    @on_tensor_device
    @torch.no_grad()
    def ar_forward(self, xq: torch.Tensor, state: Dict[str, Any]) -> Tuple[torch.Tensor, Dict[str, Any]]:
        """Autoregressive forward exactly as the reference defines it (pom/pom.py:264-275): no activation,
        polynomial or aggregation — the gate of each token multiplies that token's raw projection — and the
        returned state holds that projection as 'h' and the advanced token count.  For a running aggregate over
        chunks use :meth:`state_forward`."""
        if not xq.is_cuda:
            raise RuntimeError("pom_b200 has no CPU path: move the module and its inputs to a CUDA device")
        xq = self._tokens(self._cast(xq))
        B, T, D = xq.shape
        w_qc, se_bias = self._weights()
        P, S = self._po_dim, se_bias.shape[0]
        hs = ops.gemm(xq.contiguous().view(B * T, D), self._cast(w_qc).contiguous()).view(B, T, P + S)
        hp, z = hs[..., :P], hs[..., P:]
        bias32 = _f32(se_bias.contiguous())
        if self.n_sel_heads > 1:
            s32 = _f32(ops.select_fwd(z, bias32, _ones(B, S, xq.device)))
            sh = ops.select_heads_fwd(s32, hp, xq.dtype)
        else:
            sh = ops.select_fwd(z, bias32, hp)
        y = ops.gemm(sh.view(B * T, P), self._cast(self.ag_proj.weight)).view(B, T, self.dim)
        return self._finish(y), {"max_len": state["max_len"], "h": hp, "n": state["n"] + T}

    def reset(self, state: Dict[str, Any]) -> Dict[str, Any]:
        state["h"] = 0.0
        state["n"] = 0
        return state
