"""Autograd-level PoM operators on top of the C ABI.

``pom_layer`` is the whole layer (projections, polynomial aggregation, gating, output
projection) as one ``torch.autograd.Function``; ``polynomial_aggregation_`` /
``polynomial_selection_`` / ``pom`` keep the reference's operator names and argument
order (reference pom/pom.py:52-135) for callers that hold pre-projected features.

Execution paths inside ``pom_layer`` (all CUDA, chosen from dtype / mask / rotary kind):

* fused     bf16, no rotary, mask None or (B, N): tcgen05 GEMMs whose epilogues do the
            activation, polynomial, token reduction and gating (pom_ctx_gemm, pom_gate_gemm,
            pom_gate_bwd_gemm);
* operator  everything else (causal, rotary, fp32): plain GEMMs (tcgen05 for bf16, SIMT for
            fp32) around the stand-alone aggregation / selection kernels.

Token sharding over several GPUs (``SeqShard``) inserts the only collectives: an all-reduce
of the (B, P) partial sums for non-causal masks, an all-gather of per-rank totals followed
by a local exclusive scan for the causal mask, and the mirrored exchanges in backward.
"""
from __future__ import annotations

import functools
import weakref
from dataclasses import dataclass
from typing import Any, Optional, Tuple, Union

import torch
import torch.distributed as dist

from . import _abi, ops
from .ops import RopeSpec


def eager_only(fn):
    """Keeps ``torch.compile`` out of ``fn``: the library is called through ctypes with raw pointers, which a tracing
    compiler can neither follow nor fake, so a compiled model runs these calls as they are (a graph break)."""
    disable = getattr(getattr(torch, "compiler", None), "disable", None)
    return disable(fn) if disable is not None else fn


def on_tensor_device(fn):
    """Runs ``fn`` with the device of its first CUDA tensor argument current: the library launches on the current
    device's current stream, so a tensor on another GPU than the current one (``x.to("cuda:1")`` without
    ``torch.cuda.set_device(1)``) must switch devices first, as PyTorch's own operators do."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        dev = next((a.device for a in args if torch.is_tensor(a) and a.is_cuda), None)
        if dev is None or dev.index == torch.cuda.current_device():
            return fn(*args, **kwargs)
        with torch.cuda.device(dev):
            return fn(*args, **kwargs)

    return wrapper


# True: a fused-path layer without token sharding is two library calls (pom_layer_fwd / pom_layer_bwd).  False:
# the same kernels are launched phase by phase from Python (what per-launch timing instrumentation hooks into).
WHOLE_LAYER_CALLS = True

# --------------------------------------------------------------------------- sharding description
@dataclass
class SeqShard:
    """This rank's slice of a token-sharded sequence.

    ``token_offset`` is the global index of the local token 0 and ``n_global`` the global
    context length.  ``group`` is a torch.distributed process group (None = default group).
    Ranks hold consecutive chunks in rank order.  ``peer`` (a :class:`pom_b200.peer.PeerExchange` built on
    the same group) moves the exchanges over NVLink peer memory instead of through torch.distributed, which
    makes a sharded step capturable into a CUDA graph.
    """
    token_offset: int
    n_global: int
    group: Any = None
    reduce_weight_grads: bool = True
    peer: Any = None
    overlap_grad_reduce: bool = True   # peer transport: all-reduce the parameter gradients on a side stream
    _side: Any = None

    def side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream()
        return self._side

    @property
    def world(self) -> int:
        return dist.get_world_size(self.group)

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group)

    def _use_peer(self, t: torch.Tensor, count: int) -> bool:
        return (self.peer is not None and t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()
                and count <= self.peer.slot_floats)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum over ranks (same bits on every rank on the peer path: fixed rank order)."""
        if self._use_peer(t, t.numel()):
            self.peer.exchange(t.view(1, 1, -1), out=t.view(1, -1))
            return t
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def sum_partials(self, partial: torch.Tensor, denom: Optional[torch.Tensor] = None, scale: float = 1.0):
        """(B, chunks, P) local partial sums -> (B, P) = scale · Σ_ranks Σ_chunks / denom."""
        B, chunks, P = partial.shape
        if self._use_peer(partial, B * P):
            if chunks > 128:  # one CTA walks the chunks serially: keep that short
                partial = ops.reduce_partials(partial).view(B, 1, P)
            return self.peer.exchange(partial, denom=denom, scale=scale)
        total = self.all_reduce(ops.reduce_partials(partial)).view(B, 1, P)
        return ops.reduce_partials(total, denom=denom, scale=scale)

    def reduce_grads(self, flat: torch.Tensor) -> torch.Tensor:
        """Sum of the flat parameter-gradient buffer over ranks, in place."""
        if self.peer is not None and self.peer.owns(flat):
            self.peer.allreduce_flat(flat.numel())
            return flat
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
        return flat

    def exclusive_carry(self, total: torch.Tensor, reverse: bool = False) -> torch.Tensor:
        """Sum of ``total`` over the ranks before (or, reversed, after) this one, in rank order."""
        if self._use_peer(total, total.numel()):
            mode = _abi.PEER_SUM_AFTER if reverse else _abi.PEER_SUM_BEFORE
            return self.peer.exchange(total.view(total.shape[0], 1, -1), mode=mode).view(total.shape)
        w = self.world
        flat = torch.empty((w * total.shape[0],) + tuple(total.shape[1:]), dtype=total.dtype, device=total.device)
        dist.all_gather_into_tensor(flat, total.contiguous(), group=self.group)
        gathered = flat.view((w,) + tuple(total.shape))
        r = self.rank
        part = gathered[r + 1:] if reverse else gathered[:r]
        if part.shape[0] == 0:
            return torch.zeros_like(total)
        if not total.is_cuda:  # host-side bookkeeping only (the layer itself never runs on CPU tensors)
            return part.sum(0)
        return ops.reduce_partials(part.transpose(0, 1).contiguous())


@dataclass(frozen=True)
class BlockCausal:
    """``mask=BlockCausal(frame_len)``: token m sees every token of its own and of earlier frames, all frames
    ``frame_len`` tokens long.  Same result as the (B, N, N) block-lower-triangular 0/1 mask (reference
    pom/pom.py:41-45, 98-99) and as one ``state_forward`` call per frame (pom/pom.py:251-259), computed in one
    pass: per-frame means, then a running mean over frames."""
    frame_len: int


@dataclass
class LayerSpec:
    """Non-tensor arguments of one layer call."""
    degree: int
    mask_kind: str = "none"          # "none" | "keypad" | "causal"
    self_mixing: bool = True
    rope_ctx: Optional[RopeSpec] = None
    rope_qry: Optional[RopeSpec] = None
    shard: Optional[SeqShard] = None
    n_past: Optional[float] = None   # state_forward: number of previous calls (None = plain forward)
    want_state: bool = False
    n_sel_heads: int = 1
    frames: int = 1                  # > 1: the batch rows are (sample, frame) pairs of a block-causal sequence
    # data-parallel replicas: a peer.PeerExchange over which the parameter gradients are summed inside the backward
    # pass (bf16 on the wire, straight from the fp32 accumulators; fused bf16 path only)
    grad_peer: Any = None


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None or t.dtype == torch.float32:
        return t
    return ops.to_f32(t)


_derived = {}


def _derived_of(t: torch.Tensor, what: str, make):
    """Value derived from tensor ``t`` (an fp32 copy of a small bf16 parameter, a transposed weight), remade only
    when ``t`` changes: keyed on the tensor object, its version counter and its storage, so an optimizer step or a move
    to another device invalidates it."""
    if t.is_inference():  # no version counter to tell an in-place update from no update: remake every time
        return make(t)
    key = (id(t), what)
    ent = _derived.get(key)
    stamp = (t._version, t.data_ptr(), t.device, t.dtype)  # .data swaps (Module.to, casts) keep the version
    if ent is not None and ent[0]() is t and ent[1] == stamp:
        return ent[2]
    with torch.inference_mode(False):  # a value cached under inference mode must stay usable by a later backward
        val = make(t)
    # the entry (and the memory of its value) goes when the tensor does
    _derived[key] = (weakref.ref(t, lambda _ref, k=key: _derived.pop(k, None)), stamp, val)
    return val


def _f32_cached(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.float32:
        return t.contiguous()
    return _derived_of(t, "f32", lambda x: ops.to_f32(x.contiguous()))


MAX_BATCH = 65535  # samples per library call: the operator kernels put the sample index in a grid dimension


def _batch_slices(n_samples: int, per_call: int = MAX_BATCH):
    """Slices that cut ``n_samples`` into runs of at most ``per_call`` (samples are independent of one another)."""
    per_call = max(1, per_call)
    return [slice(i, min(i + per_call, n_samples)) for i in range(0, n_samples, per_call)]


def _cut(t, sl):
    """``t[sl]`` for a per-sample tensor, ``t`` itself for anything shared by the samples (None, "causal", ...)."""
    return t[sl] if torch.is_tensor(t) else t


def _mask_operand(mask: torch.Tensor, device, dtype) -> torch.Tensor:
    """(B, T, N) mask as a GEMM operand: rows start on 16-byte boundaries (the row stride is N rounded up to 8
    elements; the columns past N are never read, the tensor map ends at N)."""
    B, T, N = mask.shape
    ld = (N + 7) // 8 * 8
    if ld == N:
        return mask.to(device=device, dtype=dtype).contiguous()
    buf = torch.zeros((B, T, ld), device=device, dtype=dtype)
    out = buf[..., :N]
    out.copy_(mask)
    return out


def _inv_rows(row_sums: torch.Tensor) -> torch.Tensor:
    """1 / row sum of a (B, T, N) mask, 0 where a row is empty (fp32)."""
    return torch.where(row_sums > 0, 1.0 / row_sums, torch.zeros_like(row_sums))


def _like_param(g: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    if p.dtype == torch.float32:
        return g
    return ops.to_bf16(g)


def _check_inputs(xq, xc, w_qc, w_ag, coeff, spec: LayerSpec):
    if xq.dim() != 3 or xc.dim() != 3:
        raise ValueError("expected (B, T, D) / (B, N, D) inputs")
    if xq.shape[0] != xc.shape[0]:
        raise ValueError(f"queries and context differ in batch size: {xq.shape[0]} vs {xc.shape[0]}")
    if xq.shape[2] != xc.shape[2]:
        raise ValueError(f"queries and context differ in feature size: {xq.shape[2]} vs {xc.shape[2]}")
    if spec.mask_kind == "causal" and xq.shape[1] != xc.shape[1]:
        # token m gates with the prefix aggregate of token m (reference pom/pom.py:115 asserts g == t)
        raise ValueError(f'mask="causal" needs as many query tokens as context tokens, got {xq.shape[1]} and '
                         f"{xc.shape[1]}")
    if coeff.shape[1] > 16:
        raise NotImplementedError(f"polynomial degree {coeff.shape[1]} > 16 is not implemented")
    if not xq.is_cuda:
        raise RuntimeError("pom_b200 has no CPU path: move the module and its inputs to a CUDA device")
    if xq.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"unsupported dtype {xq.dtype}; use bfloat16 or float32")
    for t in (xc, w_qc, w_ag):
        if t.dtype != xq.dtype:
            raise TypeError("inputs and projection weights must share one dtype")


class _PoMLayer(torch.autograd.Function):
    """y = ((R_q · hardsigmoid(xq·Wseᵀ + b)) ⊙ agg(R_c · poly(act(xc·Wpoᵀ)))) · Woᵀ
    (reference pom/pom.py:193-231 and pom/pom_rope.py:443-526).  With ``spec.n_sel_heads > 1`` the gate has one
    value per head (Wse is (heads, D)) and multiplies all channels of its head (pom/pom.py:119-122)."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, xq, xc, w_qc, se_bias, coeff, w_ag, mask, h_past, spec: LayerSpec, residual=None):
        _check_inputs(xq, xc, w_qc, w_ag, coeff, spec)
        B, T, D = xq.shape
        N = xc.shape[1]
        P, K = coeff.shape
        heads = spec.n_sel_heads if spec.n_sel_heads > 1 else 0
        S = heads if heads else P  # width of the gate projection
        bf16 = xq.dtype == torch.bfloat16
        if bf16 and (P % 8 or D % 8 or (heads and heads % 8)):
            # rows of every bf16 operand must start on 16-byte boundaries (bulk tensor copies)
            raise NotImplementedError(
                f"bfloat16 needs dim ({D}), dim * expand ({P}) and the number of gate heads to be multiples of 8; "
                "use float32 or pad the channels")
        xq = xq.contiguous()
        xc = xq if spec.self_mixing else xc.contiguous()
        w_qc = w_qc.contiguous()
        w_ag = w_ag.contiguous()
        w_po, w_se = w_qc[:P], w_qc[P:]
        coeff32, bias32 = _f32_cached(coeff), _f32_cached(se_bias)
        need_grad = any(ctx.needs_input_grad[:6]) or (h_past is not None and ctx.needs_input_grad[7])
        shard = spec.shard
        n_glob = shard.n_global if shard is not None else N
        offset = shard.token_offset if shard is not None else 0
        causal = spec.mask_kind == "causal"
        full = spec.mask_kind == "full"
        maskf = None
        denom = None
        maskd = rowden = None
        if full:
            if shard is not None or spec.n_past is not None:
                raise NotImplementedError("(B, M, N) masks are not combined with token sharding or state")
            if mask.dim() != 3 or mask.shape[0] != B or mask.shape[2] != N or mask.shape[1] != T:
                raise ValueError(f"expected a (B, T, N) = ({B}, {T}, {N}) mask, got {tuple(mask.shape)}")
            maskd = _mask_operand(mask, xq.device, xq.dtype)
            rowden = _row_sums(mask.to(device=xq.device, dtype=torch.float32).contiguous().view(B * T, N))
        if spec.mask_kind == "keypad":
            if tuple(mask.shape) != (B, N):
                raise ValueError(f"expected a (B, N) = ({B}, {N}) mask, got {tuple(mask.shape)}")
            maskf = mask.to(device=xq.device, dtype=torch.float32).contiguous()
            denom = ops.reduce_partials(maskf.view(B, N, 1)).view(B)
            if shard is not None:
                shard.all_reduce(denom)
        # rotary embedding rides in the GEMM epilogues when the positions of every aligned 32-token group are
        # constant or consecutive (RopeSpec.steps) and the degree is at most 4; otherwise on the operator path
        rotary = spec.rope_ctx is not None or spec.rope_qry is not None
        rope_ok = K <= 4 and all(r is None or r.fusable(P) for r in (spec.rope_ctx, spec.rope_qry))
        fused = (bf16 and not heads and (not rotary or rope_ok) and not causal and not full
                 and P % 8 == 0 and D % 8 == 0)
        # token-causal: the prefix means ride in the same epilogues (running sums per 32-token group + a scan over
        # the groups), with or without rotation
        two_d = any(r is not None and r.kind == _abi.ROPE_2D for r in (spec.rope_ctx, spec.rope_qry))
        fused_causal = (causal and bf16 and not heads and (not rotary or rope_ok) and K <= 4 and D % 8 == 0
                        and P % (64 if two_d else 16) == 0)

        hp = z = Hc = s32 = None
        collapsed = False
        ctx.collapsed = False
        ctx.fused_causal = fused_causal
        ctx.composite = (fused or fused_causal) and shard is None and WHOLE_LAYER_CALLS
        if spec.grad_peer is not None and need_grad:
            if not ctx.composite or {w_qc.dtype, w_ag.dtype, se_bias.dtype, coeff.dtype} != {torch.bfloat16}:
                raise NotImplementedError("grad_peer needs the fused bf16 path with bf16 parameters and no token shard")
            if spec.grad_peer.flat_buffer((3 * P * D + P + P * K + 7) // 8 * 8) is None:
                raise ValueError("the gradient region of grad_peer is smaller than this layer's parameters "
                                 f"({3 * P * D + P + P * K} floats)")
        if ctx.composite:
            # the whole fused layer is one library call (no exchange to put between its phases)
            if spec.frames > 1 and (spec.n_past is not None or maskf is not None):
                raise NotImplementedError("BlockCausal is not combined with masks or state")
            h_past32 = None
            if spec.n_past is not None and h_past is not None:
                h_past32 = _f32(h_past.reshape(B, P).contiguous())
            out = ops.layer_fwd(
                xq, None if spec.self_mixing else xc, w_qc, w_ag, bias32, coeff32, mask=maskf, h_past=h_past32,
                n_past=spec.n_past, residual=None if residual is None else residual.contiguous(), frames=spec.frames,
                save=need_grad, rope_c=spec.rope_ctx, rope_q=spec.rope_qry, causal=fused_causal, token_offset=offset)
            y, hp, z, sh, H, denom = out[:6]
            if fused_causal:
                h_past32 = out[6]  # the running sums `pre` travel in the slot that holds h_past otherwise
            ctx.has_residual = residual is not None
            ctx.spec = spec
            ctx.fused = True
            ctx.dims = (B, T, N, D, P, K, S, heads, n_glob, offset)
            ctx.h_past_dtype = None if h_past is None else h_past.dtype
            ctx.save_for_backward(xq, xc, w_qc, w_ag, coeff32, bias32, hp, z, H, h_past32, sh, maskf, denom, None, None,
                                  None)
            ctx.param_like = (w_qc, se_bias, coeff, w_ag)
            return (y, H.view(B, 1, P)) if spec.want_state else (y, None)
        # ---------------------------------------------------------------- context phase
        if fused_causal:
            carry, hp, Hc = ops.ctx_gemm(xc, w_po, coeff32, save_hp=need_grad, rope=spec.rope_ctx, causal=True)
            carry_in = None
            if shard is not None:  # totals of the ranks before this one
                carry_in = shard.exclusive_carry(ops.reduce_partials(carry))
            ops.group_scan(carry, carry_in)          # group totals -> exclusive carries, in place
            H = carry                                # saved in the slot of the aggregate; Hc holds `pre`
        elif fused:
            partial, hp = ops.ctx_gemm(xc, w_po, coeff32, row_weight=maskf, save_hp=need_grad,
                                       tile_weight=None if maskf is None else ops.tile_weights(maskf),
                                       rope=spec.rope_ctx)
            S_part = partial  # per-tile sums; reduced (and normalised, when no exchange is needed) below
        else:
            if spec.self_mixing:
                hs = ops.gemm(xq.view(B * T, D), w_qc).view(B, T, P + S)
                hp, z = hs[..., :P], hs[..., P:]
            else:
                hp = ops.gemm(xc.view(B * N, D), w_po).view(B, N, P)
                z = ops.gemm(xq.view(B * T, D), w_se).view(B, T, S)
            if not causal and not full:
                S_part = ops.poly_agg_fwd(hp, coeff32, row_weight=maskf, rope=spec.rope_ctx)  # per-chunk sums
        if fused_causal:
            pass
        elif causal:
            carry = None
            if shard is not None:
                S_loc = ops.reduce_partials(ops.poly_agg_fwd(hp, coeff32, rope=spec.rope_ctx))
                carry = shard.exclusive_carry(S_loc)
            Hc, _ = ops.poly_agg_fwd(hp, coeff32, causal=True, rope=spec.rope_ctx, carry=carry, token_offset=offset)
            H = None
        elif full:
            # H[b, m, :] = sum_n mask[b, m, n] * features[b, n, :] (divided by the row sum inside the selection)
            feat = ops.poly_agg_fwd(hp, coeff32, rope=spec.rope_ctx, per_token=True)
            Hc = torch.empty((B, T, P), dtype=xq.dtype, device=xq.device)
            if bf16:
                ops.gemm_batched(maskd, feat, b_mn=True, out=Hc)  # all samples in one strided-batched launch
            else:
                for b in range(B):
                    ops.gemm(maskd[b], feat[b], b_mn=True, out=Hc[b])
            H = None
        else:
            scale = 1.0 if denom is not None else 1.0 / n_glob
            if shard is not None:
                H = shard.sum_partials(S_part, denom=denom, scale=scale)
            else:
                H = ops.reduce_partials(S_part, denom=denom, scale=scale)
            if spec.frames > 1:
                H = ops.frame_prefix_mean(H, spec.frames)
            if spec.n_past is not None and h_past is not None:
                H = ops.state_merge(_f32(h_past.reshape(B, P).contiguous()), H, spec.n_past)

        # ---------------------------------------------------------------- query phase
        if fused_causal:
            sh, z = ops.gate_gemm(xq, w_se, bias32, None, save_z=need_grad, rope=spec.rope_qry,
                                  causal=(Hc, H, offset))
        elif fused:
            sh, z = ops.gate_gemm(xq, w_se, bias32, H, save_z=need_grad, rope=spec.rope_qry)
        elif heads:
            ones = _ones(B, heads, xq.device)
            s32 = _f32(ops.select_fwd(z, bias32, ones, rope=spec.rope_qry))   # gate in head space (B, T, heads)
            if full:  # the division by the mask's row sums rides on the (small) gate: s / rowsum, 0 for empty rows
                s32 = s32 * _inv_rows(rowden).view(B, T, 1)
            # one aggregate per sample: the P-wide gated state and its output GEMM collapse to a (heads x D)
            # matrix per sample (pom_heads_*); per-token aggregates (causal) keep the explicit form
            # (bf16: the batched tensor-core products of the collapsed form read rows of head_dim elements)
            collapsed = (not causal and not full and ops.heads_supported(heads, D, P)
                         and (not bf16 or (P // heads) % 8 == 0))
            if collapsed:
                sh = ops.heads_mix(H, w_ag, heads)  # Mb (B, heads, D), kept in the slot of the gated state
            else:
                sh = ops.select_heads_fwd(s32, Hc if (causal or full) else H, xq.dtype)
        else:
            sh = ops.select_fwd(z, bias32, Hc if (causal or full) else H, rope=spec.rope_qry, row_denom=rowden)
        if residual is not None and not bf16:
            raise NotImplementedError("the fused residual add of the output projection is a bf16 feature")
        if collapsed:
            y = ops.heads_out_fwd(s32, sh, xq.dtype, None if residual is None else residual.contiguous())
        else:
            y = ops.gemm(sh.view(B * T, P), w_ag,
                         residual=None if residual is None else residual.contiguous().view(B * T, D)).view(B, T, D)

        ctx.has_residual = residual is not None
        ctx.spec = spec
        ctx.fused = fused
        ctx.collapsed = collapsed
        ctx.dims = (B, T, N, D, P, K, S, heads, n_glob, offset)
        ctx.h_past_dtype = None if h_past is None else h_past.dtype
        ctx.save_for_backward(xq, xc, w_qc, w_ag, coeff32, bias32, hp, z, H, Hc, sh, maskf, denom, s32, maskd, rowden)
        ctx.param_like = (w_qc, se_bias, coeff, w_ag)
        if spec.want_state:
            return y, H.view(B, 1, P)
        return y, None

    @staticmethod
    @on_tensor_device
    def backward(ctx, dy, dh_state):
        spec: LayerSpec = ctx.spec
        xq, xc, w_qc, w_ag, coeff32, bias32, hp, z, H, Hc, sh, maskf, denom, s32, maskd, rowden = ctx.saved_tensors
        B, T, N, D, P, K, S, heads, n_glob, offset = ctx.dims
        p_qc, p_bias, p_coeff, p_ag = ctx.param_like
        shard = spec.shard
        causal = spec.mask_kind == "causal"
        full = spec.mask_kind == "full"
        dev = xq.device
        dt = xq.dtype
        dy = dy.contiguous()
        dy2 = dy.view(B * T, D)
        if ctx.composite:
            h_past32 = Hc  # slot reused by the composite forward
            dh32 = None if dh_state is None else _f32(dh_state.reshape(B, P).contiguous())
            w_t = None
            if ctx.fused_causal or spec.rope_qry is not None:  # these forms read the output weight transposed
                w_t = _derived_of(p_ag, "transposed", lambda w: ops.transpose_bf16(w.contiguous()))
            dxq, dxc, flat, d_hpast = ops.layer_bwd(
                dy, xq, None if spec.self_mixing else xc, w_qc, w_ag, bias32, coeff32, hp, z, sh, H, mask=maskf,
                denom=denom, h_past=None if ctx.fused_causal else h_past32, n_past=spec.n_past, dh_state=dh32,
                frames=spec.frames, want_d_hpast=bool(ctx.needs_input_grad[7]), rope_c=spec.rope_ctx,
                rope_q=spec.rope_qry, w_ag_t=w_t, causal=h_past32 if ctx.fused_causal else None,
                token_offset=ctx.dims[9],
                flat_out=None if spec.grad_peer is None else spec.grad_peer.flat_buffer(
                    (3 * P * D + P + P * K + 7) // 8 * 8))
            if d_hpast is not None:
                d_hpast = d_hpast.view(B, 1, P)
                if ctx.h_past_dtype != torch.float32:
                    d_hpast = ops.to_bf16(d_hpast)
            n_qc, n_ag = 2 * P * D, D * P
            if spec.grad_peer is not None:
                # summed over the replicas by the exchange's own kernel, which also does the rounding to bf16; the
                # result image is copied out because the next layer's backward pass reuses it
                f16 = ops.clone(spec.grad_peer.allreduce_flat_bf16(n_qc + n_ag + P + P * K))
            else:
                f16 = ops.to_bf16(flat)
            g_qc, g_ag = f16[:n_qc].view(2 * P, D), f16[n_qc:n_qc + n_ag].view(D, P)
            g_bias, g_coeff = f16[n_qc + n_ag:n_qc + n_ag + P], f16[n_qc + n_ag + P:].view(P, K)
            if p_bias.dtype == torch.float32:
                g_bias = flat[n_qc + n_ag:n_qc + n_ag + P]
            if p_coeff.dtype == torch.float32:
                g_coeff = flat[n_qc + n_ag + P:].view(P, K)
            return (dxq, dxc, g_qc, g_bias, g_coeff, g_ag, None, d_hpast, None, dy if ctx.has_residual else None)

        # one flat fp32 buffer for all parameter gradients: a single zero fill, cast and (when sharded) all-reduce
        n_qc, n_ag = (P + S) * D, D * P
        n_flat = n_qc + n_ag + S + P * K
        flat = None
        peer_flat = shard is not None and shard.reduce_weight_grads and shard.peer is not None
        if peer_flat:  # accumulate straight into the peer-mapped gradient region
            flat = shard.peer.flat_buffer((n_flat + 7) // 8 * 8)
        if flat is not None:
            ops.fill_zero(flat)
        else:
            peer_flat = False
            flat = ops.zeros_f32(n_flat, dev)
        d_wqc = flat[:n_qc].view(P + S, D)
        d_wag = flat[n_qc:n_qc + n_ag].view(D, P)
        d_bias = flat[n_qc + n_ag:n_qc + n_ag + S]
        d_coeff = flat[n_qc + n_ag + S:n_flat].view(P, K)
        # dWo[d, p] = sum_t dY[t, d] * SH[t, p]   (collapsed multi-head path: formed from dMb further down)
        if not ctx.collapsed:
            ops.gemm(dy2, sh.view(B * T, P), a_mn=True, b_mn=True, out=d_wag, accumulate=True)

        if spec.self_mixing:
            G = torch.empty((B * T, P + S), dtype=dt, device=dev)
            g_hp, g_z = G[:, :P], G[:, P:]
        else:
            g_hp = torch.empty((B * N, P), dtype=dt, device=dev)
            g_z = torch.empty((B * T, S), dtype=dt, device=dev)

        # ---------------------------------------------------------------- query phase backward
        dH_reduced = False  # True once dH already holds the sum over all ranks
        suf = carry_b = None
        if ctx.fused_causal:
            w_t = _derived_of(p_ag, "transposed", lambda w: ops.transpose_bf16(w.contiguous()))
            db_p, suf, carry_b = ops.gate_bwd_gemm(dy, w_ag, bias32, None, z, g_z, rope=spec.rope_qry, w_o_t=w_t,
                                                   causal=(Hc, H, offset))
            ops.reduce_partials(db_p.view(1, -1, P), out=d_bias.view(1, P))
            carry_in = None
            if shard is not None:  # totals of the ranks after this one
                carry_in = shard.exclusive_carry(ops.reduce_partials(carry_b), reverse=True)
            ops.group_scan(carry_b, carry_in, reverse=True)
        elif ctx.fused:
            w_t = None
            if spec.rope_qry is not None:  # the rotary form reads the output weight transposed: (P, D)
                w_t = _derived_of(p_ag, "transposed", lambda w: ops.transpose_bf16(w.contiguous()))
            dh_p, db_p = ops.gate_bwd_gemm(dy, w_ag, bias32, H, z, g_z, rope=spec.rope_qry, w_o_t=w_t)
            if shard is not None and dh_state is None and spec.frames == 1:
                dH = shard.sum_partials(dh_p)  # chunk sums, cross-rank sum and hand-back in one exchange
                dH_reduced = True
            else:
                dH = ops.reduce_partials(dh_p)
            ops.reduce_partials(db_p.view(1, -1, P), out=d_bias.view(1, P))
        elif ctx.collapsed:
            ds32, dMb = ops.heads_out_bwd(dy, s32, sh)          # sh holds Mb here
            dH = ops.heads_mix_bwd(dMb, H, w_ag, d_wag)         # also dWo
            ds = ds32 if dt == torch.float32 else ops.to_bf16(ds32)
            ops.select_bwd(ds, z, bias32, _ones(B, heads, dev), g_z.view(B, T, heads), rope=spec.rope_qry,
                           dbias_out=d_bias)
        else:
            dsh = ops.gemm(dy2, w_ag, b_mn=True).view(B, T, P)
            if heads:
                ds32 = ops.zeros_f32(B * T * heads, dev).view(B, T, heads)
                dH = ops.select_heads_bwd(dsh, s32, Hc if (causal or full) else H, ds32)
                if full:
                    ds32 = ds32 * _inv_rows(rowden).view(B, T, 1)
                ds = ds32 if dt == torch.float32 else ops.to_bf16(ds32)
                ops.select_bwd(ds, z, bias32, _ones(B, heads, dev), g_z.view(B, T, heads), rope=spec.rope_qry,
                               dbias_out=d_bias)
            else:
                dH, _ = ops.select_bwd(dsh, z, bias32, Hc if (causal or full) else H, g_z.view(B, T, P),
                                       rope=spec.rope_qry, dbias_out=d_bias, row_denom=rowden)

        # ---------------------------------------------------------------- context phase backward
        d_hpast = None
        if ctx.fused_causal:
            ops.poly_agg_bwd(hp, coeff32, dx_out=g_hp.view(B, N, P), rope=spec.rope_ctx, fused_causal=(suf, carry_b),
                             dcoeff_out=d_coeff)
        elif causal:
            carry = None
            if shard is not None:
                _, tot = ops.poly_agg_bwd(hp, coeff32, dx_out=g_hp.view(B, N, P), dout=dH, causal=True,
                                          rope=spec.rope_ctx, token_offset=offset, want_total=True, totals_only=True)
                carry = shard.exclusive_carry(tot, reverse=True)
            ops.poly_agg_bwd(hp, coeff32, dx_out=g_hp.view(B, N, P), dout=dH, causal=True, rope=spec.rope_ctx,
                             carry=carry, token_offset=offset, dcoeff_out=d_coeff)
        elif full:
            # d features[b] = mask[b]^T (N x T) · dH[b] (T x P)
            dfeat = torch.empty((B, N, P), dtype=dt, device=dev)
            if dt == torch.bfloat16:
                ops.gemm_batched(maskd, dH, a_mn=True, b_mn=True, out=dfeat)
            else:
                for b in range(B):
                    ops.gemm(maskd[b], dH[b], a_mn=True, b_mn=True, out=dfeat[b])
            ops.poly_agg_bwd(hp, coeff32, dx_out=g_hp.view(B, N, P), dout=dfeat, per_token=True, rope=spec.rope_ctx,
                             dcoeff_out=d_coeff)
        else:
            if dh_state is not None:
                dH = ops.reduce_partials(torch.stack([dH, _f32(dh_state.reshape(B, P).contiguous())], dim=1))
            if shard is not None and not dH_reduced:
                shard.all_reduce(dH)
            if spec.frames > 1:
                dH = ops.frame_prefix_mean(dH.contiguous(), spec.frames, adjoint=True)
            scale = 1.0 if denom is not None else 1.0 / n_glob
            if spec.n_past is not None and ctx.h_past_dtype is not None:
                # H = (n_past * h_past + h_cur) / (n_past + 1)
                if ctx.needs_input_grad[7]:
                    d_hpast = ops.reduce_partials(dH.view(B, 1, P), scale=spec.n_past / (spec.n_past + 1.0))
                    d_hpast = d_hpast.view(B, 1, P)
                    if ctx.h_past_dtype != torch.float32:
                        d_hpast = ops.to_bf16(d_hpast)
                scale = scale / (spec.n_past + 1.0)
            ops.poly_agg_bwd(hp, coeff32, dx_out=g_hp.view(B, N, P), dH=dH, row_weight=maskf, denom=denom,
                             scale=scale, rope=spec.rope_ctx, dcoeff_out=d_coeff)

        # ---------------------------------------------------------------- projections backward
        dts = {p_qc.dtype, p_bias.dtype, p_coeff.dtype, p_ag.dtype}
        overlap = peer_flat and shard.overlap_grad_reduce and dts == {torch.bfloat16}
        f16 = None
        # weight-gradient products first, so that (peer transport) their all-reduce over NVLink runs on a side stream
        # beside the data-gradient products.  The GEMM's CTAs fill the shared memory of the SMs they occupy, so the
        # all-reduce's CTAs run on the SMs the GEMM leaves idle (its last, partial wave) and otherwise right after
        # it; no rank can block another for longer than that, and every wait is bounded
        if spec.self_mixing:
            ops.gemm(G, xq.view(B * T, D), a_mn=True, b_mn=True, out=d_wqc, accumulate=True)
        else:
            ops.gemm(g_hp, xc.view(B * N, D), a_mn=True, b_mn=True, out=d_wqc[:P], accumulate=True)
            ops.gemm(g_z, xq.view(B * T, D), a_mn=True, b_mn=True, out=d_wqc[P:], accumulate=True)
        # all parameters bf16 and the peer transport: the gradients cross NVLink as bf16 (half the bytes; the result
        # image is copied out because the next backward pass reuses it)
        wire_bf16 = peer_flat and dts == {torch.bfloat16}
        if overlap:
            main, side = torch.cuda.current_stream(), shard.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                f16 = ops.clone(shard.peer.allreduce_flat_bf16(n_flat))
        if spec.self_mixing:
            dxq = ops.gemm(G, w_qc, b_mn=True).view(B, T, D)
            dxc = None
        else:
            dxc = ops.gemm(g_hp, w_qc[:P], b_mn=True).view(B, N, D)
            dxq = ops.gemm(g_z, w_qc[P:], b_mn=True).view(B, T, D)
        if overlap:
            main.wait_stream(side)
            f16.record_stream(main)
        elif wire_bf16 and shard.reduce_weight_grads:
            f16 = ops.clone(shard.peer.allreduce_flat_bf16(n_flat))
        elif shard is not None and shard.reduce_weight_grads:
            shard.reduce_grads(flat)
        if dts == {torch.bfloat16}:
            if f16 is None:
                f16 = ops.to_bf16(flat)
            g_qc, g_ag = f16[:n_qc].view(P + S, D), f16[n_qc:n_qc + n_ag].view(D, P)
            g_bias, g_coeff = f16[n_qc + n_ag:n_qc + n_ag + S], f16[n_qc + n_ag + S:].view(P, K)
        else:
            if peer_flat:  # the shared region is reused by the next call: hand out copies
                own = flat[:n_flat].clone()
                d_wqc, d_wag = own[:n_qc].view(P + S, D), own[n_qc:n_qc + n_ag].view(D, P)
                d_bias, d_coeff = own[n_qc + n_ag:n_qc + n_ag + S], own[n_qc + n_ag + S:].view(P, K)
            g_qc, g_ag = _like_param(d_wqc, p_qc), _like_param(d_wag, p_ag)
            g_bias, g_coeff = _like_param(d_bias, p_bias), _like_param(d_coeff, p_coeff)
        return (dxq, dxc, g_qc, g_bias, g_coeff, g_ag, None, d_hpast, None, dy if ctx.has_residual else None)


def _row_sums(m: torch.Tensor) -> torch.Tensor:
    """Row sums of a (rows, N) fp32 matrix through the partial-sum reduction kernel (grid-limited slices)."""
    rows, n = m.shape
    out = torch.empty((rows,), dtype=torch.float32, device=m.device)
    for lo in range(0, rows, 32768):
        hi = min(rows, lo + 32768)
        ops.reduce_partials(m[lo:hi].view(hi - lo, n, 1), out=out[lo:hi].view(hi - lo, 1))
    return out


_ones_cache = {}


def _ones(b: int, n: int, device) -> torch.Tensor:
    """(b, n) fp32 ones on ``device`` (identity 'state' used to run the gate kernels in head space)."""
    key = (b, n, str(device))
    if key not in _ones_cache:
        with torch.inference_mode(False):  # cached: must stay usable by a later backward pass
            _ones_cache[key] = torch.ones((b, n), dtype=torch.float32, device=device)
    return _ones_cache[key]


@eager_only
def pom_layer(xq, xc, w_qc, se_bias, coeff, w_ag, mask=None, h_past=None, spec: Optional[LayerSpec] = None,
              residual=None):
    """Whole layer; ``residual`` (B, T, D), bf16 only, is added to the output inside the output projection."""
    if xq.numel() == 0 and xq.dim() == 3 and xq.is_cuda:
        # no query token: an empty result that still belongs to the graph (the parameters receive zero gradients)
        zero = sum(t.sum() * 0 for t in (xq, w_qc, se_bias, coeff, w_ag))
        y = xq.new_zeros((xq.shape[0], xq.shape[1], w_ag.shape[0])) + zero.to(xq.dtype)
        return (y if residual is None else y + residual), None
    frames = spec.frames if spec is not None else 1
    if xq.dim() == 3 and xq.shape[0] * frames > MAX_BATCH and (spec is None or spec.shard is None):
        # more samples than one library call takes: the samples are independent, so run them in slices
        ys, hs = [], []
        for sl in _batch_slices(xq.shape[0], MAX_BATCH // frames):
            y, h = pom_layer(xq[sl], _cut(xc, sl), w_qc, se_bias, coeff, w_ag, _cut(mask, sl), _cut(h_past, sl), spec,
                             _cut(residual, sl))
            ys.append(y)
            hs.append(h)
        return torch.cat(ys, dim=0), (None if hs[0] is None else torch.cat(hs, dim=0))
    if spec is not None and spec.frames > 1:
        F = spec.frames
        B, T, D = xq.shape
        if (spec.rope_ctx is not None or spec.rope_qry is not None or spec.shard is not None or mask is not None
                or spec.want_state or spec.n_past is not None or spec.mask_kind != "none"):
            raise NotImplementedError("BlockCausal is not combined with rotary embedding, other masks, token sharding or state")
        if T % F or (xc is not None and xc.shape[1] != T):
            raise ValueError("BlockCausal needs equal query and context lengths, a multiple of frame_len")
        fold = lambda t: None if t is None else t.contiguous().view(B * F, T // F, t.shape[-1])
        y, h = _PoMLayer.apply(fold(xq), fold(xc) if xc is not None else fold(xq), w_qc, se_bias, coeff, w_ag, None,
                               None, spec, fold(residual))
        return y.view(B, T, -1), h
    y, h = _PoMLayer.apply(xq, xc if xc is not None else xq, w_qc, se_bias, coeff, w_ag, mask, h_past, spec, residual)
    return y, h


# --------------------------------------------------------------------------- reference-named operators
class _PolyAgg(torch.autograd.Function):
    """polynomial_aggregation_ for mask None / "causal" / (B, N), optional rotary embedding."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, x, coeff, mask_kind, mask, rope):
        if not x.is_cuda:
            raise RuntimeError("pom_b200 has no CPU path: pass CUDA tensors")
        B, N, P = x.shape
        if x.stride(-1) != 1 or (B > 1 and x.stride(0) != x.stride(1) * N):
            x = x.contiguous()
        coeff32 = _f32(coeff.contiguous())
        maskf = denom = None
        if mask_kind == "causal":
            out, _ = ops.poly_agg_fwd(x, coeff32, causal=True, rope=rope)
        else:
            if mask_kind == "keypad":
                maskf = mask.to(device=x.device, dtype=torch.float32).contiguous()
                denom = ops.reduce_partials(maskf.view(B, N, 1)).view(B)
            part = ops.poly_agg_fwd(x, coeff32, row_weight=maskf, rope=rope)
            h = ops.reduce_partials(part, denom=denom, scale=1.0 if denom is not None else 1.0 / N)
            out = h.view(B, 1, P)
            if x.dtype != torch.float32:
                out = ops.to_bf16(out)
        ctx.save_for_backward(x, coeff32, maskf, denom)
        ctx.meta = (mask_kind, rope, coeff.dtype)
        return out

    @staticmethod
    @on_tensor_device
    def backward(ctx, g):
        x, coeff32, maskf, denom = ctx.saved_tensors
        mask_kind, rope, cdt = ctx.meta
        B, N, P = x.shape
        dx = torch.empty((B, N, P), dtype=x.dtype, device=x.device)
        if mask_kind == "causal":
            g = g.contiguous()
            dc, _ = ops.poly_agg_bwd(x, coeff32, dx_out=dx, dout=g, causal=True, rope=rope)
        else:
            dH = _f32(g.reshape(B, P).contiguous())
            dc, _ = ops.poly_agg_bwd(x, coeff32, dx_out=dx, dH=dH, row_weight=maskf, denom=denom,
                                     scale=1.0 if denom is not None else 1.0 / N, rope=rope)
        dc = dc.contiguous()
        if cdt != torch.float32:
            dc = ops.to_bf16(dc)
        return dx, dc, None, None, None


class _PolyAggFull(torch.autograd.Function):
    """polynomial_aggregation_ with a (B, M, N) mask: out[b, m] = sum_n mask[b, m, n] poly[b, n] / sum_n mask[b, m, n]
    (reference pom/pom.py:41-45, 98-99).  Per-token features, one tensor-core product mask[b]·features[b] per sample,
    division by the row sums inside the selection kernel (whose gate is the constant 1 here)."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, x, coeff, mask, rope):
        if not x.is_cuda:
            raise RuntimeError("pom_b200 has no CPU path: pass CUDA tensors")
        B, N, P = x.shape
        if mask.dim() != 3 or mask.shape[0] != B or mask.shape[2] != N:
            raise ValueError(f"expected a (B, M, N) mask with B = {B}, N = {N}, got {tuple(mask.shape)}")
        M = mask.shape[1]
        if x.stride(-1) != 1 or (B > 1 and x.stride(0) != x.stride(1) * N):
            x = x.contiguous()
        coeff32 = _f32(coeff.contiguous())
        maskd = _mask_operand(mask, x.device, x.dtype)
        rowden = _row_sums(mask.to(device=x.device, dtype=torch.float32).contiguous().view(B * M, N))
        feat = ops.poly_agg_fwd(x, coeff32, rope=rope, per_token=True)
        Hc = torch.empty((B, M, P), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16:
            ops.gemm_batched(maskd, feat, b_mn=True, out=Hc)
        else:
            for b in range(B):
                ops.gemm(maskd[b], feat[b], b_mn=True, out=Hc[b])
        one = _ones(1, 1, x.device).to(x.dtype).expand(B, M, P).contiguous()
        ctx.save_for_backward(x, coeff32, maskd, rowden, Hc, one)
        ctx.meta = (rope, coeff.dtype)
        return ops.select_fwd(one, None, Hc, activated=True, row_denom=rowden)

    @staticmethod
    @on_tensor_device
    def backward(ctx, g):
        x, coeff32, maskd, rowden, Hc, one = ctx.saved_tensors
        rope, cdt = ctx.meta
        B, N, P = x.shape
        dH, _ = ops.select_bwd(g.contiguous(), one, None, Hc, torch.empty_like(one), activated=True, row_denom=rowden)
        dfeat = torch.empty((B, N, P), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16:
            ops.gemm_batched(maskd, dH, a_mn=True, b_mn=True, out=dfeat)
        else:
            for b in range(B):
                ops.gemm(maskd[b], dH[b], a_mn=True, b_mn=True, out=dfeat[b])
        dx = torch.empty((B, N, P), dtype=x.dtype, device=x.device)
        dc, _ = ops.poly_agg_bwd(x, coeff32, dx_out=dx, dout=dfeat, per_token=True, rope=rope)
        dc = dc.contiguous()
        if cdt != torch.float32:
            dc = ops.to_bf16(dc)
        return dx, dc, None, None


def _mask_kind(mask) -> str:
    if mask is None:
        return "none"
    if isinstance(mask, str):
        if mask == "causal":
            return "causal"
        raise ValueError('Unsupported mask: expected None, "causal", or a 2/3-D tensor.')
    if isinstance(mask, BlockCausal):
        return "block"
    if isinstance(mask, torch.Tensor):
        if mask.dim() == 2:
            return "keypad"
        if mask.dim() == 3:
            return "full"
    raise ValueError('Unsupported mask: expected None, "causal", or a 2/3-D tensor.')


@eager_only
def polynomial_aggregation_(x: torch.Tensor, coeff: torch.Tensor, k: int, mask=None,
                            rope: Optional[RopeSpec] = None) -> torch.Tensor:
    """Polynomial aggregation over the sequence dimension (reference pom/pom.py:52-100).

    x (B, N, P), coeff (P, K).  Returns (B, 1, P) for mask None or a (B, N) mask, (B, N, P) for "causal" and
    (B, M, P) for a (B, M, N) mask (a mask row of zeros gives 0 where the reference
    divides by zero).
    """
    if coeff.shape[1] != k:
        raise ValueError(f"coeff has {coeff.shape[1]} columns but k={k}")
    if k > 16:
        raise NotImplementedError(f"polynomial degree k={k} > 16 is not implemented")
    kind = _mask_kind(mask)
    if kind == "block":
        raise ValueError("BlockCausal is a layer-level mask (PoM.forward); pass a (B, M, N) tensor to the operator")
    if x.dim() == 3 and x.shape[0] > MAX_BATCH:
        return torch.cat([polynomial_aggregation_(x[sl], coeff, k, _cut(mask, sl), rope)
                          for sl in _batch_slices(x.shape[0])], dim=0)
    if kind == "full":
        if x.dtype == torch.bfloat16 and x.shape[-1] % 8:
            # the tensor-core product mask · features reads rows of P bf16 values, which must start on 16-byte
            # boundaries: other widths take the float32 form of the same operator
            return _PolyAggFull.apply(x.float(), coeff.float(), mask, rope).to(x.dtype)
        return _PolyAggFull.apply(x, coeff, mask, rope)
    return _PolyAgg.apply(x, coeff, kind, mask if kind == "keypad" else None, rope)


class _GateMul(torch.autograd.Function):
    """s ⊙ h with h broadcast over tokens (g == 1) or matched per token (g == t)."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, s, h):
        if not s.is_cuda:
            raise RuntimeError("pom_b200 has no CPU path: pass CUDA tensors")
        s = s.contiguous()
        b, g, p = h.shape
        per_tok = g != 1
        hk = h.to(s.dtype).contiguous() if per_tok else _f32(h.reshape(b, p).contiguous())
        ctx.save_for_backward(s, hk)
        ctx.meta = (per_tok, h.dtype, h.shape)
        return ops.select_fwd(s, None, hk, activated=True)

    @staticmethod
    @on_tensor_device
    def backward(ctx, g):
        s, hk = ctx.saved_tensors
        per_tok, hdt, hshape = ctx.meta
        ds = torch.empty_like(s)
        dh, _ = ops.select_bwd(g.contiguous(), s, None, hk, ds, activated=True)
        if not per_tok:
            dh = dh.view(hshape)
            if hdt != torch.float32:
                dh = ops.to_bf16(dh)
        return ds, dh


class _GateMulHeads(torch.autograd.Function):
    """s (B, T, heads) broadcast over the channels of each head, times h (per sample or per token)."""

    @staticmethod
    @on_tensor_device
    def forward(ctx, s, h):
        if not s.is_cuda:
            raise RuntimeError("pom_b200 has no CPU path: pass CUDA tensors")
        b, g, p = h.shape
        per_tok = g != 1
        s32 = _f32(s.contiguous())
        hk = h.contiguous() if per_tok else _f32(h.reshape(b, p).contiguous())
        ctx.save_for_backward(s32, hk)
        ctx.meta = (per_tok, s.dtype, h.dtype, h.shape)
        return ops.select_heads_fwd(s32, hk, h.dtype)

    @staticmethod
    @on_tensor_device
    def backward(ctx, g):
        s32, hk = ctx.saved_tensors
        per_tok, sdt, hdt, hshape = ctx.meta
        ds32 = ops.zeros_f32(s32.numel(), s32.device).view(s32.shape)
        dh = ops.select_heads_bwd(g.contiguous(), s32, hk, ds32)
        if not per_tok:
            dh = dh.view(hshape)
            if hdt != torch.float32:
                dh = ops.to_bf16(dh)
        return (ds32 if sdt == torch.float32 else ops.to_bf16(ds32)), dh


@eager_only
def polynomial_selection_(s: torch.Tensor, h: torch.Tensor, n_sel_heads: int) -> torch.Tensor:
    """Gated selection s ⊙ h (reference pom/pom.py:103-122): s already activated, (B, T, P) — or
    (B, T, n_sel_heads) with one gate value per head —, h (B, G, P) with G == 1 or G == T."""
    b, g, dh = h.shape
    t = s.shape[1]
    assert g == 1 or t == 1 or g == t, f"incompatible shapes: g={g} t={t}"
    if b > MAX_BATCH:
        return torch.cat([polynomial_selection_(s[sl], h[sl], n_sel_heads) for sl in _batch_slices(b)], dim=0)
    if n_sel_heads > 1:
        if s.shape[2] != n_sel_heads or dh % n_sel_heads:
            raise ValueError(f"expected a (B, T, {n_sel_heads}) gate and dim divisible by n_sel_heads")
        if t == 1 and g != 1:
            s = s.expand(b, g, n_sel_heads)
        return _GateMulHeads.apply(s, h)
    if t == 1 and g != 1:
        s = s.expand(b, g, dh)
    return _GateMul.apply(s, h)


def pom(xq, xc, coeff, k, n_sel_heads, mask=None):
    """Aggregate the context polynomially, gate with the query (reference pom/pom.py:125-135)."""
    h = polynomial_aggregation_(xc, coeff, k, mask)
    return polynomial_selection_(xq, h, n_sel_heads)
