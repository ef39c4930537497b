"""pom_poly_agg_mean_noalloc: the aggregation entry point for hosts that may not allocate device
memory (fixed memory plans, allocator-free worker threads).  It must return exactly what the regular
pair pom_poly_agg_fwd + pom_reduce_partials returns, call after call, although it keeps its partial
sums in a workspace built into the library instead of a caller-provided buffer.

The file name sorts last on purpose: a run that stops at the first failure has then already executed
every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(x, coeff, row_weight=None, partial=None):
    from pom_b200 import _abi
    from pom_b200._abi import AggArgs, ptr

    B, N, P = x.shape
    a = AggArgs()
    a.x, a.coeff, a.row_weight, a.carry = ptr(x), ptr(coeff), ptr(row_weight), None
    a.partial, a.out, a.total = ptr(partial), None, None
    a.ldx, a.ld_out, a.token_offset = x.stride(1), 0, 0
    a.B, a.N, a.P, a.K = B, N, P, coeff.shape[1]
    a.dtype, a.causal = _abi.dtype_code(x.dtype), 0
    a.rope.kind, a.rope.pos_stride = _abi.ROPE_NONE, 1
    return a


def _regular(x, coeff, row_weight, denom, scale):
    from pom_b200 import _abi
    from pom_b200._abi import ptr

    L = _abi.lib()
    B, N, P = x.shape
    chunks = L.pom_agg_chunks(N)
    partial = torch.empty(B, chunks, P, device="cuda")
    out = torch.empty(B, P, device="cuda")
    a = _args(x, coeff, row_weight, partial)
    assert L.pom_poly_agg_fwd(C.byref(a), _abi.stream_ptr()) == 0
    assert L.pom_reduce_partials(ptr(partial), ptr(out), ptr(denom), scale, B, chunks, P, _abi.stream_ptr()) == 0
    return out


def _noalloc(x, coeff, row_weight, denom, scale):
    from pom_b200 import _abi
    from pom_b200._abi import ptr

    out = torch.full((x.shape[0], x.shape[2]), float("nan"), device="cuda")
    a = _args(x, coeff, row_weight)
    rc = _abi.lib().pom_poly_agg_mean_noalloc(C.byref(a), ptr(denom), scale, ptr(out), _abi.stream_ptr())
    assert rc == 0, _abi.strerror(rc)
    return out


def test_two_calls_in_a_row_match_the_regular_entry_points():
    g = torch.Generator(device="cuda").manual_seed(0)
    # call 1: bf16, plain mean; call 2: fp32, other shape, key-padding weights - it reuses the workspace
    cases = [
        (torch.randn(4, 300, 256, device="cuda", generator=g).bfloat16() * 0.5, 2, False),
        (torch.randn(3, 130, 96, device="cuda", generator=g) * 0.5, 3, True),
    ]
    for x, K, masked in cases:
        B, N, P = x.shape
        coeff = torch.randn(P, K, device="cuda", generator=g) * 0.1
        w = denom = None
        scale = 1.0 / N
        if masked:
            w = (torch.rand(B, N, device="cuda", generator=g) < 0.5).float()
            w[:, 0] = 1.0
            denom = w.sum(1)
            scale = 1.0
        want = _regular(x, coeff, w, denom, scale)
        got = _noalloc(x, coeff, w, denom, scale)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert torch.equal(got, want), float((got - want).abs().max())
    # and once more with the first shape: stale partial sums of call 2 must not leak into the result
    x, K, _ = cases[0]
    coeff = torch.randn(x.shape[2], K, device="cuda", generator=g) * 0.1
    assert torch.equal(_noalloc(x, coeff, None, None, 1.0 / x.shape[1]), _regular(x, coeff, None, None, 1.0 / x.shape[1]))


def test_oversize_request_is_refused_without_running():
    from pom_b200 import _abi
    from pom_b200._abi import ptr

    x = torch.zeros(1, 8, 64, device="cuda")
    coeff = torch.zeros(64, 2, device="cuda")
    out = torch.full((1, 64), 7.0, device="cuda")
    a = _args(x, coeff)
    a.B, a.N, a.P = 64, 8192, 2048          # 64 * 128 chunks * 2048 channels = 16 Mi floats > 4 Mi
    rc = _abi.lib().pom_poly_agg_mean_noalloc(C.byref(a), None, 1.0, ptr(out), _abi.stream_ptr())
    assert rc == -9 and "range" in _abi.strerror(rc)
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0
