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


def test_rotary_case_matches_bit_for_bit_and_free_memory_does_not_move():
    """1-D rotary aggregation through the built-in workspace equals the caller-buffer pair bit for bit, and the
    device's free memory is the same before and after the calls: nothing was allocated on the way."""
    from pom_b200 import _abi
    from pom_b200._abi import ptr
    from pom_b200.pom_rope import precompute_freqs_1d

    g = torch.Generator(device="cuda").manual_seed(1)
    B, N, P, K = 2, 200, 128, 2
    x = torch.randn(B, N, P, device="cuda", generator=g).bfloat16() * 0.5
    coeff = torch.randn(P, K, device="cuda", generator=g) * 0.1
    cos, sin = (t.cuda().contiguous() for t in precompute_freqs_1d(P, N + 16))
    pos = torch.arange(N, device="cuda", dtype=torch.int64)

    def with_rope(a):
        a.rope.kind, a.rope.pos_stride = _abi.ROPE_1D, 1
        a.rope.cos0, a.rope.sin0, a.rope.pos = ptr(cos), ptr(sin), ptr(pos)
        a.rope.len0 = cos.shape[0]
        return a

    L = _abi.lib()
    chunks = L.pom_agg_chunks(N)
    partial = torch.empty(B, chunks, P, device="cuda")
    want = torch.empty(B, P, device="cuda")
    got = torch.full((B, P), float("nan"), device="cuda")
    a = with_rope(_args(x, coeff, None, partial))
    assert L.pom_poly_agg_fwd(C.byref(a), _abi.stream_ptr()) == 0
    assert L.pom_reduce_partials(ptr(partial), ptr(want), None, 1.0 / N, B, chunks, P, _abi.stream_ptr()) == 0
    b = with_rope(_args(x, coeff))
    assert L.pom_poly_agg_mean_noalloc(C.byref(b), None, 1.0 / N, ptr(got), _abi.stream_ptr()) == 0  # warm-up call
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert L.pom_poly_agg_mean_noalloc(C.byref(b), None, 1.0 / N, ptr(got), _abi.stream_ptr()) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "device memory moved during calls that must not allocate"
    assert torch.equal(got, want), float((got - want).abs().max())


def test_the_limit_is_exact():
    """B * chunks * P == 4 194 304 floats fills the built-in workspace and is accepted; one channel more is refused."""
    from pom_b200 import _abi
    from pom_b200._abi import ptr

    B, N, P = 64, 64 * 128, 512          # 64 samples x 128 chunks x 512 channels = 4 Mi floats exactly
    assert B * _abi.lib().pom_agg_chunks(N) * P == 4 * 1024 * 1024
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(B, N, P, device="cuda", generator=g).bfloat16() * 0.5
    coeff = torch.randn(P, 2, device="cuda", generator=g) * 0.1
    got = _noalloc(x, coeff, None, None, 1.0 / N)
    want = _regular(x, coeff, None, None, 1.0 / N)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    out = torch.full((B, P + 8), 7.0, device="cuda")
    a = _args(x, coeff)
    a.P = P + 8                          # 4 Mi floats + 8192: over the limit, refused before any launch
    rc = _abi.lib().pom_poly_agg_mean_noalloc(C.byref(a), None, 1.0, ptr(out), _abi.stream_ptr())
    assert rc == -9
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0
