"""GPU parity of the operator entry points that carry the reference's own names (pom_b200/operators.py),
called the way the reference's operator tests call theirs (test_triton_correctness.py,
test_triton_masked_correctness.py, test_triton_rope_correctness.py): positional arguments in the reference's
order, seed 42 inputs scaled by 0.5, coefficients scaled by 0.1, seed 7 upstream gradient, and the mixed
criterion |a - b| <= atol + rtol * |b|.  The oracle is the CPU restatement in fp32 on the dtype-rounded inputs."""
import pytest
import torch

from oracle import pom_oracle as O

pytestmark = pytest.mark.gpu

TOLS = {torch.float32: dict(atol=1e-4, rtol=1e-3), torch.bfloat16: dict(atol=1e-2, rtol=1e-2)}


def _inputs(B, N, D, K, dtype):
    torch.manual_seed(42)
    x = (torch.randn(B, N, D) * 0.5).to(dtype)
    coeff = (torch.randn(D, K) * 0.1).to(dtype)
    return x, coeff


def _close(a, b, tol, what):
    a, b = a.float().cpu(), b.float().cpu()
    bad = (a - b).abs() > tol["atol"] + tol["rtol"] * b.abs()
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements off, max abs err {(a - b).abs().max():.3e}"


def _compare(fn_cuda, fn_oracle, tensors, dtype, grads_for=None, ctol=None):
    """Runs ``fn_oracle`` on fp32 CPU copies and ``fn_cuda`` on CUDA copies of ``tensors`` (those named in
    ``grads_for`` require gradients) and compares the output and every gradient."""
    grads_for = list(tensors) if grads_for is None else grads_for
    cpu = {k: v.float().clone().requires_grad_(k in grads_for) for k, v in tensors.items()}
    want = fn_oracle(**cpu)
    torch.manual_seed(7)
    g = torch.randn_like(want).to(dtype).float()
    wgrads = torch.autograd.grad(want, [cpu[k] for k in grads_for], g)
    dev = {k: v.cuda().requires_grad_(k in grads_for) for k, v in tensors.items()}
    got = fn_cuda(**dev)
    assert got.shape == want.shape and got.dtype == dtype
    ggrads = torch.autograd.grad(got, [dev[k] for k in grads_for], g.to(dtype).cuda())
    tol = TOLS[dtype]
    _close(got, want, tol, "forward")
    for k, a, b in zip(grads_for, ggrads, wgrads):
        t = tol
        if k == "coeff" and dtype == torch.bfloat16:  # sums B*N terms of bf16-rounded products
            t = dict(atol=tol["atol"] * 4, rtol=tol["rtol"])
        _close(a, b, ctol or t, f"grad_{k}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 64, 96), (1, 1000, 33), (3, 5, 7, 64), (17, 128)])
def test_pom_activation(shape, dtype):
    from pom_b200.operators import pom_activation

    if dtype == torch.bfloat16 and shape[-1] % 8:
        pytest.skip("bf16 rows are read 16 bytes at a time")
    torch.manual_seed(42)
    x = (torch.randn(*shape) * 4.0).to(dtype)  # reaches both clamps (-0.1 and 6)
    _compare(lambda x: pom_activation(x), lambda x: O.activation(x), {"x": x}, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,D,K", [(1, 16, 32, 1), (4, 64, 96, 3), (2, 1024, 512, 16)])
def test_poly_features(B, N, D, K, dtype):
    from pom_b200.operators import poly_features

    x, c = _inputs(B, N, D, K, dtype)
    _compare(lambda x, coeff: poly_features(x, coeff, K), lambda x, coeff: O.poly_features(x, coeff),
             {"x": x, "coeff": c}, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,D", [(1, 16, 32), (4, 100, 96), (2, 1024, 512)])
def test_apply_rope_1d(B, N, D, dtype):
    from pom_b200.operators import apply_rope_1d

    x, _ = _inputs(B, N, D, 1, dtype)
    cos, sin = O.rope_tables_1d(D, N + 40)
    torch.manual_seed(3)
    pos = torch.randint(0, N + 40, (N,))  # any positions, not only 0..N-1
    _compare(lambda x: apply_rope_1d(x, pos.cuda(), cos.cuda(), sin.cuda()),
             lambda x: O.rope_apply_1d(x, pos, cos, sin), {"x": x}, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,side,D", [(2, 4, 32), (2, 16, 96), (1, 32, 128)])
def test_apply_rope_2d(B, side, D, dtype):
    from pom_b200.pom_rope import apply_rope_2d  # where the reference defines it

    N = side * side
    x, _ = _inputs(B, N, D, 1, dtype)
    rc, rs, cc, cs = O.rope_tables_2d(D, side, side + 3)
    hw = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    _compare(lambda x: apply_rope_2d(x, hw.cuda(), rc.cuda(), rs.cuda(), cc.cuda(), cs.cuda()),
             lambda x: O.rope_apply_2d(x, hw, rc, rs, cc, cs), {"x": x}, dtype)


def test_apply_rope_rejects_positions_outside_the_table():
    from pom_b200.operators import apply_rope_1d

    x = torch.randn(1, 8, 16, device="cuda")
    cos, sin = O.rope_tables_1d(16, 8)
    with pytest.raises(IndexError):
        apply_rope_1d(x, torch.arange(1, 9).cuda(), cos.cuda(), sin.cuda())
    with pytest.raises(ValueError):
        apply_rope_1d(torch.randn(1, 8, 15, device="cuda"), torch.arange(8).cuda(), cos.cuda(), sin.cuda())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,D,K", [(1, 16, 32, 1), (4, 256, 96, 2), (2, 1024, 512, 4)])
def test_named_aggregations(B, N, D, K, dtype):
    """poly_agg_mean / _causal / _masked under the reference's names and argument order."""
    from pom_b200.operators import (TRITON_AVAILABLE, TRITON_CAUSAL_AVAILABLE, TRITON_MASKED_AVAILABLE,
                                    poly_agg_causal_triton, poly_agg_masked_triton, poly_agg_mean_triton)

    assert TRITON_AVAILABLE and TRITON_CAUSAL_AVAILABLE and TRITON_MASKED_AVAILABLE
    x, c = _inputs(B, N, D, K, dtype)
    torch.manual_seed(99)
    m = (torch.rand(B, N) < 0.5).float()
    m[:, 0] = 1.0
    t = {"x": x, "coeff": c}
    _compare(lambda x, coeff: poly_agg_mean_triton(x, coeff, K),
             lambda x, coeff: O.aggregate(O.poly_features(x, coeff), None), t, dtype)
    _compare(lambda x, coeff: poly_agg_causal_triton(x, coeff, K),
             lambda x, coeff: O.aggregate(O.poly_features(x, coeff), "causal"), t, dtype)
    _compare(lambda x, coeff: poly_agg_masked_triton(x, m.cuda(), coeff, K),
             lambda x, coeff: O.aggregate(O.poly_features(x, coeff), m), t, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("default_positions", [True, False])
@pytest.mark.parametrize("B,N,D,K", [(1, 16, 32, 1), (4, 64, 96, 2), (2, 1024, 512, 4)])
def test_named_rotary_aggregations(B, N, D, K, default_positions, dtype):
    """poly_agg_rope_mean_triton / poly_agg_rope_causal_triton(x, coeff, k, freqs_cos, freqs_sin, positions)."""
    from pom_b200.operators import TRITON_ROPE_AVAILABLE, poly_agg_rope_causal_triton, poly_agg_rope_mean_triton

    assert TRITON_ROPE_AVAILABLE
    x, c = _inputs(B, N, D, K, dtype)
    cos, sin = O.rope_tables_1d(D, N + 16)
    pos = torch.arange(N) if default_positions else torch.arange(N).flip(0) + 16
    arg = None if default_positions else pos.cuda()
    t = {"x": x, "coeff": c}
    for fn, mask in ((poly_agg_rope_mean_triton, None), (poly_agg_rope_causal_triton, "causal")):
        _compare(lambda x, coeff: fn(x, coeff, K, cos.cuda(), sin.cuda(), arg),
                 lambda x, coeff: O.aggregate(O.rope_apply_1d(O.poly_features(x, coeff), pos, cos, sin), mask),
                 t, dtype)


def test_degree_above_16_is_refused_like_the_reference():
    from pom_b200.operators import poly_agg_mean_triton

    x = torch.randn(1, 8, 16, device="cuda")
    with pytest.raises(NotImplementedError):
        poly_agg_mean_triton(x, torch.randn(16, 17, device="cuda"), 17)


@pytest.mark.parametrize("mask", [None, "causal"])
@pytest.mark.parametrize("heads", [1, 4])
def test_pom_function(mask, heads):
    """``pom(xq, xc, coeff, k, n_sel_heads, mask)`` imported from the package as in the reference
    (pom/__init__.py, pom/pom.py:125-135): aggregation of the context gated by the (already activated) queries."""
    from pom_b200 import pom

    torch.manual_seed(3)
    B, N, D, K = 2, 40, 32, 3
    s = torch.rand(B, N, heads if heads > 1 else D)
    xc, c = torch.randn(B, N, D) * 0.5, torch.randn(D, K) * 0.1
    _compare(lambda s, x, coeff: pom(s, x, coeff, K, heads, mask),
             lambda s, x, coeff: O.selection(s, O.aggregate(O.poly_features(x, coeff), mask), heads),
             {"s": s, "x": xc, "coeff": c}, torch.float32)


def test_operators_on_more_samples_than_one_library_call_takes():
    from pom_b200 import polynomial_aggregation_, polynomial_selection_
    from pom_b200.operators import apply_rope_1d, pom_activation

    torch.manual_seed(5)
    B = 70000
    x = torch.randn(B, 3, 16, device="cuda")
    c = torch.randn(16, 2, device="cuda") * 0.1
    cos, sin = (t.cuda() for t in O.rope_tables_1d(16, 8))
    pos = torch.arange(3, device="cuda")
    full = [pom_activation(x), apply_rope_1d(x, pos, cos, sin), polynomial_aggregation_(x, c, 2, None),
            polynomial_aggregation_(x, c, 2, "causal"), polynomial_selection_(torch.sigmoid(x), x[:, :1], 1)]
    sl = slice(B - 4, B)
    part = [pom_activation(x[sl]), apply_rope_1d(x[sl], pos, cos, sin), polynomial_aggregation_(x[sl], c, 2, None),
            polynomial_aggregation_(x[sl], c, 2, "causal"), polynomial_selection_(torch.sigmoid(x[sl]), x[sl, :1], 1)]
    for a, b in zip(full, part):
        assert a.shape[0] == B and torch.equal(a[sl], b)
