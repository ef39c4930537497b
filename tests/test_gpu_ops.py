"""GPU parity of the stand-alone operators, laid out like the reference's own operator tests
(test_triton_correctness.py, test_triton_masked_correctness.py, test_triton_rope_correctness.py):
seed 42 inputs scaled by 0.5, coefficients scaled by 0.1, seed 7 upstream gradient, seed 99 masks,
and the mixed criterion |a - b| <= atol + rtol * |b| with the reference's tolerances."""
import itertools

import pytest
import torch

from oracle import pom_oracle as O

pytestmark = pytest.mark.gpu

TOLS = {torch.float32: dict(atol=1e-4, rtol=1e-3), torch.bfloat16: dict(atol=1e-3, rtol=5e-3)}
ROPE_BF16 = dict(atol=1e-2, rtol=1e-2)


def _inputs(B, N, D, K, dtype):
    torch.manual_seed(42)
    x = (torch.randn(B, N, D) * 0.5).to(dtype)
    coeff = (torch.randn(D, K) * 0.1).to(dtype)
    return x, coeff


def _close(a, b, tol, what):
    a, b = a.float().cpu(), b.float().cpu()
    bad = (a - b).abs() > tol["atol"] + tol["rtol"] * b.abs()
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements off, max abs err {(a - b).abs().max():.3e}"


def _run_pair(x, coeff, k, mask, dtype, rope_ref=None, rope_spec=None, tol=None):
    """Oracle in fp32 on the dtype-rounded inputs vs the CUDA operator; forward, grad_x, grad_coeff."""
    from pom_b200 import polynomial_aggregation_

    tol = tol or TOLS[dtype]
    xr = x.float().clone().requires_grad_(True)
    cr = coeff.float().clone().requires_grad_(True)
    feat = O.poly_features(xr, cr)
    if rope_ref is not None:
        feat = rope_ref(feat)
    want = O.aggregate(feat, mask)
    torch.manual_seed(7)
    g = torch.randn_like(want).to(dtype).float()
    wdx, wdc = torch.autograd.grad(want, [xr, cr], g)

    xg = x.cuda().requires_grad_(True)
    cg = coeff.cuda().requires_grad_(True)
    mk = mask.cuda() if torch.is_tensor(mask) else mask
    got = polynomial_aggregation_(xg, cg, k, mk, rope=rope_spec)
    assert got.shape == want.shape and got.dtype == dtype
    gdx, gdc = torch.autograd.grad(got, [xg, cg], g.to(dtype).cuda())
    _close(got, want, tol, "forward")
    _close(gdx, wdx, tol, "grad_x")
    # coefficient gradients sum B*N terms; bf16 inputs leave ~1 ulp (0.4 %) on them
    ctol = tol if dtype == torch.float32 else dict(atol=tol["atol"] * 4, rtol=max(tol["rtol"], 1e-2))
    _close(gdc, wdc, ctol, "grad_coeff")


FP32_GRID = list(itertools.product([1, 4], [16, 64, 256, 1024], [32, 96, 512], [1, 2, 4, 16]))


@pytest.mark.parametrize("B,N,D,K", FP32_GRID)
@pytest.mark.parametrize("mask", [None, "causal"])
def test_poly_agg_fp32(B, N, D, K, mask):
    x, c = _inputs(B, N, D, K, torch.float32)
    _run_pair(x, c, K, mask, torch.float32)


@pytest.mark.parametrize("N,D,K", list(itertools.product([64, 512], [64, 128], [2, 4])))
@pytest.mark.parametrize("mask", [None, "causal"])
def test_poly_agg_bf16(N, D, K, mask):
    x, c = _inputs(2, N, D, K, torch.bfloat16)
    _run_pair(x, c, K, mask, torch.bfloat16)


@pytest.mark.parametrize("keep", [1.0, 0.5, 0.25])
@pytest.mark.parametrize("B,N,D,K", [(1, 16, 32, 1), (4, 64, 96, 3), (4, 256, 128, 8), (2, 1024, 512, 16), (4, 1000, 33, 2)])
def test_poly_agg_masked_fp32(B, N, D, K, keep):
    x, c = _inputs(B, N, D, K, torch.float32)
    torch.manual_seed(99)
    m = (torch.rand(B, N) < keep).float()
    m[:, 0] = 1.0
    _run_pair(x, c, K, m, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask", [None, "causal"])
@pytest.mark.parametrize("B,N,D,K", [(1, 16, 32, 1), (4, 64, 96, 2), (4, 256, 128, 4), (2, 1024, 512, 16)])
def test_poly_agg_rope_1d(B, N, D, K, mask, dtype):
    from pom_b200 import _abi
    from pom_b200.ops import RopeSpec

    x, c = _inputs(B, N, D, K, dtype)
    cos, sin = O.rope_tables_1d(D, N + 16)
    pos = torch.arange(N)
    spec = RopeSpec(_abi.ROPE_1D, cos.cuda(), sin.cuda(), pos.cuda())
    _run_pair(x, c, K, mask, dtype, rope_ref=lambda f: O.rope_apply_1d(f, pos, cos, sin), rope_spec=spec,
              tol=ROPE_BF16 if dtype == torch.bfloat16 else None)


@pytest.mark.parametrize("mask", [None, "causal"])
@pytest.mark.parametrize("B,side,D,K", [(2, 4, 32, 2), (2, 16, 96, 3), (1, 32, 128, 4)])
def test_poly_agg_rope_2d(B, side, D, K, mask):
    """The reference has no fused 2-D kernel; its PyTorch path (pom_rope.py:208-235) is the oracle."""
    from pom_b200 import _abi
    from pom_b200.ops import RopeSpec

    N = side * side
    x, c = _inputs(B, N, D, K, torch.float32)
    rc, rs, cc, cs = O.rope_tables_2d(D, side, side)
    hw = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    spec = RopeSpec(_abi.ROPE_2D, rc.cuda(), rs.cuda(), hw.cuda(), cc.cuda(), cs.cuda())
    _run_pair(x, c, K, mask, torch.float32, rope_ref=lambda f: O.rope_apply_2d(f, hw, rc, rs, cc, cs), rope_spec=spec)


@pytest.mark.parametrize("name", [f"op_{kind}_k{k}" for kind in ("none", "causal") for k in (1, 2, 4, 8, 16)])
def test_poly_agg_matches_reference_vectors(golden, name):
    """Directly against outputs the reference's polynomial_aggregation_ produced (D = 96 tail case)."""
    from pom_b200 import polynomial_aggregation_

    case = golden[name]
    x = case["x"].cuda().requires_grad_(True)
    c = case["coeff"].cuda().requires_grad_(True)
    out = polynomial_aggregation_(x, c, c.shape[1], None if "none" in name else "causal")
    dx, dc = torch.autograd.grad(out, [x, c], case["g"].cuda())
    tol = TOLS[torch.float32]
    _close(out, case["out"], tol, "forward")
    _close(dx, case["dx"], tol, "grad_x")
    _close(dc, case["dcoeff"], tol, "grad_coeff")


def test_strided_input_view_is_consumed_without_copy_errors():
    """The reference feeds the operator a strided slice of the projection output (pom.py:206)."""
    from pom_b200 import polynomial_aggregation_

    torch.manual_seed(1)
    full = torch.randn(2, 40, 128) * 0.5
    coeff = torch.randn(64, 2) * 0.1
    want = O.polynomial_aggregation(full[..., :64], coeff)
    got = polynomial_aggregation_(full.cuda()[..., :64], coeff.cuda(), 2)
    _close(got, want, TOLS[torch.float32], "forward")


@pytest.mark.parametrize("per_token", [False, True])
def test_selection_operator(per_token):
    from pom_b200 import polynomial_selection_

    torch.manual_seed(2)
    s = torch.rand(2, 20, 48)
    h = torch.randn(2, 20 if per_token else 1, 48)
    sr, hr = s.clone().requires_grad_(True), h.clone().requires_grad_(True)
    want = O.selection(sr, hr, 1)
    g = torch.randn_like(want)
    wds, wdh = torch.autograd.grad(want, [sr, hr], g)
    sg, hg = s.cuda().requires_grad_(True), h.cuda().requires_grad_(True)
    got = polynomial_selection_(sg, hg, 1)
    gds, gdh = torch.autograd.grad(got, [sg, hg], g.cuda())
    tol = TOLS[torch.float32]
    _close(got, want, tol, "forward")
    _close(gds, wds, tol, "grad_s")
    _close(gdh, wdh, tol, "grad_h")


@pytest.mark.parametrize("per_token", [False, True])
def test_selection_operator_with_one_gate_value_per_head(per_token):
    """polynomial_selection_ with n_sel_heads > 1 (reference pom/pom.py:119-122): s is (B, T, heads)."""
    from pom_b200 import polynomial_selection_

    torch.manual_seed(3)
    heads = 4
    s = torch.rand(2, 20, heads)
    h = torch.randn(2, 20 if per_token else 1, 48)
    sr, hr = s.clone().requires_grad_(True), h.clone().requires_grad_(True)
    want = O.selection(sr, hr, heads)
    g = torch.randn_like(want)
    wds, wdh = torch.autograd.grad(want, [sr, hr], g)
    sg, hg = s.cuda().requires_grad_(True), h.cuda().requires_grad_(True)
    got = polynomial_selection_(sg, hg, heads)
    gds, gdh = torch.autograd.grad(got, [sg, hg], g.cuda())
    tol = TOLS[torch.float32]
    _close(got, want, tol, "forward")
    _close(gds, wds, tol, "grad_s")
    _close(gdh, wdh, tol, "grad_h")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_poly_agg_with_a_three_dimensional_mask(dtype):
    """(B, M, N) mask through the operator entry (reference pom/pom.py:41-45, 98-99): M query rows, each its own
    weighted mean over the N context tokens; M != N, half of the entries masked out, the diagonal kept."""
    B, M, N, D, K = 2, 24, 40, 64, 3
    x, coeff = _inputs(B, N, D, K, dtype)
    torch.manual_seed(99)
    mask = (torch.rand(B, M, N) < 0.5).float()
    mask[:, torch.arange(M), torch.arange(M)] = 1.0
    tol = TOLS[dtype] if dtype == torch.float32 else ROPE_BF16  # bf16: features and sums are rounded twice
    _run_pair(x, coeff, K, mask, dtype, tol=tol)
