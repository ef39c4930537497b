"""Token-causal layer on the fused path (bf16): running sums per 32-token group inside the context and
gate-backward epilogues, the scan over groups, and the gate epilogue that rebuilds the prefix means — against the
CPU oracle (linear-time causal mean), with and without rotary embedding, both GEMM kernels, ragged lengths."""
import pytest
import torch

from oracle import pom_oracle as O
from tests.helpers import BF16_TOL, assert_close, assert_status_clean, cuda_run, make_cuda_module, oracle_run

pytestmark = pytest.mark.gpu


def _case(B, N, D, K, E, seed, rope=None, side=None, bias_scale=0.3):
    params = O.init_params(D, K, E, seed=seed, coeff_scale=0.1)
    g = torch.Generator().manual_seed(seed + 1)
    params["se_bias"] = torch.randn(params["se_bias"].shape, generator=g) * bias_scale
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x = O.bf16_round(torch.randn(B, N, D, generator=g))
    gy = O.bf16_round(torch.randn(B, N, D, generator=g))
    cfg = dict(dim=D, degree=K, expand=E, heads=1)
    kw = {"mask": "causal"}
    if rope == "2d":
        cfg["rope"] = dict(two_d=True, max_h=side, max_w=side)
        kw["positions_hw"] = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    elif rope == "1d":
        cfg["rope"] = dict(two_d=False, max_seq_len=max(N, 32))
    return cfg, params, x, gy, kw


def _spy_operator_path(monkeypatch):
    """Counts calls of the stand-alone causal operator, to tell which path a layer call took."""
    from pom_b200 import ops

    calls = []
    fn = ops.poly_agg_fwd

    def wrapped(*a, **k):
        calls.append(1)
        return fn(*a, **k)

    monkeypatch.setattr(ops, "poly_agg_fwd", wrapped)
    return calls


@pytest.mark.parametrize("gemm_mode", [1, 2], ids=["one_cta", "cta_pair"])
@pytest.mark.parametrize("shape", [
    # B, N, D, K, E, rope, side
    (2, 320, 128, 3, 2, None, None),    # no rotation, degree 3, a partial last tile
    (3, 200, 96, 2, 2, "1d", None),     # 1-D rotary, ragged tokens (last group has 8 tokens)
    (1, 1024, 64, 2, 2, "2d", 32),      # 2-D rotary on a 32 x 32 grid
    (2, 24, 16, 4, 2, None, None),      # shorter than one group
], ids=["plain_k3", "rope1d_ragged", "rope2d", "tiny"])
def test_fused_causal_layer_against_oracle(shape, gemm_mode, monkeypatch):
    from pom_b200 import _abi

    B, N, D, K, E, rope, side = shape
    cfg, params, x, gy, kw = _case(B, N, D, K, E, seed=61, rope=rope, side=side)
    calls = _spy_operator_path(monkeypatch)
    want_y, want_g = oracle_run(cfg, params, x, None, kw, gy)
    assert _abi.lib().pom_set_gemm_mode(gemm_mode) == 0
    try:
        mod = make_cuda_module(cfg, params, torch.bfloat16)
        y, grads = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    finally:
        _abi.lib().pom_set_gemm_mode(0)
    assert_status_clean()
    assert not calls, "the layer left the fused token-causal path"
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


def test_fused_causal_long_sequence():
    """8192 tokens (256 groups, a scan over 8 segments of groups) against the linear-time oracle."""
    cfg, params, x, gy, kw = _case(1, 8192, 64, 2, 2, seed=62)
    want_y, want_g = oracle_run(cfg, params, x, None, kw, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


def test_fused_causal_cross_mixing():
    """Queries and context are different tensors of equal length."""
    B, N, D, K, E = 2, 160, 64, 2, 2
    cfg, params, x, gy, kw = _case(B, N, D, K, E, seed=63)
    xc = O.bf16_round(torch.randn(B, N, D, generator=torch.Generator().manual_seed(9)))
    want_y, want_g = oracle_run(cfg, params, x, xc, kw, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, xc, kw, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


@pytest.mark.parametrize("case", [
    # B, N, D, K, E, rope, side, mask
    (2, 320, 128, 3, 2, None, None, "causal"),
    (1, 1024, 64, 2, 2, "2d", 32, "causal"),
    (3, 200, 96, 2, 2, "1d", None, "causal"),
    (1, 1024, 64, 2, 2, "2d", 32, None),
    (3, 200, 96, 2, 2, "1d", None, None),
], ids=["causal_plain", "causal_rope2d", "causal_rope1d", "rope2d", "rope1d"])
def test_whole_layer_calls_equal_the_phase_calls(case, monkeypatch):
    """A layer without token sharding runs as two library calls (pom_layer_fwd / pom_layer_bwd); with sharding the
    host calls the phases one by one and puts the exchanges between them.  Both sequence the same kernels on the same
    buffers, so outputs and every gradient agree bit for bit — with rotary embedding, the token-causal mask, or both."""
    from pom_b200 import functional

    B, N, D, K, E, rope, side, mask = case
    cfg, params, x, gy, kw = _case(B, N, D, K, E, seed=64, rope=rope, side=side)
    kw["mask"] = mask
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    assert functional.WHOLE_LAYER_CALLS
    y1, g1 = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    monkeypatch.setattr(functional, "WHOLE_LAYER_CALLS", False)
    y2, g2 = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    assert_status_clean()
    assert torch.equal(y1, y2)
    for k in g1:
        assert torch.equal(g1[k], g2[k]), k


@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("shape", [(1, 1, 32), (2, 33, 100), (1, 2048, 2304), (3, 70, 8)])
def test_group_scan_matches_cumsum(shape, reverse):
    from pom_b200 import ops

    B, G, P = shape
    g = torch.Generator().manual_seed(3)
    sums = torch.randn(B, G, P, generator=g)
    carry = torch.randn(B, P, generator=g)
    ref = sums.double()
    if reverse:
        ref = ref.flip(1)
    excl = torch.cumsum(ref, 1) - ref + carry.double().view(B, 1, P)
    if reverse:
        excl = excl.flip(1)
    dev = sums.cuda()
    total = ops.group_scan(dev, carry.cuda(), reverse=reverse, want_total=True)
    torch.testing.assert_close(dev.cpu().double(), excl, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(total.cpu().double(), sums.double().sum(1), rtol=1e-5, atol=1e-4)
    dev2 = sums.cuda()
    ops.group_scan(dev2, None, reverse=reverse)
    torch.testing.assert_close(dev2.cpu().double(), excl - carry.double().view(B, 1, P), rtol=1e-5, atol=1e-4)
