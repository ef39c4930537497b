"""Oracle parity at the channel widths of the benchmark configurations, on cut-down batch and length:
key-padding masks at D = 1024 with degree 3, the block-causal layer stack at D = 1024 with expand 4, and
the 2-D rotary layer at D = 1152 (P = 2304), non-causal and token-causal."""
import pytest
import torch

from oracle import pom_oracle as O
from tests.helpers import BF16_TOL, assert_close, assert_status_clean, cuda_run, make_cuda_module, oracle_run

pytestmark = pytest.mark.gpu


def _rounded_case(B, N, D, K, E, seed, bias_scale=0.1):
    # a small gate bias keeps z + b away from the hardsigmoid's kinks at +-3: with millions of gate values a wide
    # bias leaves a few within one bf16 step of a kink, where the stored (rounded) z and the oracle's unrounded z
    # take different derivatives and a whole row of dX moves by one full term
    params = O.init_params(D, K, E, seed=seed, coeff_scale=0.1)
    g = torch.Generator().manual_seed(seed + 1)
    params["se_bias"] = torch.randn(params["se_bias"].shape, generator=g) * bias_scale
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x = O.bf16_round(torch.randn(B, N, D, generator=g))
    gy = O.bf16_round(torch.randn(B, N, D, generator=g))
    return dict(dim=D, degree=K, expand=E, heads=1), params, x, gy


def test_masked_configuration_width():
    """Configuration 3 at B = 2: D = 1024, degree 3, expand 2, N = 2048, valid lengths 256 and 2048; the padded
    rows of the short sample hold noise that must not reach the result."""
    B, N, D, K, E = 2, 2048, 1024, 3, 2
    cfg, params, x, gy = _rounded_case(B, N, D, K, E, seed=31)
    lengths = torch.tensor([256, 2048])
    mask = (torch.arange(N).view(1, N) < lengths.view(B, 1)).float()
    want_y, want_g = oracle_run(cfg, params, x, None, {"mask": mask}, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, {"mask": mask}, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")
    x2 = x.clone()
    x2[0, 256:] = O.bf16_round(torch.randn(N - 256, D, generator=torch.Generator().manual_seed(5)))
    y2, _ = cuda_run(mod, x2, None, {"mask": mask}, gy, torch.bfloat16)
    assert torch.equal(y[0, :256], y2[0, :256]), "noise in padded context rows changed valid outputs"


def test_video_stack_configuration_width():
    """Configuration 4 at B = 2: D = 1024, degree 2, expand 4 (P = 4096), two frames of 256 tokens, two layers of
    x += PoM.state_forward(x); x += W2 gelu(W1 x).  Per-layer bound: each mixer call against the oracle on the same
    (GPU-produced) input stays within the bf16 tolerance; the stack output accumulates two layers of it."""
    from pom_b200.stack import PoMStack

    B, F, L, D, K, E, layers = 2, 2, 256, 1024, 2, 4, 2
    torch.manual_seed(41)
    stack = PoMStack(D, K, E, layers)
    with torch.no_grad():
        for m in stack.mixers:
            m.po_coeff.copy_(torch.randn_like(m.po_coeff) * 0.1)
        for p in stack.parameters():
            p.copy_(O.bf16_round(p))
    x = O.bf16_round(torch.randn(B, F * L, D))
    oracles = [O.OraclePoM({k: v.detach().clone() for k, v in m.state_dict().items()}, K, E) for m in stack.mixers]
    states, outs = [None] * layers, []
    with torch.no_grad():
        for f in range(F):
            h = x[:, f * L:(f + 1) * L]
            for i in range(layers):
                y, states[i] = oracles[i].state_forward(h, None, states[i])
                h = h + y
                h = h + torch.nn.functional.gelu(h @ stack.ffn_in[i].weight.t()) @ stack.ffn_out[i].weight.t()
            outs.append(h)
    want = torch.cat(outs, 1)
    stack = stack.cuda()
    for p in stack.parameters():
        p.data = p.data.bfloat16()
    xg = x.cuda().bfloat16()
    got = stack(xg, L)
    assert_status_clean()
    assert_close(got, want, 2 * BF16_TOL, "stack output (two layers)")
    assert_close(stack.forward_single_pass(xg, L), want, 2 * BF16_TOL, "single-pass block-causal stack output")
    # one mixer call on its own: the per-layer error the stack bound is made of
    with torch.no_grad():
        y0, st = stack.mixers[0].state_forward(xg[:, :L])
        w0, _ = oracles[0].state_forward(x[:, :L], None, None)
    assert_close(y0, w0, BF16_TOL, "first mixer call")
    assert_close(st["h"], oracles[0].state_forward(x[:, :L], None, None)[1]["h"], BF16_TOL, "state after one frame")


@pytest.mark.parametrize("mask", [None, "causal"])
def test_long_sequence_configuration_width(mask):
    """Configuration 5 at N = 4096: D = 1152, degree 2, expand 2, 2-D rotary positions of a 64 x 64 grid."""
    side, D, K, E = 64, 1152, 2, 2
    N = side * side
    cfg, params, x, gy = _rounded_case(1, N, D, K, E, seed=51)
    cfg["rope"] = dict(two_d=True, max_h=side, max_w=side)
    kw = {"mask": mask, "positions_hw": torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)}
    want_y, want_g = oracle_run(cfg, params, x, None, kw, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, f"y mask={mask}")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k} mask={mask}")
