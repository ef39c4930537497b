"""Pins the CPU oracle against vectors produced by the reference implementation itself
(tests/golden/make_golden.py).  Runs without a GPU."""
import pytest
import torch

from oracle import pom_oracle as O

TOL = 2e-5  # fp32 arithmetic in a different association order than the reference


def _oracle_from_case(case, requires_grad=True):
    cfg = case["cfg"]
    params = {}
    for k, v in case["params"].items():
        if k in ("qc_proj.weight", "se_bias", "po_coeff", "ag_proj.weight", "po_proj.weight", "se_proj.weight",
                 "se_proj.bias", "po_proj.bias", "ag_proj.bias"):
            params[k] = v.clone().requires_grad_(requires_grad)
    rope = None
    if "rope" in cfg:
        r = cfg["rope"]
        rope = O.RopeConfig(two_d=r["two_d"], max_seq_len=r.get("max_seq_len", 4096), max_h=r.get("max_h", 64),
                            max_w=r.get("max_w", 64))
    return O.OraclePoM(params, cfg["degree"], cfg["expand"], cfg["heads"], rope), params


MODULE_CASES = [
    "pom_none", "pom_causal", "pom_mask2d", "pom_mask3d", "pom_cross", "pom_cross_mask2d",
    "pom_heads4_none", "pom_heads4_causal", "pom_heads4_mask3d",
    "rope1d_none", "rope1d_causal", "rope1d_mask2d", "rope1d_positions", "rope1d_cross",
    "rope2d_none", "rope2d_causal", "rope2d_heads4_none", "rope1d_heads4_causal",
    "pom_groups2_none", "pom_groups2_causal", "pom_groups2_cross_mask2d", "pom_groups2_heads4_none",
    "pom_groups2_bias_none", "pom_groups2_bias_causal", "pom_groups2_bias_cross",
]


@pytest.mark.parametrize("name", MODULE_CASES)
def test_layer_matches_reference_vectors(golden, name):
    case = golden[name]
    model, params = _oracle_from_case(case)
    xq = case["xq"].clone().requires_grad_(True)
    xc = None if case["xc"] is None else case["xc"].clone().requires_grad_(True)
    y = model.forward(xq, xc, **case["kwargs"])
    n2, mx = O.rel_errors(y, case["y"])
    assert n2 < TOL and mx < TOL, (name, n2, mx)
    ins = [xq] + ([xc] if xc is not None else [])
    order = ["se_bias", "po_coeff", "qc_proj.weight", "ag_proj.weight"]
    if "po_proj.weight" in params:
        order = ["po_proj.weight", "se_proj.weight", "se_proj.bias", "po_coeff", "ag_proj.weight"]
    order += [k for k in ("po_proj.bias", "ag_proj.bias") if k in params]
    grads = torch.autograd.grad(y, ins + [params[k] for k in order], case["gy"])
    want = [case["grads"][f"d_in{i}"] for i in range(len(ins))] + [case["grads"]["d_" + k] for k in order]
    for g, w, label in zip(grads, want, [f"in{i}" for i in range(len(ins))] + order):
        n2, mx = O.rel_errors(g, w)
        assert n2 < 5 * TOL and mx < 5 * TOL, (name, label, n2, mx)


def test_state_forward_matches_reference_vectors(golden):
    case = golden["pom_state"]
    model, _ = _oracle_from_case(case, requires_grad=False)
    state = None
    for f, want in zip(case["frames"], case["ys"]):
        y, state = model.state_forward(f, f, state)
        n2, mx = O.rel_errors(y, want)
        assert n2 < TOL and mx < TOL
    assert state["n"] == case["n"] == 3  # the counter advances once per call, not per token
    n2, mx = O.rel_errors(state["h"], case["h"])
    assert n2 < TOL and mx < TOL


@pytest.mark.parametrize("name", ["pom_ar", "pom_ar_heads4"])
def test_ar_forward_matches_reference_vectors(golden, name):
    case = golden[name]
    model, _ = _oracle_from_case(case, requires_grad=False)
    y, st = model.ar_forward(case["xq"], {"max_len": case["max_len"], "h": 0.0, "n": case["n"] - case["xq"].shape[1]})
    assert st["n"] == case["n"] and st["max_len"] == case["max_len"]
    for got, want in ((y, case["y"]), (st["h"], case["h"])):
        n2, mx = O.rel_errors(got, want)
        assert n2 < TOL and mx < TOL, (name, n2, mx)


@pytest.mark.parametrize("k", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("kind", ["none", "causal"])
def test_operator_matches_reference_vectors(golden, k, kind):
    case = golden[f"op_{kind}_k{k}"]
    x = case["x"].clone().requires_grad_(True)
    c = case["coeff"].clone().requires_grad_(True)
    out = O.polynomial_aggregation(x, c, None if kind == "none" else "causal")
    assert torch.allclose(out, case["out"], atol=1e-6, rtol=1e-4)
    dx, dc = torch.autograd.grad(out, [x, c], case["g"])
    assert torch.allclose(dx, case["dx"], atol=1e-6, rtol=1e-4)
    assert torch.allclose(dc, case["dcoeff"], atol=1e-5, rtol=1e-4)


def test_reference_cpu_configuration_replayed_from_seeds(golden):
    """benchmark configuration 1: fp32, B=2, N=256, D=256, degree 2, expand 2, seed 0 weights and inputs."""
    from pom_b200.pom import PoM

    case = golden["cfg1_fp32"]
    torch.manual_seed(0)
    mod = PoM(256, 2, 2, 1, 1)  # same parameter creation order as the reference => same weights
    assert torch.equal(mod.qc_proj.weight[::64, ::32], case["w_qc_sample"])
    assert torch.equal(mod.po_coeff[::64], case["coeff_sample"])
    torch.manual_seed(0)
    x = torch.randn(2, 256, 256)
    params = {k: v.detach() for k, v in mod.state_dict().items()}
    y = O.OraclePoM(params, 2, 2).forward(x)
    n2, mx = O.rel_errors(y[:, ::8, ::8], case["y_sample"])
    assert n2 < TOL and mx < TOL, (n2, mx)
    assert abs(y.abs().mean().item() - case["y_abs_mean"]) < 1e-3 * case["y_abs_mean"]


def test_linear_time_causal_equals_triangular_product():
    torch.manual_seed(3)
    h = torch.randn(2, 37, 8, dtype=torch.float64)
    tri = torch.tril(torch.ones(37, 37, dtype=torch.float64)).unsqueeze(0).expand(2, -1, -1)
    assert torch.allclose(O.aggregate(h, "causal"), O.aggregate(h, tri), atol=1e-12)


def test_block_causal_equals_frame_loop_with_equal_frames():
    params = O.init_params(16, 2, 2, seed=5, coeff_scale=0.1, dtype=torch.float64)
    model = O.OraclePoM(params, 2, 2)
    torch.manual_seed(6)
    x = torch.randn(2, 24, 16, dtype=torch.float64)
    full = model.forward(x, mask=O.block_causal_mask(24, 6, 2, torch.float64))
    state, outs = None, []
    for i in range(4):
        f = x[:, i * 6:(i + 1) * 6]
        y, state = model.state_forward(f, f, state)
        outs.append(y)
    assert torch.allclose(full, torch.cat(outs, dim=1), atol=1e-10)


def test_sharded_causal_carry_matches_full_sequence():
    torch.manual_seed(8)
    h = torch.randn(1, 40, 6, dtype=torch.float64)
    full = O.aggregate(h, "causal")
    first = O.aggregate(h[:, :24], "causal")
    second = O.aggregate(h[:, 24:], "causal", token_offset=24, carry=h[:, :24].sum(1))
    assert torch.allclose(full, torch.cat([first, second], 1), atol=1e-12)


def test_invalid_mask_raises_value_error():
    with pytest.raises(ValueError):
        O.aggregate(torch.zeros(1, 2, 3), "diagonal")
