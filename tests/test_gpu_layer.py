"""GPU parity of the whole layer (forward + every gradient) against the reference's own
vectors (fp32 mode) and against the CPU oracle on bf16-rounded inputs (bf16 mode)."""
import pytest
import torch

from oracle import pom_oracle as O
from tests.helpers import (BF16_TOL, FP32_TOL, PARAM_ORDER, param_order, assert_close, assert_status_clean, cuda_run,
                           make_cuda_module, oracle_run)

pytestmark = pytest.mark.gpu

LAYER_CASES = ["pom_none", "pom_causal", "pom_mask2d", "pom_mask3d", "pom_cross", "pom_cross_mask2d",
               "rope1d_none", "rope1d_causal", "rope1d_mask2d", "rope1d_positions", "rope1d_cross",
               "rope2d_none", "rope2d_causal"]


HEAD_CASES = ["pom_heads4_none", "pom_heads4_causal", "pom_heads4_mask3d", "rope2d_heads4_none", "rope1d_heads4_causal"]
GROUP_CASES = ["pom_groups2_none", "pom_groups2_causal", "pom_groups2_cross_mask2d", "pom_groups2_heads4_none",
               "pom_groups2_bias_none", "pom_groups2_bias_causal", "pom_groups2_bias_cross"]


@pytest.mark.parametrize("name", LAYER_CASES + HEAD_CASES + GROUP_CASES)
def test_fp32_layer_matches_reference_vectors(golden, name):
    case = golden[name]
    mod = make_cuda_module(case["cfg"], case["params"], torch.float32)
    y, grads = cuda_run(mod, case["xq"], case["xc"], case["kwargs"], case["gy"], torch.float32)
    assert_close(y, case["y"], FP32_TOL, f"{name} y")
    n_in = 1 if case["xc"] is None else 2
    for i in range(n_in):
        assert_close(grads[f"in{i}"], case["grads"][f"d_in{i}"], FP32_TOL, f"{name} d_in{i}")
    for k in param_order(case["params"]):
        assert_close(grads[k], case["grads"]["d_" + k], FP32_TOL, f"{name} d_{k}")


@pytest.mark.parametrize("name", ["pom_ar", "pom_ar_heads4"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ar_forward_matches_reference_vectors(golden, name, dtype):
    """ar_forward as the reference defines it (gate x raw projection per token, state = that projection)."""
    case = golden[name]
    params, x = case["params"], case["xq"]
    want_y, want_h = case["y"], case["h"]
    tol = FP32_TOL
    if dtype == torch.bfloat16:
        params = {k: O.bf16_round(v) for k, v in params.items()}
        x = O.bf16_round(x)
        model = O.OraclePoM(params, case["cfg"]["degree"], case["cfg"]["expand"], case["cfg"]["heads"])
        want_y, st = model.ar_forward(x, {"max_len": case["max_len"], "n": 0})
        want_h, tol = st["h"], BF16_TOL
    mod = make_cuda_module(case["cfg"], params, dtype)
    y, st = mod.ar_forward(x.cuda().to(dtype), {"max_len": case["max_len"], "h": 0.0, "n": case["n"] - x.shape[1]})
    assert st["n"] == case["n"] and st["max_len"] == case["max_len"]
    assert_close(y, want_y, tol, f"{name} y")
    assert_close(st["h"], want_h, tol, f"{name} state h")


@pytest.mark.parametrize("name", LAYER_CASES + ["pom_groups2_none", "pom_groups2_causal", "pom_groups2_bias_none",
                                                "pom_groups2_bias_causal", "pom_groups2_bias_cross",
                                                "pom_heads4_mask3d", "pom_heads4_causal"])
def test_bf16_layer_matches_oracle_on_rounded_inputs(golden, name):
    case = golden[name]
    cfg = case["cfg"]
    params = {k: O.bf16_round(case["params"][k]) for k in param_order(case["params"])}
    xq = O.bf16_round(case["xq"])
    xc = None if case["xc"] is None else O.bf16_round(case["xc"])
    gy = O.bf16_round(case["gy"])
    want_y, want_g = oracle_run(cfg, params, xq, xc, case["kwargs"], gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, xq, xc, case["kwargs"], gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, f"{name} y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"{name} d_{k}")


def _seeded_case(B, N, D, K, E, seed=0, coeff_scale=None, bias_scale=0.0):
    params = O.init_params(D, K, E, seed=seed, coeff_scale=coeff_scale)
    g = torch.Generator().manual_seed(seed + 1)
    if bias_scale:
        params["se_bias"] = torch.randn(params["se_bias"].shape, generator=g) * bias_scale
    x = torch.randn(B, N, D, generator=g)
    gy = torch.randn(B, N, D, generator=g)
    return dict(dim=D, degree=K, expand=E, heads=1), params, x, gy


def test_fp32_reference_cpu_configuration(golden):
    """benchmark configuration 1 (fp32, B=2, N=256, D=256, degree 2, expand 2, seed 0) on the GPU."""
    from pom_b200 import PoM

    case = golden["cfg1_fp32"]
    torch.manual_seed(0)
    mod = PoM(256, 2, 2, 1, 1)
    torch.manual_seed(0)
    x = torch.randn(2, 256, 256)
    y = mod.cuda()(x.cuda())
    assert_close(y[:, ::8, ::8], case["y_sample"], FP32_TOL, "cfg1 y sample")
    assert abs(y.abs().mean().item() - case["y_abs_mean"]) < 1e-3 * case["y_abs_mean"]


@pytest.mark.parametrize("coeff_scale", [None, 0.1])
@pytest.mark.parametrize("shape", [(2, 1024, 1152, 2, 2), (3, 200, 96, 3, 2), (2, 130, 64, 4, 1)])
def test_bf16_fused_path_against_oracle(shape, coeff_scale):
    """DiT-style no-mask layer (benchmark configuration 2 at reduced batch) and ragged shapes that leave partial
    tiles in every dimension; default (tiny) and O(1) polynomial coefficients."""
    B, N, D, K, E = shape
    cfg, params, x, gy = _seeded_case(B, N, D, K, E, coeff_scale=coeff_scale, bias_scale=0.5)
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x, gy = O.bf16_round(x), O.bf16_round(gy)
    want_y, want_g = oracle_run(cfg, params, x, None, {}, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, {}, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask", [None, "causal"])
@pytest.mark.parametrize("B,N,D,K,E", [(1, 1, 8, 1, 1), (3, 1, 64, 2, 2), (1, 2, 8, 3, 4), (5, 33, 16, 2, 1)])
def test_smallest_shapes(B, N, D, K, E, mask, dtype):
    """One token, one sample, eight channels: every tile is partial in every dimension."""
    cfg, params, x, gy = _seeded_case(B, N, D, K, E, seed=21, coeff_scale=0.1, bias_scale=0.5)
    tol = FP32_TOL
    if dtype == torch.bfloat16:
        params = {k: O.bf16_round(v) for k, v in params.items()}
        x, gy, tol = O.bf16_round(x), O.bf16_round(gy), BF16_TOL
    want_y, want_g = oracle_run(cfg, params, x, None, {"mask": mask}, gy)
    mod = make_cuda_module(cfg, params, dtype)
    y, grads = cuda_run(mod, x, None, {"mask": mask}, gy, dtype)
    assert_status_clean()
    assert_close(y, want_y, tol, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, tol, f"d_{k}")


@pytest.mark.parametrize("heads", [1, 4])
@pytest.mark.parametrize("N,T", [(37, 5), (3, 3), (9, 130), (130, 9)])
def test_bf16_ragged_full_masks(N, T, heads):
    """(B, T, N) masks whose row length is not a multiple of 8 elements (the mask operand's rows are padded to
    16-byte boundaries), with and without a multi-head gate."""
    B, D, K, E = 2, 64, 2, 2
    params = O.init_params(D, K, E, n_sel_heads=heads, seed=31, coeff_scale=0.1)
    params = {k: O.bf16_round(v) for k, v in params.items()}
    g = torch.Generator().manual_seed(32)
    xq, xc = O.bf16_round(torch.randn(B, T, D, generator=g)), O.bf16_round(torch.randn(B, N, D, generator=g))
    gy = O.bf16_round(torch.randn(B, T, D, generator=g))
    mask = ((torch.rand(B, T, N, generator=g) < 0.5).float() + torch.eye(T, N)).clamp(max=1.0)
    cfg = dict(dim=D, degree=K, expand=E, heads=heads)
    want_y, want_g = oracle_run(cfg, params, xq, xc, {"mask": mask}, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, xq, xc, {"mask": mask}, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


def test_bf16_widths_that_are_not_multiples_of_8_are_refused_with_a_reason():
    from pom_b200 import PoM

    mod = PoM(100, 2, 1).cuda().to(torch.bfloat16)
    with pytest.raises(NotImplementedError, match="multiples of 8"):
        mod(torch.randn(2, 16, 100, device="cuda", dtype=torch.bfloat16))
    y = PoM(100, 2, 1).cuda()(torch.randn(2, 16, 100, device="cuda"))  # float32 takes any width
    assert y.shape == (2, 16, 100)


def test_inference_mode_tensors_are_accepted():
    """Tensors made under torch.inference_mode() carry no version counter, which the per-parameter and
    per-position caches are keyed on: modules built, and positions made, inside such a block still work and give
    the results of ordinary tensors."""
    from pom_b200 import PoM, PoMRoPE

    torch.manual_seed(0)
    x = torch.randn(2, 64, 64, device="cuda").bfloat16()
    hw = torch.stack([torch.arange(64) // 8, torch.arange(64) % 8], 1).cuda()
    plain = PoM(64, 2, 2, n_groups=2).cuda().bfloat16()
    rope = PoMRoPE(64, 2, 2, rope_2d=True, max_h=8, max_w=8).cuda().bfloat16()
    want_plain, want_rope = plain(x), rope(x, positions_hw=hw)
    r1 = PoMRoPE(64, 2, 2, max_seq_len=64).cuda().bfloat16()
    with torch.inference_mode():
        inside = PoM(64, 2, 2, n_groups=2).cuda().bfloat16()
        inside.load_state_dict(plain.state_dict())
        assert torch.equal(inside(x), want_plain)
        inside.se_proj.bias.add_(1.0)  # an in-place update that no version counter records
        assert not torch.equal(inside(x), want_plain)
        assert torch.equal(rope(x, positions_hw=hw.clone()), want_rope)
        assert torch.equal(rope(x, positions_hw=hw), want_rope)
        y_in = r1(x)  # default positions first requested inside the block
    assert torch.equal(r1(x), y_in)
    # what the first call cached inside the block (fp32 copies of the coefficients, the assembled grouped
    # projection of a frozen module) must not poison a later training step
    xg = x.clone().requires_grad_(True)
    r1(xg).sum().backward()
    for p_ in plain.parameters():
        p_.requires_grad_(False)
    with torch.inference_mode():
        plain(x)
    plain(xg).sum().backward()
    assert bool(torch.isfinite(xg.grad).all())


def test_module_cast_after_first_use():
    """nn.Module.to / .float() swap the parameters' storage without touching their version counters: values the
    layer derived from them (fp32 copies of coefficients and bias) must follow."""
    from pom_b200 import PoM

    torch.manual_seed(0)
    mod = PoM(64, 2, 2).cuda().bfloat16()
    with torch.no_grad():
        mod.po_coeff.copy_(torch.randn_like(mod.po_coeff) * 0.1)
    x = torch.randn(2, 40, 64, device="cuda")
    y16 = mod(x.bfloat16())
    mod.float()
    y32 = mod(x)
    assert y32.dtype == torch.float32
    assert_close(y32, y16.float().cpu(), BF16_TOL, "fp32 after bf16")
    with torch.no_grad():
        mod.po_coeff.mul_(2.0)  # in-place update: version counter
    assert not torch.allclose(mod(x), y32)
    mod.po_coeff.data = mod.po_coeff.data / 2.0  # storage swap: no version change
    assert torch.allclose(mod(x), y32, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("mask", [None, "causal"])
@pytest.mark.parametrize("D,E,heads", [(16, 2, 8), (8, 1, 8), (24, 1, 3), (64, 2, 128)])
def test_bf16_gate_heads_of_a_few_channels(D, E, heads, mask):
    """Heads of 4, 1, 8 and 1 channels: too narrow for the batched tensor-core products of the collapsed form
    (rows of head_dim elements), so the explicit per-head selection runs."""
    params = O.init_params(D, 2, E, n_sel_heads=heads, seed=3, coeff_scale=0.1)
    params = {k: O.bf16_round(v) for k, v in params.items()}
    g = torch.Generator().manual_seed(4)
    x, gy = O.bf16_round(torch.randn(3, 20, D, generator=g)), O.bf16_round(torch.randn(3, 20, D, generator=g))
    cfg = dict(dim=D, degree=2, expand=E, heads=heads)
    want_y, want_g = oracle_run(cfg, params, x, None, {"mask": mask}, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, {"mask": mask}, gy, torch.bfloat16)
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask", [None, "causal", "block"])
def test_more_samples_than_one_library_call_takes(mask, dtype):
    """70 000 short sequences (windowed use): the sample index lives in a grid dimension of the operator kernels
    (65 535 at most), so the layer runs the samples in slices; every sample equals its own small-batch result."""
    from pom_b200 import BlockCausal, PoM

    torch.manual_seed(0)
    mod = PoM(8, 2, 2).cuda().to(dtype)
    B = 70000 if mask != "block" else 35000  # 2 frames per sample: 70 000 (sample, frame) rows
    x = torch.randn(B, 4, 8, device="cuda", dtype=dtype, requires_grad=True)
    m = BlockCausal(2) if mask == "block" else mask
    y = mod(x, mask=m)
    y.float().sum().backward()
    assert y.shape == (B, 4, 8) and bool(torch.isfinite(x.grad).all())
    for sl in (slice(0, 3), slice(B - 3, B)):
        assert torch.equal(y[sl], mod(x[sl], mask=m))


def test_torch_compile_runs_the_layer_as_it_is():
    """The library is called through ctypes, which a tracing compiler cannot follow: a compiled model takes a
    graph break around the layer and gets the eager result."""
    from pom_b200 import PoM

    torch.manual_seed(0)
    mod = PoM(64, 2, 2).cuda().bfloat16()
    x = torch.randn(2, 64, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    want = mod(x)
    got = torch.compile(mod)(x)
    assert torch.equal(got, want)
    got.float().sum().backward()
    assert bool(torch.isfinite(x.grad).all())


@pytest.mark.parametrize("kind", ["plain", "causal", "heads4", "rope1d", "grouped_bias"])
def test_bf16_autocast_with_fp32_master_weights(kind):
    """Under torch.autocast(bfloat16) the reference's Linear layers compute in bf16 from fp32 parameters.  The layer
    does the same: an fp32 module inside autocast equals a bf16 module holding the rounded weights, its output is
    bf16 and its parameter gradients arrive in fp32."""
    from pom_b200 import PoM, PoMRoPE

    torch.manual_seed(0)
    kw, mk = {}, {}
    if kind == "causal":
        kw["mask"] = "causal"
    if kind == "rope1d":
        make = lambda: PoMRoPE(64, 2, 2, max_seq_len=64)
    elif kind == "grouped_bias":
        make = lambda: PoM(64, 2, 2, n_groups=2, bias=True)
    else:
        make = lambda: PoM(64, 2, 2, n_sel_heads=4 if kind == "heads4" else 1)
    master = make().cuda()
    with torch.no_grad():
        master.po_coeff.copy_(torch.randn_like(master.po_coeff) * 0.1)
        for p_ in master.parameters():  # bf16-representable values, so that both modules hold the same numbers
            p_.copy_(p_.bfloat16().float())
    low = make().cuda()
    low.load_state_dict(master.state_dict())
    for p_ in low.parameters():
        p_.data = p_.data.bfloat16()
    x = torch.randn(2, 48, 64, device="cuda")
    xm = x.clone().requires_grad_(True)
    xl = x.bfloat16().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ym = master(xm, **kw)
    yl = low(xl, **kw)
    assert ym.dtype == torch.bfloat16 and torch.equal(ym, yl)
    g = torch.randn_like(yl)
    ym.backward(g)
    yl.backward(g)
    assert xm.grad.dtype == torch.float32 and torch.equal(xm.grad, xl.grad.float())
    for (n, pm), pl in zip(master.named_parameters(), low.parameters()):
        assert pm.grad.dtype == torch.float32, n
        assert_close(pm.grad, pl.grad.float().cpu(), 1e-2, f"d_{n}")  # fp32 accumulators rounded once to bf16 in `low`
    with torch.autocast("cuda", dtype=torch.bfloat16), torch.no_grad():
        assert torch.equal(master(x, **kw), yl)  # cached casts of the weights
        master.ag_proj.weight.mul_(2.0)
        assert not torch.equal(master(x, **kw), yl)


def test_a_small_model_trains_and_memory_stays_flat():
    """Two mixer blocks with fp32 master weights under bf16 autocast, AdamW, sequences of varying length: the loss of
    a simple regression (reproduce the running mean of the tokens) falls, and device memory does not creep."""
    import torch.nn as nn

    from pom_b200 import PoM

    torch.manual_seed(0)

    class Block(nn.Module):
        def __init__(self, d):
            super().__init__()
            self.norm, self.mix = nn.LayerNorm(d), PoM(d, 2, 2)

        def forward(self, x):
            return x + self.mix(self.norm(x), mask="causal").float()

    model = nn.Sequential(Block(64), Block(64)).cuda()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    losses, mem = [], []
    for it in range(120):
        n = 64 + 8 * (it % 5)
        x = torch.randn(8, n, 64, device="cuda")
        target = x.cumsum(1) / torch.arange(1, n + 1, device="cuda").view(1, n, 1)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = model(x)
        loss = (y - x - target).square().mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
        if it % 5 == 4:
            mem.append(torch.cuda.memory_allocated())
    assert_status_clean()
    first, last = sum(losses[:10]) / 10, sum(losses[-10:]) / 10
    assert last < 0.5 * first, (first, last)
    assert max(mem[4:]) <= mem[3], mem  # after the first rounds over the five lengths nothing grows


def test_empty_batch_gives_an_empty_result():
    """No sample, or no query token: the reference's PyTorch path returns an empty tensor; so does this one, and
    the backward pass gives the parameters zero gradients."""
    from pom_b200 import PoM

    mod = PoM(64, 2, 2).cuda().to(torch.bfloat16)
    x = torch.zeros(0, 16, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = mod(x)
    assert y.shape == (0, 16, 64)
    y.sum().backward()
    assert x.grad.shape == x.shape and float(mod.qc_proj.weight.grad.abs().max()) == 0.0
    y = mod(torch.zeros(2, 0, 64, device="cuda", dtype=torch.bfloat16), torch.randn(2, 8, 64, device="cuda").bfloat16())
    assert y.shape == (2, 0, 64)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_query_token_against_a_long_context(dtype):
    """Cross-mixing with T = 1 (a decode step reading a prefilled context) and with N = 1 (many queries, one
    context token)."""
    for T, N in ((1, 300), (300, 1)):
        cfg, params, xq, gy = _seeded_case(2, T, 64, 2, 2, seed=22, coeff_scale=0.1, bias_scale=0.5)
        xc = torch.randn(2, N, 64, generator=torch.Generator().manual_seed(23))
        tol = FP32_TOL
        if dtype == torch.bfloat16:
            params = {k: O.bf16_round(v) for k, v in params.items()}
            xq, xc, gy, tol = O.bf16_round(xq), O.bf16_round(xc), O.bf16_round(gy), BF16_TOL
        want_y, want_g = oracle_run(cfg, params, xq, xc, {}, gy)
        mod = make_cuda_module(cfg, params, dtype)
        y, grads = cuda_run(mod, xq, xc, {}, gy, dtype)
        assert_status_clean()
        assert_close(y, want_y, tol, f"T={T} N={N} y")
        for k, w in want_g.items():
            assert_close(grads[k], w, tol, f"T={T} N={N} d_{k}")


@pytest.mark.parametrize("mask", [None, "causal"])
@pytest.mark.parametrize("rope", [None, "1d", "2d"])
@pytest.mark.parametrize("heads", [16, 4, 12])
def test_bf16_multi_head_gating_against_oracle(mask, rope, heads):
    """n_sel_heads = 16 is the setting of the reference's own benchmark scripts (bench_attn_vs_pom.py:94-97);
    4 and 12 heads are not a multiple of 8 and run with repeated gate heads (``PoM._head_copies``)."""
    B, side, D, K, E = 2, 16, (96 if heads == 12 else 64), 2, 2
    N = side * side
    params = O.init_params(D, K, E, n_sel_heads=heads, seed=9, coeff_scale=0.1)
    g = torch.Generator().manual_seed(10)
    params["se_bias"] = torch.randn(heads, generator=g) * 0.5
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x = O.bf16_round(torch.randn(B, N, D, generator=g))
    gy = O.bf16_round(torch.randn(B, N, D, generator=g))
    cfg = dict(dim=D, degree=K, expand=E, heads=heads)
    kw = {"mask": mask}
    if rope == "1d":
        cfg["rope"] = dict(two_d=False, max_seq_len=N)
    elif rope == "2d":
        cfg["rope"] = dict(two_d=True, max_h=side, max_w=side)
        kw["positions_hw"] = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    want_y, want_g = oracle_run(cfg, params, x, None, kw, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cross", [False, True])
def test_block_causal_fast_path_matches_block_triangular_mask(dtype, cross):
    """``BlockCausal(L)`` (per-frame means + running mean over frames) against the oracle run with the explicit
    (B, N, N) block-lower-triangular mask: outputs and every gradient."""
    from pom_b200 import BlockCausal

    B, F, L, D, K, E = 2, 5, 48, 64, 3, 2
    N = F * L
    cfg, params, x, gy = _seeded_case(B, N, D, K, E, seed=13, coeff_scale=0.1, bias_scale=0.3)
    xc = torch.randn(B, N, D, generator=torch.Generator().manual_seed(14)) if cross else None
    if dtype == torch.bfloat16:
        params = {k: O.bf16_round(v) for k, v in params.items()}
        x, gy = O.bf16_round(x), O.bf16_round(gy)
        xc = O.bf16_round(xc) if cross else None
    tol = FP32_TOL if dtype == torch.float32 else BF16_TOL
    want_y, want_g = oracle_run(cfg, params, x, xc, {"mask": O.block_causal_mask(N, L, B)}, gy)
    mod = make_cuda_module(cfg, params, dtype)
    y, grads = cuda_run(mod, x, xc, {"mask": BlockCausal(L)}, gy, dtype)
    assert_close(y, want_y, tol, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, 2 * tol if dtype == torch.float32 else tol, f"d_{k}")


def test_block_causal_rejects_ragged_lengths():
    from pom_b200 import BlockCausal, PoM

    mod = PoM(64, 2, 2, 1, 1).cuda()
    with pytest.raises(ValueError):
        mod(torch.randn(1, 100, 64, device="cuda"), mask=BlockCausal(48))


@pytest.mark.parametrize("rope", [None, "2d"])
def test_block_causal_mask_equals_frame_loop(rope):
    """A (B, N, N) block-lower-triangular mask reproduces state_forward's frame loop when all frames have
    the same length (single layer); bf16, against the oracle with the same mask."""
    B, F, L, D, K, E = 2, 4, 64, 64, 2, 2
    N = F * L
    cfg, params, x, gy = _seeded_case(B, N, D, K, E, seed=12, coeff_scale=0.1, bias_scale=0.3)
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x, gy = O.bf16_round(x), O.bf16_round(gy)
    mask = O.block_causal_mask(N, L, B)
    kw = {"mask": mask}
    if rope:
        cfg = dict(cfg, rope=dict(two_d=True, max_h=16, max_w=16))
        kw["positions_hw"] = torch.stack([torch.arange(N) // 16, torch.arange(N) % 16], 1)
    want_y, want_g = oracle_run(cfg, params, x, None, kw, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")
    if not rope:
        state, outs = None, []
        with torch.no_grad():
            for f in range(F):
                yf, state = mod.state_forward(x[:, f * L:(f + 1) * L].cuda().bfloat16().contiguous(), None, state)
                outs.append(yf)
        assert_close(torch.cat(outs, 1), y, BF16_TOL, "frame loop vs block-causal mask")


def test_prefix_length_mask_with_empty_tiles_matches_oracle():
    """Key-padding by valid lengths: 128-token tiles that the mask empties are skipped by the context GEMM (their
    saved projection is never written), which must not change outputs or gradients.  The allocator is primed with
    NaNs so that any use of an unwritten row would show."""
    B, N, D, K, E = 3, 512, 64, 2, 2
    cfg, params, x, gy = _seeded_case(B, N, D, K, E, seed=21, coeff_scale=0.1, bias_scale=0.3)
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x, gy = O.bf16_round(x), O.bf16_round(gy)
    lengths = torch.tensor([100, 256, 512])
    mask = (torch.arange(N).view(1, N) < lengths.view(B, 1)).float()
    want_y, want_g = oracle_run(cfg, params, x, None, {"mask": mask}, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    junk = torch.full((32 << 20,), float("nan"), device="cuda", dtype=torch.bfloat16)
    del junk
    y, grads = cuda_run(mod, x, None, {"mask": mask}, gy, torch.bfloat16)
    assert_status_clean()
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert torch.isfinite(grads[k].float()).all(), k
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")


def test_bf16_masked_layer_ignores_padded_noise():
    """benchmark configuration 3 at reduced size: key-padding mask from per-sample lengths, noise in the padding."""
    B, N, D, K, E = 4, 512, 128, 3, 2
    cfg, params, x, gy = _seeded_case(B, N, D, K, E, seed=3, coeff_scale=0.1)
    params = {k: O.bf16_round(v) for k, v in params.items()}
    g = torch.Generator().manual_seed(3)
    lengths = torch.randint(64, N + 1, (B,), generator=g)
    mask = (torch.arange(N).view(1, N) < lengths.view(B, 1)).float()
    x, gy = O.bf16_round(x), O.bf16_round(gy)
    want_y, want_g = oracle_run(cfg, params, x, None, {"mask": mask}, gy)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y, grads = cuda_run(mod, x, None, {"mask": mask}, gy, torch.bfloat16)
    assert_close(y, want_y, BF16_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, BF16_TOL, f"d_{k}")
    # replacing the padded context rows by other noise must not change the valid outputs at all
    x2 = x.clone()
    pad = mask == 0
    x2[pad] = O.bf16_round(torch.randn(int(pad.sum()), D, generator=g))
    y2, _ = cuda_run(mod, x2, None, {"mask": mask}, gy, torch.bfloat16)
    valid = mask.bool().cuda()
    assert torch.equal(y[valid], y2[valid])


def test_all_masked_sample_aggregates_to_zero():
    """A sample whose mask has no valid token yields zeros (not NaN)."""
    cfg, params, x, gy = _seeded_case(2, 64, 32, 2, 2, seed=5, coeff_scale=0.1)
    mask = torch.ones(2, 64)
    mask[1] = 0
    mod = make_cuda_module(cfg, params, torch.float32)
    y = mod(x.cuda(), mask=mask.cuda())
    assert torch.isfinite(y).all()
    assert float(y[1].detach().abs().max()) == 0.0


def test_state_forward_matches_reference_vectors(golden):
    case = golden["pom_state"]
    mod = make_cuda_module(case["cfg"], case["params"], torch.float32)
    state = None
    for f, want in zip(case["frames"], case["ys"]):
        y, state = mod.state_forward(f.cuda(), None, state)
        assert_close(y, want, FP32_TOL, "state_forward y")
    assert state["n"] == case["n"]
    assert_close(state["h"], case["h"], FP32_TOL, "state h")


def test_block_causal_video_stack_frame_loop():
    """benchmark configuration 4 at reduced size: a residual stack of PoM + GELU FFN layers run frame by frame
    with state_forward equals the oracle's frame loop; bf16."""
    B, F, L, D, K, E, layers = 2, 4, 64, 64, 2, 4, 3
    g = torch.Generator().manual_seed(4)
    x = O.bf16_round(torch.randn(B, F * L, D, generator=g))
    stack = []
    for l in range(layers):
        p = {k: O.bf16_round(v) for k, v in O.init_params(D, K, E, seed=10 + l, coeff_scale=0.1).items()}
        w1 = O.bf16_round((torch.rand(4 * D, D, generator=g) * 2 - 1) / D ** 0.5)
        w2 = O.bf16_round((torch.rand(D, 4 * D, generator=g) * 2 - 1) / (4 * D) ** 0.5)
        stack.append((p, w1, w2))
    cfg = dict(dim=D, degree=K, expand=E, heads=1)

    def run(layer_fn, xin, to_dev):
        states = [None] * layers
        outs = []
        for f in range(F):
            h = to_dev(xin[:, f * L:(f + 1) * L])
            for l, (p, w1, w2) in enumerate(stack):
                y, states[l] = layer_fn(l, h, states[l])
                h = h + y
                h = h + torch.nn.functional.gelu(h @ to_dev(w1).t().to(h.dtype)) @ to_dev(w2).t().to(h.dtype)
            outs.append(h)
        return torch.cat(outs, 1)

    oracles = [O.OraclePoM(p, K, E) for p, _, _ in stack]
    want = run(lambda l, h, s: oracles[l].state_forward(h, None, s), x, lambda t: t.float())
    mods = [make_cuda_module(cfg, p, torch.bfloat16) for p, _, _ in stack]
    with torch.no_grad():
        got = run(lambda l, h, s: mods[l].state_forward(h, None, s), x, lambda t: t.cuda().bfloat16())
    assert_close(got, want, 3 * BF16_TOL, "video stack output")  # bf16 residual stream over 3 layers x 4 frames


def test_pom_stack_matches_oracle_frame_loop():
    """PoMStack (fused residual / GELU epilogues, state carried across frames) against the oracle's frame loop."""
    from pom_b200.stack import PoMStack

    B, F, L, D, K, E, layers = 2, 4, 64, 64, 2, 4, 3
    torch.manual_seed(11)
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
    got = stack(x.cuda().bfloat16(), L)
    assert_close(got, want, 3 * BF16_TOL, "stack output")  # bf16 residual stream over 3 layers x 4 frames
    one_pass = stack.forward_single_pass(x.cuda().bfloat16(), L)
    assert_close(one_pass, want, 3 * BF16_TOL, "single-pass block-causal stack output")
    assert_close(one_pass, got, 3 * BF16_TOL, "single pass vs frame loop")


def test_token_causal_long_sequence_against_linear_time_oracle():
    """Token-causal forward at a length where the reference's N x N mask would be impractical."""
    cfg, params, x, gy = _seeded_case(1, 8192, 64, 2, 2, seed=6, coeff_scale=0.1, bias_scale=0.3)
    want_y, want_g = oracle_run(cfg, params, x, None, {"mask": "causal"}, gy)
    mod = make_cuda_module(cfg, params, torch.float32)
    y, grads = cuda_run(mod, x, None, {"mask": "causal"}, gy, torch.float32)
    assert_close(y, want_y, FP32_TOL, "y")
    for k, w in want_g.items():
        assert_close(grads[k], w, 2 * FP32_TOL, f"d_{k}")


def test_rope2d_grid_bf16_against_oracle():
    """benchmark configuration 5 at reduced size: 2-D axial rotary positions on a 32 x 32 grid, non-causal and causal."""
    D, K, E, side = 64, 2, 2, 32
    N = side * side
    cfg, params, x, gy = _seeded_case(1, N, D, K, E, seed=7, coeff_scale=0.1)
    cfg = dict(cfg, rope=dict(two_d=True, max_h=side, max_w=side))
    params = {k: O.bf16_round(v) for k, v in params.items()}
    x, gy = O.bf16_round(x), O.bf16_round(gy)
    hw = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    for mask in (None, "causal"):
        kw = {"mask": mask, "positions_hw": hw}
        want_y, want_g = oracle_run(cfg, params, x, None, kw, gy)
        mod = make_cuda_module(cfg, params, torch.bfloat16)
        y, grads = cuda_run(mod, x, None, kw, gy, torch.bfloat16)
        assert_close(y, want_y, BF16_TOL, f"y mask={mask}")
        for k, w in want_g.items():
            assert_close(grads[k], w, BF16_TOL, f"d_{k} mask={mask}")


def test_results_are_bitwise_reproducible():
    cfg, params, x, gy = _seeded_case(2, 384, 128, 2, 2, seed=8, coeff_scale=0.1)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    y1, g1 = cuda_run(mod, x, None, {}, gy, torch.bfloat16)
    y2, g2 = cuda_run(mod, x, None, {}, gy, torch.bfloat16)
    assert torch.equal(y1, y2)
    for k in ("in0", "se_bias", "po_coeff"):
        assert torch.equal(g1[k], g2[k]), k


def test_full_size_dit_layer_properties():
    """benchmark configuration 2 at full size (B=32, N=1024, D=1152): size-independent properties.
    (1) permuting the tokens of a sample permutes its outputs (no-mask mixing is a set function);
    (2) the backward pass is linear in the upstream gradient."""
    B, N, D, K, E = 32, 1024, 1152, 2, 2
    cfg, params, _, _ = _seeded_case(1, 8, D, K, E, seed=0, coeff_scale=0.1)
    mod = make_cuda_module(cfg, params, torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(B, N, D, device="cuda", generator=gen).bfloat16()
    perm = torch.randperm(N, device="cuda", generator=gen)
    with torch.no_grad():
        y = mod(x)
        yp = mod(x[:, perm].contiguous())
    n2, mx = O.rel_errors(yp, y[:, perm])
    assert n2 < 5e-3 and mx < 2e-2, (n2, mx)  # only the summation order inside H changes
    g1 = torch.randn(B, N, D, device="cuda", generator=gen).bfloat16()
    g2 = torch.randn(B, N, D, device="cuda", generator=gen).bfloat16()
    xr = x.clone().requires_grad_(True)
    out = mod(xr)
    d1, = torch.autograd.grad(out, xr, g1, retain_graph=True)
    d2, = torch.autograd.grad(out, xr, g2, retain_graph=True)
    d12, = torch.autograd.grad(out, xr, (g1.float() + g2.float()).bfloat16())
    n2, mx = O.rel_errors(d12, d1.float() + d2.float())
    assert n2 < BF16_TOL, (n2, mx)
    assert_status_clean()


@pytest.mark.parametrize("kind", ["plain", "rope2d_causal"])
def test_tensors_beyond_two_billion_elements(kind):
    """16 sequences of 65 536 tokens at D = 1152: the projected tensors hold 2.4e9 elements, past 32-bit element
    indices.  Size-independent properties: samples are independent (each half of the batch reproduces its part
    of the output and of the input gradient bit for bit) and parameter gradients add up over the halves."""
    from pom_b200 import PoM, PoMRoPE

    B, N, D = 16, 65536, 1152
    if torch.cuda.mem_get_info()[0] < 60 << 30:
        pytest.skip("needs 60 GB of free device memory")
    torch.manual_seed(0)
    kw = {}
    if kind == "plain":
        mod = PoM(D, 2, 2).cuda()
    else:
        mod = PoMRoPE(D, 2, 2, rope_2d=True, max_h=256, max_w=256).cuda()
        kw = dict(mask="causal", positions_hw=torch.stack([torch.arange(N) // 256, torch.arange(N) % 256], 1).cuda())
    for p_ in mod.parameters():
        p_.data = p_.data.bfloat16()
    with torch.no_grad():
        mod.po_coeff.copy_(torch.randn_like(mod.po_coeff) * 0.1)
    x = torch.randn(B, N, D, device="cuda", dtype=torch.bfloat16)
    gy = torch.randn(B, N, D, device="cuda", dtype=torch.bfloat16)

    def step(xs, gs):
        xs = xs.clone().requires_grad_(True)
        y = mod(xs, **kw)
        y.backward(gs)
        grads = [p_.grad.float().clone() for p_ in mod.parameters()]
        for p_ in mod.parameters():
            p_.grad = None
        return y.detach(), xs.grad, grads

    y, dx, g = step(x, gy)
    assert_status_clean()
    assert bool(torch.isfinite(y).all()) and bool(torch.isfinite(dx).all())
    h = B // 2
    y0, dx0, g0 = step(x[:h], gy[:h])
    y1, dx1, g1 = step(x[h:], gy[h:])
    assert torch.equal(y[:h], y0) and torch.equal(y[h:], y1)
    assert torch.equal(dx[:h], dx0) and torch.equal(dx[h:], dx1)
    for a, b, c in zip(g, g0, g1):  # each gradient was rounded to bf16 once
        assert float((a - (b + c)).norm() / a.norm()) < 1e-2


def test_cpu_tensors_are_rejected_loudly():
    from pom_b200 import PoM

    with pytest.raises(RuntimeError, match="no CPU path"):
        PoM(16, 2, 2)(torch.randn(1, 4, 16))


def test_unsupported_mask_and_degree_raise_like_the_reference():
    from pom_b200 import PoM, polynomial_aggregation_

    mod = PoM(16, 2, 2).cuda()
    with pytest.raises(ValueError):
        mod(torch.randn(1, 4, 16, device="cuda"), mask="diagonal")
    with pytest.raises(NotImplementedError):
        polynomial_aggregation_(torch.randn(1, 4, 16, device="cuda"), torch.randn(16, 17, device="cuda"), 17)
