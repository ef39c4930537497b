"""Seeded random configurations of the layer against the CPU oracle: batch, lengths (1..200, cross-mixing with
other query lengths), widths, degree, expansion, gate heads, mask kind (none, causal, (B, N), (B, T, N)), rotary
kind (none, 1-D with default or arbitrary positions, 2-D grids), bf16 and fp32.  Every combination the reference's
constructor accepts is fair game; output and every gradient are compared."""
import random

import pytest
import torch

from oracle import pom_oracle as O
from tests.helpers import BF16_TOL, FP32_TOL, cuda_run, make_cuda_module, oracle_run

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _draw(rng, case):
    dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float32])
    bf = dtype == torch.bfloat16
    B, K, E = rng.randint(1, 4), rng.randint(1, 5), rng.randint(1, 3)
    heads = rng.choice([1, 1, 2, 4, 8])
    rope = rng.choice([None, None, "1d", "2d"])
    D = 8 * rng.randint(1, 16) if bf else rng.choice([4, 8, 12, 20, 36, 64])
    side = rng.randint(1, 12)
    N = side * side if rope == "2d" else rng.randint(1, 200)
    P = D * E
    if heads > 1 and P % heads:  # the constraints of the reference's constructors (pom/pom.py:172, pom_rope.py:343-359)
        heads = 1
    if rope == "1d" and (P % 2 or (heads > 1 and (heads % 2 or P // heads < 2))):
        rope = None
    if rope == "2d" and (P % 4 or (heads > 1 and (heads % 4 or P // heads < 4))):
        rope = None
    cross = rng.random() < 0.3 and rope != "2d"
    T = rng.randint(1, 60) if cross else N
    mask_kind = rng.choice([None, "causal", "keypad", "full"])
    if mask_kind == "causal" and cross:
        mask_kind = None
    g = torch.Generator().manual_seed(1000 + case)
    cfg = dict(dim=D, degree=K, expand=E, heads=heads)
    kw = {}
    if rope == "1d":
        cfg["rope"] = dict(two_d=False, max_seq_len=max(N, T) + 4)
        if rng.random() < 0.5:
            kw["positions"] = torch.randint(0, max(N, T) + 4, (T,), generator=g)
            kw["ctx_positions"] = torch.randint(0, max(N, T) + 4, (N,), generator=g)
    if rope == "2d":
        cfg["rope"] = dict(two_d=True, max_h=side, max_w=side)
        kw["positions_hw"] = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    if mask_kind == "causal":
        kw["mask"] = "causal"
    elif mask_kind == "keypad":
        kw["mask"] = (torch.rand(B, N, generator=g) < 0.6).float()
        kw["mask"][:, 0] = 1
    elif mask_kind == "full":
        kw["mask"] = (torch.rand(B, T, N, generator=g) < 0.5).float()
        kw["mask"][:, :, 0] = 1
    params = O.init_params(D, K, E, n_sel_heads=heads, seed=case, coeff_scale=0.1)
    params["se_bias"] = torch.randn(params["se_bias"].shape, generator=g) * 0.5
    xq, gy = torch.randn(B, T, D, generator=g), torch.randn(B, T, D, generator=g)
    xc = torch.randn(B, N, D, generator=g) if cross else None
    if bf:
        params = {k: O.bf16_round(v) for k, v in params.items()}
        xq, gy = O.bf16_round(xq), O.bf16_round(gy)
        xc = None if xc is None else O.bf16_round(xc)
    desc = (f"#{case} {str(dtype)[6:]} B={B} T={T} N={N} D={D} K={K} E={E} heads={heads} rope={rope} "
            f"mask={mask_kind} cross={cross} positions={'positions' in kw}")
    return dtype, cfg, kw, params, xq, xc, gy, desc


@pytest.mark.parametrize("seed", [0, 1])
def test_random_configurations_against_the_oracle(seed):
    rng = random.Random(seed)
    failures = []
    for case in range(150):
        dtype, cfg, kw, params, xq, xc, gy, desc = _draw(rng, case)
        bf = dtype == torch.bfloat16
        want_y, want_g = oracle_run(cfg, params, xq, xc, kw, gy)
        y, grads = cuda_run(make_cuda_module(cfg, params, dtype), xq, xc, kw, gy, dtype)
        errs = {"y": _rel(y, want_y)}
        errs.update({k: _rel(grads[k], w) for k, w in want_g.items() if float(w.norm()) > 1e-6})
        for k, e in errs.items():
            tol = BF16_TOL if bf else FP32_TOL
            if bf and k == "se_bias":
                # a handful of numbers (one per gate head), each the sum over all tokens of terms of both signs:
                # when they cancel, the bf16 rounding of the terms weighs more against the result's norm
                tol = 3 * BF16_TOL
            if not e <= tol:
                failures.append(f"{desc}: {k} off by {e:.2e}")
        if not all(bool(torch.isfinite(v.float()).all()) for v in grads.values()):
            failures.append(f"{desc}: a gradient is not finite")
    assert not failures, "\n".join(failures)


def _operator_case(rng, case):
    """One random call of an operator-level function: returns (description, oracle closure, CUDA closure, inputs)."""
    from pom_b200 import operators as P
    from pom_b200 import polynomial_aggregation_, polynomial_selection_

    dtype = rng.choice([torch.bfloat16, torch.float32])
    bf = dtype == torch.bfloat16
    B, N, K = rng.randint(1, 4), rng.randint(1, 300), rng.randint(1, 16)
    D = rng.choice([1, 2, 3, 4, 7, 8, 12, 16, 33, 48, 64, 96, 100, 128, 130, 256])
    kind = rng.choice(["none", "causal", "keypad", "full", "rope_mean", "rope_causal", "features", "act", "rot1",
                       "rot2", "select"])
    g = torch.Generator().manual_seed(9000 + case)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    x, c = rnd(B, N, D) * 0.5, rnd(D, K) * (0.1 if K <= 4 else 0.02)
    dev = lambda t: t.cuda()
    second = "coeff"
    if kind in ("none", "causal"):
        m = None if kind == "none" else "causal"
        ref = lambda x, c: O.aggregate(O.poly_features(x, c), m)
        run = lambda x, c: polynomial_aggregation_(x, c, K, m)
    elif kind == "keypad":
        m = (torch.rand(B, N, generator=g) < 0.5).float()
        m[:, 0] = 1
        ref = lambda x, c: O.aggregate(O.poly_features(x, c), m)
        run = lambda x, c: polynomial_aggregation_(x, c, K, dev(m))
    elif kind == "full":
        m = (torch.rand(B, rng.randint(1, 40), N, generator=g) < 0.5).float()
        m[:, :, 0] = 1
        ref = lambda x, c: O.aggregate(O.poly_features(x, c), m)
        run = lambda x, c: polynomial_aggregation_(x, c, K, dev(m))
    elif kind in ("rope_mean", "rope_causal", "rot1"):
        if D % 2:
            return None
        cos, sin = O.rope_tables_1d(D, N + 9)
        pos = torch.randint(0, N + 9, (N,), generator=g)
        if kind == "rot1":
            second = None
            ref = lambda x, c: O.rope_apply_1d(x, pos, cos, sin)
            run = lambda x, c: P.apply_rope_1d(x, dev(pos), dev(cos), dev(sin))
        else:
            m = None if kind == "rope_mean" else "causal"
            fn = P.poly_agg_rope_mean_triton if m is None else P.poly_agg_rope_causal_triton
            ref = lambda x, c: O.aggregate(O.rope_apply_1d(O.poly_features(x, c), pos, cos, sin), m)
            run = lambda x, c: fn(x, c, K, dev(cos), dev(sin), dev(pos))
    elif kind == "rot2":
        if D % 4:
            return None
        hh, ww = rng.randint(1, 9), rng.randint(1, 9)
        tabs = O.rope_tables_2d(D, hh, ww)
        hw = torch.stack([torch.randint(0, hh, (N,), generator=g), torch.randint(0, ww, (N,), generator=g)], 1)
        second = None
        ref = lambda x, c: O.rope_apply_2d(x, hw, *tabs)
        run = lambda x, c: P.apply_rope_2d(x, dev(hw), *[dev(t) for t in tabs])
    elif kind == "features":
        ref = lambda x, c: O.poly_features(x, c)
        run = lambda x, c: P.poly_features(x, c, K)
    elif kind == "act":
        second = None
        ref = lambda x, c: O.activation(x * 8)
        run = lambda x, c: P.pom_activation(x * 8)
    else:  # selection: x plays the gate, c the aggregate
        heads = rng.choice([1, 1, 2, 4])
        heads = heads if D % heads == 0 else 1
        x = torch.rand(B, N, heads if heads > 1 else D, generator=g)
        c = rnd(B, rng.choice([1, N]), D)
        second = "aggregate"
        ref = lambda x, c: O.selection(x, c, heads)
        run = lambda x, c: polynomial_selection_(x, c, heads)
    if bf:
        x, c = O.bf16_round(x), O.bf16_round(c)
    desc = f"#{case} {kind} {str(dtype)[6:]} B={B} N={N} D={D} K={K}"
    return desc, dtype, ref, run, x, c, second, g


def test_random_operator_calls_against_the_oracle():
    """The operator-level functions (aggregation with every mask kind, the rotary forms, per-token features,
    activation, rotation alone, selection) on random shapes — channel counts from 1 to 256 that are and are not
    multiples of the vector widths, degrees 1 to 16 — in bf16 and fp32: forward and every gradient."""
    rng = random.Random(0)
    failures = []
    for case in range(250):
        drawn = _operator_case(rng, case)
        if drawn is None:
            continue
        desc, dtype, ref, run, x, c, second, g = drawn
        bf = dtype == torch.bfloat16
        xr, cr = x.clone().requires_grad_(True), c.clone().requires_grad_(True)
        xg, cg = x.cuda().to(dtype).requires_grad_(True), c.cuda().to(dtype).requires_grad_(True)
        want, got = ref(xr, cr), run(xg, cg)
        if got.shape != want.shape or got.dtype != dtype:
            failures.append(f"{desc}: shape/dtype {tuple(got.shape)} {got.dtype} vs {tuple(want.shape)}")
            continue
        gy = torch.randn(want.shape, generator=g)
        gy = O.bf16_round(gy) if bf else gy
        ins_r, ins_g = ([xr, cr], [xg, cg]) if second else ([xr], [xg])
        want_g = torch.autograd.grad(want, ins_r, gy)
        got_g = torch.autograd.grad(got, ins_g, gy.cuda().to(dtype))
        errs = [_rel(got.detach(), want.detach())]
        errs += [_rel(a, b) for a, b in zip(got_g, want_g) if float(b.norm()) > 1e-6]
        if not max(errs) <= (BF16_TOL if bf else 2 * FP32_TOL):
            failures.append(f"{desc}: off by {[f'{e:.1e}' for e in errs]}")
    assert not failures, "\n".join(failures)
