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
