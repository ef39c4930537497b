"""Generate golden input/output vectors by running the reference implementation on CPU.

Usage (only where the reference checkout is available; it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/davidpicard-pom

Writes ``tests/golden/pom_golden.pt``: a dict of cases, each holding the exact inputs,
parameters, outputs and gradients the reference package (pom.PoM / pom.PoMRoPE /
pom.pom.polynomial_aggregation_, pure-PyTorch CPU path) produced.  Small shapes keep the
file to a few hundred kilobytes; the one full-size case (the reference's CPU configuration,
B=2 N=256 D=256) stores a strided sample of the output plus summary statistics and is
replayed from seeds.
"""
import os
import sys

import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from pom import PoM, PoMRoPE  # noqa: E402
    from pom.pom import polynomial_aggregation_  # noqa: E402

    torch.set_num_threads(1)  # fixed summation order
    cases = {}

    def grads_of(module, inputs, out, seed=7):
        torch.manual_seed(seed)
        g = torch.randn_like(out)
        params = [p for p in module.parameters()]
        res = torch.autograd.grad(out, list(inputs) + params, g, allow_unused=True)
        names = [f"d_in{i}" for i in range(len(inputs))] + ["d_" + n for n, _ in module.named_parameters()]
        return g, {n: (r if r is not None else torch.zeros(0)) for n, r in zip(names, res)}

    def make_module(cls, dim, degree, expand, heads=1, seed=0, **kw):
        torch.manual_seed(seed)
        m = cls(dim, degree, expand, 1, heads, **kw)
        with torch.no_grad():
            torch.manual_seed(seed + 100)
            m.po_coeff.copy_(torch.randn_like(m.po_coeff) * 0.1)
            m.se_bias.copy_(torch.randn_like(m.se_bias) * 0.5)
        return m

    def record(name, module, kwargs_fn, xq, xc=None, cfg=None):
        xq = xq.clone().requires_grad_(True)
        ins = [xq]
        if xc is not None:
            xc = xc.clone().requires_grad_(True)
            ins.append(xc)
        kwargs = kwargs_fn()
        y = module(xq, xc, **kwargs) if xc is not None else module(xq, **kwargs)
        g, grads = grads_of(module, ins, y)
        cases[name] = {
            "cfg": cfg,
            "params": {k: v.detach().clone() for k, v in module.state_dict().items()},
            "xq": xq.detach().clone(),
            "xc": None if xc is None else xc.detach().clone(),
            "kwargs": {k: v for k, v in kwargs.items()},
            "y": y.detach().clone(),
            "gy": g,
            "grads": {k: v.detach().clone() for k, v in grads.items()},
        }

    B, N, D, K, E = 2, 24, 16, 3, 2
    cfg = dict(dim=D, degree=K, expand=E, heads=1)
    torch.manual_seed(11)
    x = torch.randn(B, N, D)
    torch.manual_seed(12)
    xq_cross = torch.randn(B, 10, D)

    m = make_module(PoM, D, K, E)
    record("pom_none", m, lambda: dict(mask=None), x, cfg=cfg)
    record("pom_causal", m, lambda: dict(mask="causal"), x, cfg=cfg)
    torch.manual_seed(99)
    m2 = (torch.rand(B, N) < 0.5).float()
    m2[:, 0] = 1.0
    record("pom_mask2d", m, lambda: dict(mask=m2), x, cfg=cfg)
    torch.manual_seed(98)
    m3 = (torch.rand(B, N, N) < 0.5).float()
    m3[:, torch.arange(N), torch.arange(N)] = 1.0
    record("pom_mask3d", m, lambda: dict(mask=m3), x, cfg=cfg)
    record("pom_cross", m, lambda: dict(mask=None), xq_cross, xc=x, cfg=cfg)
    torch.manual_seed(97)
    m2c = (torch.rand(B, N) < 0.6).float()
    m2c[:, 0] = 1.0
    record("pom_cross_mask2d", m, lambda: dict(mask=m2c), xq_cross, xc=x, cfg=cfg)

    # multi-head scalar gating
    cfg_h = dict(dim=D, degree=K, expand=E, heads=4)
    mh = make_module(PoM, D, K, E, heads=4)
    record("pom_heads4_none", mh, lambda: dict(mask=None), x, cfg=cfg_h)
    record("pom_heads4_causal", mh, lambda: dict(mask="causal"), x, cfg=cfg_h)
    record("pom_heads4_mask3d", mh, lambda: dict(mask=m3), x, cfg=cfg_h)

    # grouped polynomial projection (n_groups = 2): po_proj is a grouped 1x1 convolution, se_proj a biased Linear
    def make_grouped(cls, heads=1, seed=3, **kw):
        torch.manual_seed(seed)
        mg = cls(D, K, E, 2, heads, **kw)
        with torch.no_grad():
            torch.manual_seed(seed + 100)
            mg.po_coeff.copy_(torch.randn_like(mg.po_coeff) * 0.1)
            mg.se_proj.bias.copy_(torch.randn_like(mg.se_proj.bias) * 0.5)
        return mg

    cfg_g = dict(dim=D, degree=K, expand=E, heads=1, groups=2)
    mg = make_grouped(PoM)
    record("pom_groups2_none", mg, lambda: dict(mask=None), x, cfg=cfg_g)
    record("pom_groups2_causal", mg, lambda: dict(mask="causal"), x, cfg=cfg_g)
    record("pom_groups2_cross_mask2d", mg, lambda: dict(mask=m2c), xq_cross, xc=x, cfg=cfg_g)
    mgh = make_grouped(PoM, heads=4)
    record("pom_groups2_heads4_none", mgh, lambda: dict(mask=None), x, cfg=dict(cfg_g, heads=4))
    # bias=True: the grouped convolution and the output projection both carry a bias (pom/pom.py:182, 191)
    mgb = make_grouped(PoM, seed=5, bias=True)
    with torch.no_grad():
        torch.manual_seed(205)
        mgb.po_proj.bias.copy_(torch.randn_like(mgb.po_proj.bias) * 0.3)
        mgb.ag_proj.bias.copy_(torch.randn_like(mgb.ag_proj.bias) * 0.3)
    cfg_gb = dict(cfg_g, bias=True)
    record("pom_groups2_bias_none", mgb, lambda: dict(mask=None), x, cfg=cfg_gb)
    record("pom_groups2_bias_causal", mgb, lambda: dict(mask="causal"), x, cfg=cfg_gb)
    record("pom_groups2_bias_cross", mgb, lambda: dict(mask=None), xq_cross, xc=x, cfg=cfg_gb)

    # ar_forward as the reference defines it (no aggregation: the gate multiplies the raw projection)
    with torch.no_grad():
        y_ar, st_ar = m.ar_forward(x, {"max_len": 64, "h": 0.0, "n": 5})
        yh_ar, sth_ar = mh.ar_forward(x, {"max_len": 64, "h": 0.0, "n": 0})
    cases["pom_ar"] = {"cfg": cfg, "params": {k: v.detach().clone() for k, v in m.state_dict().items()},
                       "xq": x.clone(), "y": y_ar.clone(), "h": st_ar["h"].clone(), "n": int(st_ar["n"]),
                       "max_len": st_ar["max_len"]}
    cases["pom_ar_heads4"] = {"cfg": cfg_h, "params": {k: v.detach().clone() for k, v in mh.state_dict().items()},
                              "xq": x.clone(), "y": yh_ar.clone(), "h": sth_ar["h"].clone(), "n": int(sth_ar["n"]),
                              "max_len": sth_ar["max_len"]}

    # state_forward over three frames of unequal length
    frames = [x[:, :8], x[:, 8:14], x[:, 14:]]
    state, ys = None, []
    with torch.no_grad():
        for f in frames:
            y, state = m.state_forward(f, f, state)
            ys.append(y.clone())
    cases["pom_state"] = {
        "cfg": cfg,
        "params": {k: v.detach().clone() for k, v in m.state_dict().items()},
        "frames": [f.clone() for f in frames],
        "ys": ys,
        "h": state["h"].clone(),
        "n": int(state["n"]),
    }

    # rotary variants
    rcfg1 = dict(cfg, rope=dict(two_d=False, max_seq_len=64))
    r1 = make_module(PoMRoPE, D, K, E, max_seq_len=64)
    record("rope1d_none", r1, lambda: dict(mask=None), x, cfg=rcfg1)
    record("rope1d_causal", r1, lambda: dict(mask="causal"), x, cfg=rcfg1)
    record("rope1d_mask2d", r1, lambda: dict(mask=m2), x, cfg=rcfg1)
    pos = torch.arange(N) * 2 + 3
    record("rope1d_positions", r1, lambda: dict(mask=None, positions=pos), x, cfg=rcfg1)
    record("rope1d_cross", r1, lambda: dict(mask=None, positions=torch.arange(10) + 5,
                                            ctx_positions=torch.arange(N)), xq_cross, xc=x, cfg=rcfg1)
    rcfg2 = dict(cfg, rope=dict(two_d=True, max_h=8, max_w=8))
    r2 = make_module(PoMRoPE, D, K, E, rope_2d=True, max_h=8, max_w=8)
    hw = torch.stack([torch.arange(N) // 6, torch.arange(N) % 6], dim=1)
    record("rope2d_none", r2, lambda: dict(mask=None, positions_hw=hw), x, cfg=rcfg2)
    record("rope2d_causal", r2, lambda: dict(mask="causal", positions_hw=hw), x, cfg=rcfg2)
    rcfg2h = dict(cfg_h, rope=dict(two_d=True, max_h=8, max_w=8))
    r2h = make_module(PoMRoPE, D, K, E, heads=4, rope_2d=True, max_h=8, max_w=8)
    record("rope2d_heads4_none", r2h, lambda: dict(mask=None, positions_hw=hw), x, cfg=rcfg2h)
    rcfg1h = dict(cfg_h, rope=dict(two_d=False, max_seq_len=64))
    r1h = make_module(PoMRoPE, D, K, E, heads=4, max_seq_len=64)
    record("rope1d_heads4_causal", r1h, lambda: dict(mask="causal"), x, cfg=rcfg1h)

    # operator level, following the reference's own test recipe (seed 42, x * 0.5, coeff * 0.1; seed 7 gradient)
    for k in (1, 2, 4, 8, 16):
        for mask_kind in ("none", "causal"):
            torch.manual_seed(42)
            xo = (torch.randn(2, 16, 96) * 0.5).requires_grad_(True)
            co = (torch.randn(96, k) * 0.1).requires_grad_(True)
            out = polynomial_aggregation_(xo, co, k, None if mask_kind == "none" else "causal")
            torch.manual_seed(7)
            go = torch.randn_like(out)
            dx, dc = torch.autograd.grad(out, [xo, co], go)
            cases[f"op_{mask_kind}_k{k}"] = {"x": xo.detach().clone(), "coeff": co.detach().clone(), "out": out.detach().clone(),
                                            "g": go, "dx": dx, "dcoeff": dc}

    # the reference's CPU configuration: replayed from seeds, sampled output
    torch.manual_seed(0)
    big = PoM(256, 2, 2, 1, 1)
    torch.manual_seed(0)
    xb = torch.randn(2, 256, 256)
    with torch.no_grad():
        yb = big(xb)
    cases["cfg1_fp32"] = {
        "cfg": dict(dim=256, degree=2, expand=2, heads=1, B=2, N=256),
        "y_sample": yb[:, ::8, ::8].clone(),
        "y_abs_mean": yb.abs().mean().item(),
        "y_std": yb.std().item(),
        "w_qc_sample": big.qc_proj.weight[::64, ::32].detach().clone(),
        "coeff_sample": big.po_coeff[::64].detach().clone(),
    }

    out_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pom_golden.pt")
    torch.save(cases, out_path)
    print(f"wrote {out_path}: {len(cases)} cases, {os.path.getsize(out_path) / 1024:.0f} KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a davidpicard/pom checkout>")
    main(sys.argv[1])
