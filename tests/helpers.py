"""Shared helpers of the GPU parity tests: build modules from golden parameters, run the
CUDA layer and the CPU oracle on the same tensors, compare with norm-relative errors."""
import torch

from oracle import pom_oracle as O

FP32_TOL = 1e-4   # norm-relative and max-normalised bound of the fp32 mode
BF16_TOL = 2e-2   # bound for bf16 storage with fp32 accumulation

PARAM_ORDER = ["qc_proj.weight", "se_bias", "po_coeff", "ag_proj.weight"]
GROUPED_PARAM_ORDER = ["po_proj.weight", "se_proj.weight", "se_proj.bias", "po_coeff", "ag_proj.weight"]


def param_order(params):
    """Trainable-parameter names of a case: the fused layout, or the grouped one when po_proj is present."""
    order = GROUPED_PARAM_ORDER if "po_proj.weight" in params else PARAM_ORDER
    return order + [k for k in ("po_proj.bias", "ag_proj.bias") if k in params]


def rope_cfg(cfg):
    if "rope" not in cfg:
        return None
    r = cfg["rope"]
    return O.RopeConfig(two_d=r["two_d"], max_seq_len=r.get("max_seq_len", 4096), max_h=r.get("max_h", 64),
                        max_w=r.get("max_w", 64))


def make_cuda_module(cfg, params, dtype, device="cuda"):
    """pom_b200 module holding ``params`` (fp32 CPU tensors) cast to ``dtype``; rotary tables stay fp32."""
    from pom_b200 import PoM, PoMRoPE

    r = cfg.get("rope")
    groups = cfg.get("groups", 1)
    if r is None:
        mod = PoM(cfg["dim"], cfg["degree"], cfg["expand"], groups, cfg["heads"], bias=cfg.get("bias", False))
    else:
        mod = PoMRoPE(cfg["dim"], cfg["degree"], cfg["expand"], groups, cfg["heads"], rope_2d=r["two_d"],
                      max_seq_len=r.get("max_seq_len", 4096), max_h=r.get("max_h", 64), max_w=r.get("max_w", 64),
                      bias=cfg.get("bias", False))
    with torch.no_grad():
        named = dict(mod.named_parameters())
        for k in param_order(params):
            named[k].copy_(params[k])
    mod = mod.to(device)
    for p in mod.parameters():
        p.data = p.data.to(dtype)
    return mod


def oracle_run(cfg, params, xq, xc, kwargs, gy):
    """Oracle forward + gradients in fp32 on the given (already rounded) CPU tensors."""
    order = param_order(params)
    ps = {k: params[k].clone().float().requires_grad_(True) for k in order}
    model = O.OraclePoM(ps, cfg["degree"], cfg["expand"], cfg["heads"], rope_cfg(cfg))
    xq = xq.clone().float().requires_grad_(True)
    ins = [xq]
    if xc is not None:
        xc = xc.clone().float().requires_grad_(True)
        ins.append(xc)
    y = model.forward(xq, xc, **kwargs)
    grads = torch.autograd.grad(y, ins + [ps[k] for k in order], gy.float())
    names = [f"in{i}" for i in range(len(ins))] + order
    return y.detach(), dict(zip(names, grads))


def cuda_run(mod, xq, xc, kwargs, gy, dtype, device="cuda"):
    xq = xq.to(device=device, dtype=dtype).requires_grad_(True)
    ins = [xq]
    if xc is not None:
        xc = xc.to(device=device, dtype=dtype).requires_grad_(True)
        ins.append(xc)
    kw = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in kwargs.items()}
    y = mod(xq, xc, **kw) if xc is not None else mod(xq, **kw)
    named = dict(mod.named_parameters())
    order = param_order(named)
    ps = [named[k] for k in order]
    grads = torch.autograd.grad(y, ins + ps, gy.to(device=device, dtype=dtype))
    names = [f"in{i}" for i in range(len(ins))] + order
    return y.detach(), dict(zip(names, grads))


def assert_close(got, want, tol, label):
    n2, mx = O.rel_errors(got.float().cpu(), want.float().cpu())
    assert n2 <= tol and mx <= tol, f"{label}: rel2={n2:.3e} relmax={mx:.3e} > {tol:.1e}"


def assert_status_clean(device="cuda"):
    from pom_b200 import _abi

    assert _abi.read_status(device) == 0, "a device-side wait timed out"
