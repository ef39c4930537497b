"""One process, two GPUs: tensors on a device that is not the current one.  The library launches on the current
device's current stream and keeps per-device state (function attributes, status words), so every entry point of
the Python layer switches to the device of its tensors first, as PyTorch's own operators do."""
import pytest
import torch

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


def _step(mod, x, **kw):
    x = x.clone().requires_grad_(True)
    y = mod(x, **kw)
    y.float().square().sum().backward()
    grads = [x.grad] + [p.grad for p in mod.parameters()]
    for p in mod.parameters():
        p.grad = None
    return [y.detach()] + [g.detach() for g in grads]


@needs_two
@pytest.mark.parametrize("kind", ["plain", "causal", "rope2d", "heads", "fp32"])
def test_layer_on_the_device_that_is_not_current(kind):
    from pom_b200 import PoM, PoMRoPE

    torch.cuda.set_device(0)
    torch.manual_seed(0)
    dtype = torch.float32 if kind == "fp32" else torch.bfloat16
    kw = {}
    if kind == "rope2d":
        mod = PoMRoPE(64, 2, 2, rope_2d=True, max_h=16, max_w=16)
        kw["positions_hw"] = torch.stack([torch.arange(256) // 16, torch.arange(256) % 16], 1)
    else:
        mod = PoM(64, 2, 2, n_sel_heads=8 if kind == "heads" else 1)
    if kind == "causal":
        kw["mask"] = "causal"
    x = torch.randn(2, 256, 64).to(dtype)
    outs = {}
    for dev in ("cuda:0", "cuda:1"):
        m = mod.to(dev).to(dtype)
        k = {a: (b.to(dev) if torch.is_tensor(b) else b) for a, b in kw.items()}
        outs[dev] = [t.cpu() for t in _step(m, x.to(dev), **k)]
        assert torch.cuda.current_device() == 0
    if kind == "heads":  # the per-head gate gradient is accumulated with atomics: equal up to summation order
        for a, b in zip(outs["cuda:0"], outs["cuda:1"]):
            assert torch.allclose(a.float(), b.float(), rtol=2e-2, atol=1e-3)
    else:
        for a, b in zip(outs["cuda:0"], outs["cuda:1"]):
            assert torch.equal(a, b)


@needs_two
def test_operators_on_the_device_that_is_not_current():
    from pom_b200 import polynomial_aggregation_
    from pom_b200.operators import apply_rope_1d, pom_activation
    from pom_b200.pom_rope import precompute_freqs_1d

    torch.cuda.set_device(0)
    torch.manual_seed(1)
    x = torch.randn(2, 100, 64)
    c = torch.randn(64, 2) * 0.1
    cos, sin = precompute_freqs_1d(64, 128)
    res = {}
    for dev in ("cuda:0", "cuda:1"):
        xd = x.to(dev)
        res[dev] = [polynomial_aggregation_(xd, c.to(dev), 2, "causal").cpu(), pom_activation(xd).cpu(),
                    apply_rope_1d(xd, torch.arange(100, device=dev), cos.to(dev), sin.to(dev)).cpu()]
        assert torch.cuda.current_device() == 0
    for a, b in zip(res["cuda:0"], res["cuda:1"]):
        assert torch.equal(a, b)
