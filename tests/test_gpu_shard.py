"""Token-sharded layer on two GPUs (NCCL): forward output, input gradient and the all-reduced parameter
gradients of each rank's slice must match the single-GPU layer on the full sequence.  Needs two devices."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import pom_oracle as O
        from pom_b200 import PoM, PoMRoPE, SeqShard

        mask, rope2d = case
        D, K, E, side = 64, 2, 2, 16
        N = side * side
        torch.manual_seed(0)
        mod = (PoMRoPE(D, K, E, 1, 1, rope_2d=True, max_h=side, max_w=side) if rope2d else PoM(D, K, E, 1, 1))
        with torch.no_grad():
            mod.po_coeff.copy_(torch.randn_like(mod.po_coeff) * 0.1)
        mod = mod.cuda()
        for p in mod.parameters():
            p.data = p.data.bfloat16()
        g = torch.Generator().manual_seed(1)
        x = torch.randn(1, N, D, generator=g).bfloat16().cuda()
        gy = torch.randn(1, N, D, generator=g).bfloat16().cuda()
        hw = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1).cuda()
        params = list(mod.parameters())

        def run(xs, gys, **kw):
            xr = xs.clone().requires_grad_(True)
            y = mod(xr, **kw)
            grads = torch.autograd.grad(y, [xr] + params, gys)
            return y.detach(), grads

        kw_full = {"mask": mask}
        if rope2d:
            kw_full["positions_hw"] = hw
        y_full, g_full = run(x, gy, **kw_full)

        n_loc = N // world
        lo = rank * n_loc
        kw = {"mask": mask, "shard": SeqShard(token_offset=lo, n_global=N)}
        if rope2d:
            kw["positions_hw"] = hw[lo:lo + n_loc].contiguous()
        y_loc, g_loc = run(x[:, lo:lo + n_loc].contiguous(), gy[:, lo:lo + n_loc].contiguous(), **kw)
        errs = [O.rel_errors(y_loc, y_full[:, lo:lo + n_loc])[0], O.rel_errors(g_loc[0], g_full[0][:, lo:lo + n_loc])[0]]
        errs += [O.rel_errors(a, b)[0] for a, b in zip(g_loc[1:], g_full[1:])]
        ret[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", [(None, False), ("causal", False), (None, True), ("causal", True)])
def test_two_gpu_token_sharding_matches_single_gpu(case):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    port = _free_port()
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, case, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        # both sides are bf16 results of the same kernels; only summation order and rounding of partials differ
        assert max(ret.values()) < 1.5e-2, dict(ret)
