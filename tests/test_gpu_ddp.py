"""The layer under torch.nn.parallel.DistributedDataParallel on two GPUs (batch sharding: the data-parallel use of
the benchmark's default workload).  The loss is a mean over the rank's samples, so the parameter gradients that DDP
averages over the ranks must equal the gradients of the whole batch's mean on one GPU; so must the sums that the
layer's own gradient exchange (``grad_peer``) produces, divided by the number of ranks.  Needs two devices."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    from pom_b200 import PoM

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        torch.manual_seed(0)
        mod = PoM(64, 2, 2).cuda().bfloat16()
        with torch.no_grad():
            mod.po_coeff.copy_(torch.randn_like(mod.po_coeff) * 0.1)
        g = torch.Generator().manual_seed(1)
        x = torch.randn(4 * world, 96, 64, generator=g).bfloat16().cuda()
        # the whole batch on this GPU, without DDP
        y = mod(x)
        y.float().square().mean().backward()
        want = [p.grad.float().clone() for p in mod.parameters()]
        for p in mod.parameters():
            p.grad = None
        # this rank's samples under DDP (gradients averaged over ranks by its hooks)
        ddp = DDP(mod, device_ids=[rank])
        xs = x[4 * rank:4 * rank + 4]
        for _ in range(2):  # twice: the second step reuses DDP's buckets
            for p in mod.parameters():
                p.grad = None
            ddp(xs).float().square().mean().backward()
        got = [p.grad.float() for p in mod.parameters()]
        worst = max(float((a - b).norm() / (b.norm() + 1e-20)) for a, b in zip(got, want))
        # the same with the library's own exchange: the backward pass sums the gradients over the ranks itself
        from pom_b200 import _abi
        from pom_b200.peer import PeerExchange

        n_params = sum(p.numel() for p in mod.parameters())
        peer = PeerExchange(slot_floats=4096, flat_floats=n_params + 8)
        for _ in range(2):
            for p in mod.parameters():
                p.grad = None
            mod(xs, grad_peer=peer).float().square().mean().backward()
        assert _abi.read_status(torch.device("cuda", rank)) == 0, "an exchange wait expired"
        got = [p.grad.float() / world for p in mod.parameters()]  # sums over the ranks, where DDP averages
        worst = max([worst] + [float((a - b).norm() / (b.norm() + 1e-20)) for a, b in zip(got, want)])
        peer.close()
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


def test_layer_under_distributed_data_parallel():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    port = _free_port()
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        codes = [p.exitcode for p in procs]
        for p in procs:
            if p.exitcode is None:
                p.kill()
        assert codes == [0, 0], codes
        assert max(ret.values()) < 1.5e-2, dict(ret)  # bf16 gradients summed in two halves
