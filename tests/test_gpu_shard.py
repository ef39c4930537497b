"""Token-sharded layer on two GPUs (NCCL or the peer-memory exchange kernels, eager and replayed from a CUDA
graph): forward output, input gradient and the all-reduced parameter
gradients of each rank's slice must match the single-GPU layer on the full sequence — the library against itself,
which other tests pin to the oracle on one GPU — and, directly, the CPU oracle run on the whole sequence (2e-2).
Needs two devices."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


COMBOS = ((None, False), ("causal", False), (None, True), ("causal", True), ("keypad", False))


def _one_combo(rank, world, mask, rope2d, transport, peer):
    from oracle import pom_oracle as O
    from pom_b200 import PoM, PoMRoPE, SeqShard

    keypad = mask == "keypad"
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
    if keypad:
        mask = (torch.rand(1, N, generator=g) < 0.7).float().cuda()
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
    kw = {"mask": mask[:, lo:lo + n_loc].contiguous() if keypad else mask,
          "shard": SeqShard(token_offset=lo, n_global=N, peer=peer)}
    if rope2d:
        kw["positions_hw"] = hw[lo:lo + n_loc].contiguous()
    xs, gys = x[:, lo:lo + n_loc].contiguous(), gy[:, lo:lo + n_loc].contiguous()
    y_loc, g_loc = run(xs, gys, **kw)
    if transport == "peer_graph":  # the whole sharded step replayed from a CUDA graph (epochs advance on the device)
        side_stream = torch.cuda.Stream()
        with torch.cuda.stream(side_stream):
            run(xs, gys, **kw)
        torch.cuda.current_stream().wait_stream(side_stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_loc, g_loc = run(xs, gys, **kw)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    errs = [O.rel_errors(y_loc, y_full[:, lo:lo + n_loc])[0], O.rel_errors(g_loc[0], g_full[0][:, lo:lo + n_loc])[0]]
    errs += [O.rel_errors(a, b)[0] for a, b in zip(g_loc[1:], g_full[1:])]
    # and against the CPU oracle on the whole sequence (fp32 on the same bf16-rounded values): this rank's slice of
    # the output and of the input gradient, and the parameter gradients summed over the ranks
    names = [n for n, _ in mod.named_parameters()]
    ps = {n: p.detach().float().cpu().requires_grad_(True) for n, p in mod.named_parameters()}
    rope = O.RopeConfig(two_d=True, max_seq_len=4096, max_h=side, max_w=side) if rope2d else None
    xo = x.float().cpu().requires_grad_(True)
    kw_o = {"mask": mask.cpu() if keypad else mask}
    if rope2d:
        kw_o["positions_hw"] = hw.cpu()
    want = O.OraclePoM(ps, K, E, 1, rope).forward(xo, **kw_o)
    want_g = torch.autograd.grad(want, [xo] + [ps[n] for n in names], gy.float().cpu())
    errs_o = [O.rel_errors(y_loc, want[:, lo:lo + n_loc])[0], O.rel_errors(g_loc[0], want_g[0][:, lo:lo + n_loc])[0]]
    errs_o += [O.rel_errors(a, b)[0] for a, b in zip(g_loc[1:], want_g[1:])]
    assert max(errs_o) < 2e-2, (mask if not keypad else "keypad", rope2d, transport, errs_o)
    return max(errs)


def _worker(rank, world, port, transport, ret):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from pom_b200 import _abi

        peer = None
        if transport != "nccl":
            from pom_b200.peer import PeerExchange
            peer = PeerExchange(slot_floats=4096, flat_floats=1 << 16)
        worst = {}
        for mask, rope2d in COMBOS:
            worst[f"{mask}/{rope2d}"] = _one_combo(rank, world, mask, rope2d, transport, peer)
        assert _abi.read_status(torch.device("cuda", rank)) == 0, "an exchange wait expired"
        ret[rank] = worst
        if peer is not None:
            peer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["nccl", "peer", "peer_graph"])
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
        codes = [p.exitcode for p in procs]
        for p in procs:
            if p.exitcode is None:
                p.kill()
        assert codes == [0, 0], codes
        # both sides are bf16 results of the same kernels; only summation order and rounding of partials differ
        for rank_worst in ret.values():
            assert max(rank_worst.values()) < 1.5e-2, dict(ret)
