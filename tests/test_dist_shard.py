"""Token sharding over ranks (world size 2, gloo, CPU): the exchange logic of SeqShard combined with the
oracle's arithmetic must reproduce the single-rank result for the non-causal all-reduce and for the causal
exclusive prefix / suffix scans, including a split that does not fall on a chunk boundary."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pom_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, split, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pom_b200.functional import SeqShard

        torch.manual_seed(0)
        B, N, P, K = 2, 50, 12, 3
        x = torch.randn(B, N, P, dtype=torch.float64)
        coeff = torch.randn(P, K, dtype=torch.float64) * 0.1
        feat = O.poly_features(x, coeff)
        bounds = [0, split, N]
        lo, hi = bounds[rank], bounds[rank + 1]
        shard = SeqShard(token_offset=lo, n_global=N)
        assert shard.world == world and shard.rank == rank
        local = feat[:, lo:hi]

        # non-causal: all-reduce of the partial sums, divide by the global length
        S = local.sum(1)
        shard.all_reduce(S)
        ok_mean = torch.allclose(S / N, O.aggregate(feat, None).squeeze(1), atol=1e-12)

        # causal forward: exclusive prefix of rank totals as carry, global index in the divisor
        carry = shard.exclusive_carry(local.sum(1))
        got = O.aggregate(local, "causal", token_offset=lo, carry=carry)
        ok_causal = torch.allclose(got, O.aggregate(feat, "causal")[:, lo:hi], atol=1e-12)

        # causal backward: exclusive suffix of rank totals of dout[m] / (m + 1)
        dout = torch.randn(B, N, P, dtype=torch.float64)
        w = dout / torch.arange(1, N + 1, dtype=torch.float64).view(1, N, 1)
        suffix_full = w.flip(1).cumsum(1).flip(1)            # W[n] = sum_{m >= n} dout[m] / (m + 1)
        carry_b = shard.exclusive_carry(w[:, lo:hi].sum(1), reverse=True)
        got_b = w[:, lo:hi].flip(1).cumsum(1).flip(1) + carry_b.unsqueeze(1)
        ok_suffix = torch.allclose(got_b, suffix_full[:, lo:hi], atol=1e-12)
        ret[rank] = (ok_mean, ok_causal, ok_suffix)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("split", [25, 7])
def test_token_sharded_exchanges_match_single_rank(split):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, split, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        for r in range(world):
            assert ret[r] == (True, True, True), (r, ret[r])


def test_failed_rank_is_reported_by_exit_code():
    """Failure detection without a GPU: a rank that raises before joining shows up as a non-zero exit code
    on the host, and the surviving process is not left waiting (it never enters a collective)."""
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_raise)
    p.start()
    p.join(60)
    assert p.exitcode not in (0, None)


def _raise():
    raise RuntimeError("injected host-side failure")
