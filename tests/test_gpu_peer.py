"""Peer-memory exchange kernels on one GPU with a group of one rank: the push / flag / wait / sum protocol
runs against the rank's own buffer, so sums must equal the local reduction, prefix and suffix carries are
zero, the in-place gradient all-reduce is the identity, and replaying from a CUDA graph keeps working
(device-side epochs).  The two-rank behaviour is covered by tests/test_gpu_shard.py (needs two GPUs)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def peer():
    import torch.distributed as dist
    from pom_b200.peer import PeerExchange

    created = False
    if not dist.is_initialized():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=0, world_size=1)
        created = True
    torch.cuda.set_device(0)
    px = PeerExchange(slot_floats=8192, flat_floats=4096)
    yield px
    px.close()
    if created:
        dist.destroy_process_group()


def test_exchange_with_one_rank_equals_local_reduction(peer):
    from pom_b200 import _abi, ops

    g = torch.Generator().manual_seed(0)
    for B, chunks, P in ((1, 1, 2304), (3, 7, 100), (2, 128, 512)):
        part = torch.randn(B, chunks, P, generator=g).cuda()
        denom = (torch.rand(B, generator=g) + 0.5).cuda()
        want = ops.reduce_partials(part, denom=denom, scale=0.25)
        for _ in range(3):  # consecutive epochs alternate the slot parity
            got = peer.exchange(part, denom=denom, scale=0.25)
            torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
        for mode in (_abi.PEER_SUM_BEFORE, _abi.PEER_SUM_AFTER):
            assert float(peer.exchange(part, mode=mode).abs().max()) == 0.0
    assert _abi.read_status("cuda:0") == 0


def test_exchange_rejects_oversize_messages(peer):
    with pytest.raises(ValueError):
        peer.exchange(torch.zeros(1, 1, peer.slot_floats + 4, device="cuda"))


def test_flat_allreduce_with_one_rank_is_identity_and_graph_replay_advances_epochs(peer):
    from pom_b200 import _abi

    ref = torch.randn(4096, generator=torch.Generator().manual_seed(1)).cuda()
    peer.flat.copy_(ref)
    peer.allreduce_flat(4096)
    assert torch.equal(peer.flat, ref)
    part = torch.randn(2, 5, 64, generator=torch.Generator().manual_seed(2)).cuda()
    want = part.sum(1)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        peer.exchange(part)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = peer.exchange(part)
        peer.allreduce_flat(4096)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    assert torch.equal(peer.flat, ref)
    assert _abi.read_status("cuda:0") == 0
