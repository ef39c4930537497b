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


def test_a_wait_on_a_silent_rank_runs_out_and_reports_it():
    """Two-rank layout on one GPU whose second rank never runs: rank 0 pushes its message, waits the configured
    20 ms for a flag that nobody sets, records POM_ERR_TIMEOUT in the status word and returns; the next exchange
    sees the word and does not wait again.  Nothing faults and nothing spins for ever."""
    import ctypes as C

    from pom_b200 import _abi

    lib = _abi.lib()
    lay = (C.c_ulonglong * 3)()
    assert lib.pom_peer_layout(2, 256, 0, lay) == 0
    bufs = [torch.zeros(int(lay[2]), dtype=torch.uint8, device="cuda") for _ in range(2)]
    comm = _abi.PeerComm()
    comm.rank, comm.world, comm.slot_floats, comm.flat_floats = 0, 2, 256, 0
    comm.wait_ns = 20_000_000
    for r in range(2):
        comm.base[r] = bufs[r].data_ptr()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")  # a word of its own: the shared one stays clean
    part = torch.ones(1, 1, 64, device="cuda")
    out = torch.empty(1, 64, device="cuda")
    a = _abi.PeerXchgArgs()
    a.partial, a.out, a.scale, a.B, a.chunks, a.P, a.mode = part.data_ptr(), out.data_ptr(), 1.0, 1, 1, 64, 0

    def launch():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        assert lib.pom_peer_exchange(C.byref(comm), C.byref(a), _abi.ptr(status), _abi.stream_ptr()) == 0
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    ms = launch()
    assert int(status.item()) == -7, "the expired wait must be recorded as POM_ERR_TIMEOUT"
    assert 15.0 < ms < 500.0, f"expected about 20 ms of waiting, measured {ms:.1f} ms"
    ms2 = launch()
    assert int(status.item()) == -7
    assert ms2 < 10.0, f"an exchange after a recorded timeout must not wait again ({ms2:.1f} ms)"
    assert "time" in _abi.strerror(-7).lower()
