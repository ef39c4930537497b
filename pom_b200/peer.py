"""``PeerExchange`` — the cross-rank sums of a token-sharded layer over NVLink peer memory.

Each rank allocates one exchange buffer, exports it as a CUDA IPC handle, and maps the buffers of the
other ranks of the node; the kernels behind ``pom_peer_exchange`` / ``pom_peer_allreduce_flat`` then push
and pull the messages with plain peer stores and loads.  Unlike library collectives these launches can be
captured into a CUDA graph together with the rest of the layer step.

The reference is single-GPU (pom/pom.py:216-231 runs the whole sequence on one device); this is the
transport for the ``SeqShard`` extension of :mod:`pom_b200.functional`.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _abi
from ._abi import PeerComm, PeerXchgArgs, ptr


class PeerExchange:
    """Exchange buffers of all ranks of ``group`` (one node, one GPU per rank).

    ``slot_floats``: largest message (B·P fp32 values) a single exchange may carry.
    ``flat_floats``: size of the parameter-gradient region that ``allreduce_flat`` sums in place.
    ``wait_ms``: limit of every device-side wait on another rank (0 = the library default of 2 s).
    Collective: every rank of the group must construct it at the same point of the program.
    """

    def __init__(self, group=None, slot_floats: int = 1 << 16, flat_floats: int = 0, device=None,
                 wait_ms: float = 0.0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > _abi.PEER_MAX_RANKS:
            raise ValueError(f"at most {_abi.PEER_MAX_RANKS} ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        slot_floats = (int(slot_floats) + 3) // 4 * 4
        flat_floats = (int(flat_floats) + 7) // 8 * 8
        lay = (C.c_ulonglong * 3)()
        lib = _abi.lib()
        _abi.check(lib.pom_peer_layout(self.world, slot_floats, flat_floats, lay), "pom_peer_layout")
        self._slots_off, self._flat_off, total = int(lay[0]), int(lay[1]), int(lay[2])
        self.slot_floats, self.flat_floats = slot_floats, flat_floats
        # an allocation of its own (>= 20 MiB requests bypass the allocator's shared segments)
        self.mem = torch.zeros(max(total, 32 << 20), dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize(self.device)

        # Every step below is agreed on by all ranks, so a failure on one of them raises everywhere instead of
        # leaving the others waiting in a collective.
        handle = (C.c_ubyte * _abi.PEER_HANDLE_BYTES)()
        offset = C.c_ulonglong(0)
        rc = lib.pom_peer_export(ptr(self.mem), handle, C.byref(offset))
        mine = (bytes(handle), int(offset.value)) if rc == 0 else None
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        if any(e is None for e in everyone):
            raise RuntimeError("CUDA IPC export of the exchange buffer failed on rank(s) "
                               f"{[r for r, e in enumerate(everyone) if e is None]}")

        self._opened = []
        self.comm = PeerComm()
        self.comm.rank, self.comm.world = self.rank, self.world
        self.comm.slot_floats, self.comm.flat_floats = slot_floats, flat_floats
        self.comm.wait_ns = int(wait_ms * 1e6)  # 0: the library's default limit (2 s) for every wait on a peer
        mapped = True
        for r, (h, off) in enumerate(everyone):
            if r == self.rank:
                self.comm.base[r] = self.mem.data_ptr()
                continue
            buf = (C.c_ubyte * _abi.PEER_HANDLE_BYTES).from_buffer_copy(h)
            base = C.c_void_p()
            if lib.pom_peer_open(buf, C.byref(base)) != 0:
                mapped = False
                break
            self._opened.append(base.value)
            self.comm.base[r] = base.value + off
        verdicts = [None] * self.world
        dist.all_gather_object(verdicts, mapped, group=group)  # also: nobody pushes before every buffer is mapped
        if not all(verdicts):
            for base in self._opened:
                lib.pom_peer_close(C.c_void_p(base))
            self._opened = []
            raise RuntimeError(f"mapping a peer's exchange buffer failed on rank(s) "
                               f"{[r for r, v in enumerate(verdicts) if not v]}")
        self.flat = self.mem[self._flat_off:self._flat_off + 4 * flat_floats].view(torch.float32)
        res_off = self._flat_off + 6 * flat_floats   # after the fp32 accumulators and their bf16 staging image
        self.flat_bf16 = self.mem[res_off:res_off + 2 * flat_floats].view(torch.bfloat16)

    # ------------------------------------------------------------------ exchanges
    def exchange(self, partial: torch.Tensor, *, mode: int = _abi.PEER_SUM_ALL, denom: Optional[torch.Tensor] = None,
                 scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """(B, chunks, P) fp32 local partial sums -> (B, P) sum over chunks and over the ranks ``mode`` selects."""
        B, chunks, P = partial.shape
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise TypeError("expected a contiguous fp32 (B, chunks, P) tensor")
        if B * P > self.slot_floats:
            raise ValueError(f"message of {B * P} values exceeds slot_floats={self.slot_floats}")
        if out is None:
            out = torch.empty((B, P), dtype=torch.float32, device=partial.device)
        a = PeerXchgArgs()
        a.partial, a.out, a.denom = ptr(partial), ptr(out), ptr(denom)
        a.scale, a.B, a.chunks, a.P, a.mode = float(scale), B, chunks, P, mode
        _abi.check(_abi.lib().pom_peer_exchange(C.byref(self.comm), C.byref(a), ptr(_abi.status_word(partial.device)),
                                                _abi.stream_ptr()), "pom_peer_exchange")
        return out

    def flat_buffer(self, n: int) -> Optional[torch.Tensor]:
        """The first ``n`` floats of the gradient region (None when it is too small)."""
        return self.flat[:n] if n <= self.flat_floats else None

    def owns(self, t: torch.Tensor) -> bool:
        return t.data_ptr() == self.flat.data_ptr()

    def allreduce_flat(self, n: int) -> None:
        """In-place sum over ranks of the first ``n`` floats (rounded up to 4) of the gradient region."""
        n4 = (n + 3) // 4 * 4
        _abi.check(_abi.lib().pom_peer_allreduce_flat(C.byref(self.comm), n4, ptr(_abi.status_word(self.device)),
                                                      _abi.stream_ptr()), "pom_peer_allreduce_flat")

    def allreduce_flat_bf16(self, n: int) -> torch.Tensor:
        """Sum over ranks of the first ``n`` gradient accumulators with bf16 on the wire; returns the bf16 result
        as a view of this rank's result image (valid until the next call: copy what must outlive it)."""
        n8 = (n + 7) // 8 * 8
        _abi.check(_abi.lib().pom_peer_allreduce_flat_bf16(C.byref(self.comm), n8, ptr(_abi.status_word(self.device)),
                                                           _abi.stream_ptr()), "pom_peer_allreduce_flat_bf16")
        return self.flat_bf16[:n]

    def check(self) -> None:
        """Synchronising read of the device status word: raises when a wait on another rank ran out of time.
        After that the exchange buffers are out of step (the rank that gave up has advanced its epochs): build a
        new ``PeerExchange`` and clear the status word (``_abi.status_word(device).zero_()``) before going on."""
        code = int(_abi.status_word(self.device).item())
        if code:
            raise _abi.PomError(code, "peer exchange")

    def close(self) -> None:
        """Unmap the peers' buffers (after a barrier: nobody may still be reading ours)."""
        if self._opened:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            for base in self._opened:
                _abi.lib().pom_peer_close(C.c_void_p(base))
            self._opened = []
