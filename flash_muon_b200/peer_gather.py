"""Copy-engine all-gather for ``Muon.step`` inside one NVLink-connected box.

Stands in for ``dist.all_gather_into_tensor(update_buffer, g, async_op=True)``
(flash_muon/muon.py:108).  NCCL's all-gather runs as a kernel and needs SMs, but the persistent
tcgen05 GEMM kernels of the next round's Newton-Schulz hold every SM, so on B200 the two do not
overlap (measured at 8 GPUs: ~10 ms of a 75 ms step exposed).  Here every rank *pushes* its
finished slot into the gather buffers of its peers with DMA copy engines, and the exchange is
ordered by 32-bit flags that the CUDA streams themselves write and wait on
(``fm_stream_write32`` / ``fm_stream_wait32_geq``): no kernel, no SM, no host synchronisation.

Per numel group there are several gather buffers (rounds rotate through them) and, for each, two
flag rows:

* ``READY[r]`` -- written by producer ``r`` into every consumer after its slot has landed;
* ``ACK[q]``   -- written by consumer ``q`` into producer ``r`` once ``q`` has applied the update
  that read ``r``'s slot, i.e. the slot in ``q``'s buffer may be overwritten.

Flag values are per-(producer, buffer) use counters that every rank advances identically, so no
value is ever reused and a late flag can never be mistaken for an early one.
Process-to-process addresses come from CUDA IPC handles exchanged once through the existing
``torch.distributed`` group.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ._lib import check, lib

READY, ACK = 0, 1


def _export(t: torch.Tensor):
    handle = ctypes.create_string_buffer(64)
    off = ctypes.c_uint64(0)
    check(lib.fm_ipc_export(t.data_ptr(), handle, ctypes.byref(off)))
    return handle.raw, off.value


def _import(handle: bytes, offset: int) -> int:
    out = ctypes.c_void_p(0)
    check(lib.fm_ipc_import(handle, offset, ctypes.byref(out)))
    return out.value


class PeerRound:
    """What ``Muon.step`` holds for a round in flight: ``wait()`` before the update reads the
    buffer, ``done()`` after it has."""

    def __init__(self, owner: "PeerGather", gi: int, b: int, producers: list[int], seqs: list[int]):
        self.owner, self.gi, self.b, self.producers, self.seqs = owner, gi, b, producers, seqs

    def wait(self) -> None:
        o = self.owner
        st = torch.cuda.current_stream(o.device).cuda_stream
        for r, s in zip(self.producers, self.seqs):
            if r != o.rank:
                check(lib.fm_stream_wait32_geq(o.flag_addr(o.rank, self.gi, self.b, READY, r), s, st))

    def done(self) -> None:
        o = self.owner
        st = torch.cuda.current_stream(o.device).cuda_stream
        for r, s in zip(self.producers, self.seqs):
            if r != o.rank:
                check(lib.fm_stream_write32(o.flag_addr(r, self.gi, self.b, ACK, o.rank), s, st))


class PeerGather:
    """Collective constructor: every rank of the default group must call it with the same list of
    buffer lists (one list per numel group, ``[world_size, numel]`` bf16 each)."""

    def __init__(self, rank: int, world_size: int, buffers: list[list[torch.Tensor]]):
        self.rank, self.ws = rank, world_size
        self.device = buffers[0][0].device
        self.ngroups = len(buffers)
        self.nbuf = max(len(bl) for bl in buffers)
        self.buffers = buffers
        self.buffer_ptrs = [[b.data_ptr() for b in bl] for bl in buffers]
        # [group, buffer, kind, rank] use counters written by peers
        self.flags = torch.zeros(self.ngroups, self.nbuf, 2, world_size, dtype=torch.int32,
                                 device=self.device)
        torch.cuda.synchronize(self.device)
        mine = {"flags": _export(self.flags),
                "bufs": [[_export(b) for b in bl] for bl in buffers]}
        everyone: list = [None] * world_size
        dist.all_gather_object(everyone, mine)
        self._flag_base = [0] * world_size
        self._buf_base = [None] * world_size
        for r, info in enumerate(everyone):
            if r == rank:
                self._flag_base[r] = self.flags.data_ptr()
                self._buf_base[r] = self.buffer_ptrs
            else:
                self._flag_base[r] = _import(*info["flags"])
                self._buf_base[r] = [[_import(*h) for h in hl] for hl in info["bufs"]]
        dist.barrier()  # nobody writes a flag before everybody has zeroed and mapped them
        self.streams = {q: torch.cuda.Stream(device=self.device) for q in range(world_size) if q != rank}
        # host-side mirror of the use counters: seq[group][buffer][producer]
        self.seq = [[[0] * world_size for _ in range(self.nbuf)] for _ in range(self.ngroups)]
        # events of this rank's copies out of its slot, per (group, buffer)
        self.push_events = [[[] for _ in range(self.nbuf)] for _ in range(self.ngroups)]

    def flag_addr(self, holder: int, gi: int, b: int, kind: int, idx: int) -> int:
        return self._flag_base[holder] + 4 * ((((gi * self.nbuf + b) * 2 + kind) * self.ws) + idx)

    def before_slot_write(self, gi: int, b: int, stream: torch.cuda.Stream) -> None:
        """``stream`` is about to overwrite this rank's slot of buffer ``b``: earlier copies out
        of it must have finished."""
        for ev in self.push_events[gi][b]:
            stream.wait_event(ev)
        self.push_events[gi][b] = []

    def publish(self, gi: int, b: int, slot: torch.Tensor, producers: list[int]) -> PeerRound:
        """Called on the stream that produced ``slot`` (this rank's row of buffer ``b``)."""
        seqs = []
        for r in producers:
            self.seq[gi][b][r] += 1
            seqs.append(self.seq[gi][b][r])
        if self.rank in producers:
            s = self.seq[gi][b][self.rank]
            nbytes = slot.numel() * slot.element_size()
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(self.device))
            for q, st in self.streams.items():
                st.wait_event(ready)
                sp = st.cuda_stream
                # q has applied the update that read my previous slot in its buffer b
                check(lib.fm_stream_wait32_geq(self.flag_addr(self.rank, gi, b, ACK, q), s - 1, sp))
                dst = self._buf_base[q][gi][b] + self.rank * nbytes
                check(lib.fm_copy_async(dst, slot.data_ptr(), nbytes, sp))
                check(lib.fm_stream_write32(self.flag_addr(q, gi, b, READY, self.rank), s, sp))
                ev = torch.cuda.Event()
                ev.record(st)
                self.push_events[gi][b].append(ev)
        return PeerRound(self, gi, b, producers, seqs)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        lib.fm_ipc_close_all()
