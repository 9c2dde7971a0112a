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

The same machinery carries a second kind of exchange: instead of gathering every update and
letting every rank apply it, the OWNER applies decay + update to its copy of the parameter and
pushes the updated parameter into the replicas of its peers.  All replicas are bit-identical
before the step and the update is deterministic, so the result is the one the reference computes
on every rank -- but a rank streams 1/world_size of the parameters through HBM instead of all of
them.  Since the destination is then live model state rather than a scratch buffer, a producer
additionally waits for ``STEP[q]``, which consumer ``q`` writes when it enters the same step
(after whatever it did with the parameters before, e.g. the backward pass).
Process-to-process addresses come from CUDA IPC handles exchanged once through the existing
``torch.distributed`` group.

All device-facing operations go through a small ``ops`` object (``CudaOps`` here); the protocol
itself is plain bookkeeping, which lets a test drive it against simulated streams under
arbitrary interleavings.

A stream that waits on a flag waits for ever if the peer that should write it has left (an
exception between steps, a crashed process): unlike an NCCL collective, a stream memory operation
has no timeout.  The deadline is therefore kept on the host.  Every step leaves a record of the
flag values its streams wait for and an event behind its last operation; ``poll()`` -- called by a
small watchdog thread once a second and by every ``begin_step`` -- looks at the oldest unfinished
step, and if it is older than ``timeout_s`` it writes the awaited values into this rank's own flag
words from a separate stream, so that every parked stream drains, marks the exchange ``failed``
and makes the next ``begin_step`` raise.  All awaited flags live in this rank's own memory, so the
release needs nothing from the peer that is gone.
"""
from __future__ import annotations

import ctypes
import os
import threading
import time

import torch
import torch.distributed as dist

from ._lib import check, lib

READY, ACK = 0, 1


class PeerExchangeError(RuntimeError):
    """A peer did not take part in a step within the deadline; the parameters of that step are
    not to be trusted (the parked streams were released without their data)."""


class CudaOps:
    """The device operations the protocol needs, on real CUDA streams of one device."""

    def __init__(self, device: torch.device):
        self.device = device

    # -- set-up (collective)
    def alloc_flags(self, n: int):
        t = torch.zeros(n, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        return t, t.data_ptr()

    def export(self, addr: int) -> tuple:
        handle = ctypes.create_string_buffer(64)
        off = ctypes.c_uint64(0)
        check(lib.fm_ipc_export(addr, handle, ctypes.byref(off)))
        return handle.raw, off.value

    def import_(self, exported: tuple) -> int:
        out = ctypes.c_void_p(0)
        check(lib.fm_ipc_import(exported[0], exported[1], ctypes.byref(out)))
        return out.value

    def exchange(self, obj, world_size: int) -> list:
        everyone: list = [None] * world_size
        dist.all_gather_object(everyone, obj)
        return everyone

    def barrier(self) -> None:
        dist.barrier()

    # -- streams and events
    def new_stream(self):
        return torch.cuda.Stream(device=self.device)

    def current_stream(self):
        return torch.cuda.current_stream(self.device)

    def record(self, stream):
        ev = torch.cuda.Event()
        ev.record(stream)
        return ev

    def wait_event(self, stream, event) -> None:
        stream.wait_event(event)

    def query(self, event) -> bool:
        return event.query()

    def now(self) -> float:
        return time.monotonic()

    # -- stream-ordered memory operations
    def wait32_geq(self, stream, addr: int, value: int) -> None:
        check(lib.fm_stream_wait32_geq(addr, value, stream.cuda_stream))

    def write32(self, stream, addr: int, value: int) -> None:
        check(lib.fm_stream_write32(addr, value, stream.cuda_stream))

    def copy(self, stream, dst: int, src: int, nbytes: int) -> None:
        check(lib.fm_copy_async(dst, src, nbytes, stream.cuda_stream))


class PeerRound:
    """What ``Muon.step`` holds for a round in flight: ``wait()`` before the update reads the
    buffer, ``done()`` after it has (both on the stream that is current at the call)."""

    def __init__(self, owner: "PeerGather", gi: int, b: int, producers: list[int], seqs: list[int]):
        self.owner, self.gi, self.b, self.producers, self.seqs = owner, gi, b, producers, seqs

    def wait(self) -> None:
        o = self.owner
        st = o.ops.current_stream()
        for r, s in zip(self.producers, self.seqs):
            if r != o.rank:
                o._wait(st, o.flag_addr(o.rank, self.gi, self.b, READY, r), s)

    def done(self) -> None:
        o = self.owner
        st = o.ops.current_stream()
        for r, s in zip(self.producers, self.seqs):
            if r != o.rank:
                o.ops.write32(st, o.flag_addr(r, self.gi, self.b, ACK, o.rank), s)


class PeerGather:
    """Collective constructor: every rank must call it with the same structure of buffers.

    ``buffer_addrs[g][b]`` is the device address of buffer ``b`` of numel group ``g`` (each
    ``[world_size, numel]``, rows contiguous) on this rank."""

    def __init__(self, rank: int, world_size: int, buffer_addrs: list[list[int]], ops,
                 param_addrs: list[list[int]] | None = None, timeout_s: float | None = None):
        self.rank, self.ws, self.ops = rank, world_size, ops
        self.timeout_s = timeout_s          # None: no deadline
        self.failed: str | None = None      # set by the watchdog; begin_step raises once it is
        self._inflight: list = []           # per unfinished step: [event, enqueue time, waits]
        self._waits: dict = {}              # flag address -> largest value this step waits for
        self._lock = threading.Lock()
        self._release_stream = None
        self.ngroups = len(buffer_addrs)
        self.nbuf = max(len(bl) for bl in buffer_addrs)
        self.buffer_ptrs = [list(bl) for bl in buffer_addrs]
        self.param_ptrs = [list(pl) for pl in (param_addrs or [])]
        # [group, buffer, kind, rank] use counters written by peers, then STEP[rank]
        self._step_flags = self.ngroups * self.nbuf * 2 * world_size
        self._flags_keepalive, flag_addr = ops.alloc_flags(self._step_flags + world_size)
        mine = {"flags": ops.export(flag_addr),
                "bufs": [[ops.export(a) for a in bl] for bl in buffer_addrs],
                "params": [[ops.export(a) for a in pl] for pl in self.param_ptrs]}
        everyone = ops.exchange(mine, world_size)
        self._flag_base = [0] * world_size
        self._buf_base = [None] * world_size
        self._param_base = [None] * world_size
        for r, info in enumerate(everyone):
            if r == rank:
                self._flag_base[r] = flag_addr
                self._buf_base[r] = self.buffer_ptrs
                self._param_base[r] = self.param_ptrs
            else:
                self._flag_base[r] = ops.import_(info["flags"])
                self._buf_base[r] = [[ops.import_(h) for h in hl] for hl in info["bufs"]]
                self._param_base[r] = [[ops.import_(h) for h in hl] for hl in info["params"]]
        self.step_no = 0
        self._step_waited: set = set()
        self._step_events: list = []
        ops.barrier()  # nobody writes a flag before everybody has zeroed and mapped them
        # peers in rotated order, so that the ranks of a box do not all push to rank 0 first
        # (FM_MUON_PEER_STREAMS=<n>: the copies to all peers share n streams instead of one each)
        n_streams = int(os.environ.get("FM_MUON_PEER_STREAMS", "0")) or (world_size - 1)
        pool = [ops.new_stream() for _ in range(max(1, min(n_streams, world_size - 1)))]
        self.streams = {(rank + i) % world_size: pool[(i - 1) % len(pool)]
                        for i in range(1, world_size)}
        self._release_stream = ops.new_stream()
        # host-side mirror of the use counters: seq[group][buffer][producer]
        self.seq = [[[0] * world_size for _ in range(self.nbuf)] for _ in range(self.ngroups)]
        # events of this rank's copies out of its slot, per (group, buffer)
        self.push_events = [[[] for _ in range(self.nbuf)] for _ in range(self.ngroups)]

    def flag_addr(self, holder: int, gi: int, b: int, kind: int, idx: int) -> int:
        return self._flag_base[holder] + 4 * ((((gi * self.nbuf + b) * 2 + kind) * self.ws) + idx)

    def step_flag_addr(self, holder: int, idx: int) -> int:
        return self._flag_base[holder] + 4 * (self._step_flags + idx)

    def _wait(self, stream, addr: int, value: int) -> None:
        """A flag wait of the current step, remembered so that the watchdog can release it."""
        with self._lock:
            if value > self._waits.get(addr, 0):
                self._waits[addr] = value
        self.ops.wait32_geq(stream, addr, value)

    def poll(self, now: float | None = None) -> bool:
        """Host-side deadline: True if the exchange is healthy.  Looks at the oldest step whose
        streams have not drained; past the deadline it writes every flag value that step (and any
        later one) waits for, so that the streams drain, and marks the exchange failed."""
        with self._lock:
            if self.failed:
                return False
            while self._inflight and self.ops.query(self._inflight[0][0]):
                self._inflight.pop(0)
            if not self._inflight or self.timeout_s is None:
                return True
            now = self.ops.now() if now is None else now
            if now - self._inflight[0][1] <= self.timeout_s:
                return True
            release: dict = {}
            for _, _, waits in self._inflight:
                for addr, value in waits.items():
                    release[addr] = max(value, release.get(addr, 0))
            for addr, value in self._waits.items():   # a step still being enqueued
                release[addr] = max(value, release.get(addr, 0))
            for addr, value in release.items():
                self.ops.write32(self._release_stream, addr, value)
            self.failed = (f"rank {self.rank}: a peer did not take part in the parameter exchange "
                           f"within {self.timeout_s} s; the waiting streams were released")
            self._inflight = []
            return False

    def check(self) -> None:
        if not self.poll():
            raise PeerExchangeError(self.failed)

    def begin_step(self, stream) -> None:
        """``stream`` carries whatever this rank did with its parameters before the step: once it
        gets here, peers may write updated parameters into this rank's replicas."""
        self.check()
        with self._lock:
            self._waits = {}
        self.step_no += 1
        self._step_waited = set()
        self._step_events = []
        for q in self.streams:
            self.ops.write32(stream, self.step_flag_addr(q, self.rank), self.step_no)

    def end_step(self, stream) -> None:
        """Copies out of this rank's parameters must finish before ``stream`` goes on (the next
        step rewrites them)."""
        for ev in self._step_events:
            self.ops.wait_event(stream, ev)
        self._step_events = []
        with self._lock:
            self._inflight.append([self.ops.record(stream), self.ops.now(), self._waits])
            self._waits = {}

    def param_addr(self, holder: int, gi: int, index: int) -> int:
        return self._param_base[holder][gi][index]

    def before_slot_write(self, gi: int, b: int, stream) -> None:
        """``stream`` is about to overwrite this rank's slot of buffer ``b``: earlier copies out
        of it must have finished."""
        for ev in self.push_events[gi][b]:
            self.ops.wait_event(stream, ev)
        self.push_events[gi][b] = []

    def publish(self, gi: int, b: int, slot_addr: int, nbytes: int, producers: list[int],
                param_index: int | None = None) -> PeerRound:
        """Called on the stream that produced the ``nbytes`` at ``slot_addr``.  By default they
        are this rank's row of buffer ``b`` and go to the same row of every peer's buffer ``b``;
        with ``param_index`` they are this rank's updated parameter ``param_index`` of group
        ``gi`` and go to the peers' replicas of that parameter."""
        seqs = []
        for r in producers:
            self.seq[gi][b][r] += 1
            seqs.append(self.seq[gi][b][r])
        if self.rank in producers:
            s = self.seq[gi][b][self.rank]
            ready = self.ops.record(self.ops.current_stream())
            for q, st in self.streams.items():
                self.ops.wait_event(st, ready)
                # q has consumed what I sent it in the previous use of buffer / flag row b
                self._wait(st, self.flag_addr(self.rank, gi, b, ACK, q), s - 1)
                if param_index is None:
                    dst = self._buf_base[q][gi][b] + self.rank * nbytes
                else:
                    if q not in self._step_waited:  # q has entered this step
                        self._wait(st, self.step_flag_addr(self.rank, q), self.step_no)
                        self._step_waited.add(q)
                    dst = self.param_addr(q, gi, param_index)
                self.ops.copy(st, dst, slot_addr, nbytes)
                self.ops.write32(st, self.flag_addr(q, gi, b, READY, self.rank), s)
                ev = self.ops.record(st)
                if param_index is None:  # copies out of the slot: it may not be rewritten before
                    self.push_events[gi][b].append(ev)
                self._step_events.append(ev)
        return PeerRound(self, gi, b, producers, seqs)

    def close(self) -> None:
        lib.fm_ipc_close_all()


class Watchdog(threading.Thread):
    """Calls ``PeerGather.poll`` once a second from a daemon thread, so that the deadline also
    fires while the main thread is blocked in a synchronisation on the parked streams."""

    def __init__(self, gather: PeerGather, device, period_s: float = 1.0):
        super().__init__(daemon=True, name="flash-muon-peer-watchdog")
        self.gather, self.device, self.period_s = gather, device, period_s
        self._halt = threading.Event()

    def run(self) -> None:
        if self.device is not None:
            torch.cuda.set_device(self.device)
        while not self._halt.wait(self.period_s):
            try:
                if not self.gather.poll():
                    return
            except Exception:  # noqa: BLE001 -- a dying context must not take the process along
                return

    def stop(self) -> None:
        self._halt.set()
