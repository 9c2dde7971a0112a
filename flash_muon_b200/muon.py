"""``Muon`` optimizer with the reference's constructor and ``step()`` (flash_muon/muon.py:36-110).

Same parameter grouping (by ``numel``), same round-robin ownership (rank ``r`` owns
``params[base + r]`` of every round), same order of operations and the same rounding points.
What differs is how the device work is issued:

* momentum + Nesterov is one fused kernel (``fm_momentum``) instead of two ``lerp_`` launches; it
  also leaves the partial sums of the Frobenius norm behind, so Newton-Schulz does not read the
  matrix once more for ``X.norm()`` (flash_muon/muon.py:23);
* Newton-Schulz is one C-ABI call whose last GEMM epilogue writes the flat update straight into
  this rank's slot of the gather buffer (no ``.flatten()`` copy, no staging tensor);
* matrices too small to fill the GPU (a 1024-wide product is 10 tiles for 74 CTA pairs) go
  through Newton-Schulz several at a time: every GEMM of the iteration is one launch over the
  whole batch (``fm_newtonschulz_batched``);
* rounds rotate through several gather buffers, so a round may fill its slot while older rounds
  are still being gathered and applied;
* the all-gather (flash_muon/muon.py:106-108) overlaps the next round's Newton-Schulz like the
  reference's ``async_op=True`` call.  Inside one box it is done by DMA copy engines pushing
  each finished slot into the peers' buffers, ordered by stream-side flags
  (``peer_gather.py``): NCCL's all-gather kernel cannot become resident next to the persistent
  GEMM kernels, a copy engine needs no SM.  ``FM_MUON_GATHER=nccl`` (or a failed peer set-up)
  selects the in-place NCCL all-gather through ``torch.distributed`` instead;
* weight decay + scaled update of all ``world_size`` parameters of a round is one multi-tensor
  kernel (``fm_update_multi``) instead of ``2 * world_size`` launches, enqueued on a second
  stream so that this HBM-bound pass runs under the tensor-core work of the following rounds;
* with the copy-engine exchange the OWNER applies decay + update to its replica and pushes the
  updated parameter into the replicas of its peers, instead of every rank gathering and applying
  every update.  That equals the reference only while all replicas hold the same bits before the
  step, which is checked once when the exchange is set up (a mismatch selects the gather of
  updates, as does ``FM_MUON_EXCHANGE=updates``).  The waits for what the peers push sit on a
  landing stream that only the end of the step joins, so none of a rank's own work waits for a
  peer inside a step;
* with ``world_size == 1`` and no hooks the whole step is one C call (``fm_muon_step``), which
  does the stream and event bookkeeping of the round loop inside the library
  (``FM_MUON_NATIVE=0`` keeps the loop below).

Numel groups are walked from the largest to the smallest (the reference walks a Python set,
flash_muon/muon.py:68; groups are independent): the last round of a step, whose exchange nothing
can hide, is then a small matrix.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import warnings

import torch
import torch.distributed as dist
from torch import Tensor

from ._lib import MuonGroup, check, current_stream_ptr, dtype_code, lib
from .ops import fast_newtonschulz, newtonschulz_workspace_bytes

__all__ = ["Muon"]

_NATIVE_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
_lib_flags_sumsq_ready = 2  # FM_NS_FAITHFUL | FM_NS_SUMSQ_READY


class Muon(torch.optim.Optimizer):
    """Muon - MomentUm Orthogonalized by Newton-schulz, data-parallel with round-robin ownership.

    Arguments mirror ``flash_muon.Muon`` (flash_muon/muon.py:60), including ``weight_decay`` as
    the third positional parameter:
        lr, weight_decay, momentum, nesterov, ns_steps, rank, world_size.
    With ``world_size == 1`` no process group is needed (the reference still calls the
    collective); otherwise the default ``torch.distributed`` group must be initialised with NCCL.

    ``param_groups`` carries exactly the reference's keys (``update_buffer``,
    ``update_buffer_views`` and the hyper-parameters), so ``state_dict()`` has the reference's
    layout and a checkpoint written by the reference loads (``load_state_dict`` matches numel
    groups by the width of their ``update_buffer``).  The additional gather buffers the rotation
    needs live outside ``param_groups`` and are never part of a checkpoint.
    """

    # Device of the gather buffers ("cuda" = the current CUDA device, flash_muon/muon.py:69).
    _buffer_device = "cuda"
    # Apply the decay + update of a finished round on a second stream, under the next GEMMs.
    _overlap_updates = True
    # Rounds rotate over several streams ("lanes"): the GEMM kernels are persistent and
    # statically scheduled, so a kernel's last wave leaves SMs idle; independent matrices in
    # flight on other streams take the idle SMs.  Two gather buffers per lane.
    _two_lanes = True          # False: a single compute stream
    _small_dim = 1536          # round loop: groups at most this narrow get 4 lanes
    _large_lanes = 2           # lanes of the other groups
    _max_batch = 16            # matrices per batched Newton-Schulz pass (single-call step)
    _rounds_per_pass = 0       # round loop: > 0 fixes the rounds per pass (tests), 0 = by plan
    # Host-side deadline of the copy-engine exchange: a peer that has not taken part in a step
    # this long after the step was enqueued is taken for gone (NCCL's watchdog default is of
    # the same order).  FM_MUON_PEER_TIMEOUT=<seconds> overrides it, 0 switches it off.
    _peer_timeout_s = 600.0

    def __init__(self, params, lr=0.02, weight_decay=0.01, momentum=0.95, nesterov=True,
                 ns_steps=5, rank=None, world_size=None):
        if (rank is None) or (world_size is None):
            raise Exception("world_size and rank params required, if you want to use this optimizer on a single GPU, pass rank=0 and world_size=1.")
        self.rank = rank
        self.world_size = world_size
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                        ns_steps=ns_steps)
        params: list[Tensor] = [*params]
        param_groups = []
        # one group per distinct numel (flash_muon/muon.py:68), largest first, the same order on
        # every rank whatever its hash seed
        for size in sorted({p.numel() for p in params}, reverse=True):
            b = torch.empty(world_size, size, dtype=torch.bfloat16, device=self._buffer_device)
            group = dict(params=[p for p in params if p.numel() == size],
                         update_buffer=b, update_buffer_views=[b[i] for i in range(world_size)])
            param_groups.append(group)
        super().__init__(param_groups, defaults)
        self._pool: dict = {}         # group index -> gather buffers beyond group["update_buffer"]
        self._workspaces: dict = {}   # lane -> Newton-Schulz scratch
        self._lane = 0
        self._peer = None             # PeerGather once set up; False if NCCL is to be used
        self._peer_recheck = False    # every rank went through load_state_dict: re-validate together
        self._push_params = True      # replicas were bit-identical when the exchange was set up
        self._watchdog = None

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _narrow(group) -> int:
        """Largest smaller-dimension among the matrices of a group (conv filters as size(0) x rest)."""
        return max(min(p.size(0), p.numel() // max(p.size(0), 1)) for p in group["params"])

    def _pairs(self) -> int:
        """CTA pairs of the device (one 256 x 256 tile in flight each)."""
        n = getattr(self, "_pairs_cached", None)
        if n is None:
            buf = self.param_groups[0]["update_buffer"]
            n = torch.cuda.get_device_properties(buf.device).multi_processor_count // 2 if buf.is_cuda else 74
            self._pairs_cached = n
        return n

    def _plan(self, group, native: bool) -> tuple[int, int]:
        """(lanes, batch) of a group.  The single-call step sends narrow matrices through
        Newton-Schulz several at a time -- as many as fill two waves of CTA pairs with the tiles
        of ``X @ X.T``: 14 matrices of 1024 rows, 4 of 2048 -- and matrices that fill the GPU alone
        (3072 rows or more) two at a time (tile lists twice as long leave a smaller share of a
        wave idle at their end, and half as many kernel boundaries), both over two lanes.  The
        round loop runs one matrix per round, narrow ones over four lanes."""
        narrow = self._narrow(group)
        if native:
            t = -(-narrow // 256)
            small = 2 * (self._pairs() // (t * (t + 1) // 2))
            batch = min(self._max_batch, small) if small >= 2 else 2
            forced = os.environ.get("FM_MUON_BATCH" if small >= 2 else "FM_MUON_BATCH_LARGE")
            if forced:
                batch = max(1, min(16, int(forced)))
            lanes = max(1, min(4, int(os.environ.get("FM_MUON_LANES", "2"))))
            return lanes, batch
        return (4 if narrow <= self._small_dim else self._large_lanes), 1

    def _loop_plan(self, group) -> tuple[int, int, int]:
        """(lanes, rounds per pass, gather buffers) of a group in the round loop.  The matrices a
        rank owns in consecutive rounds go through Newton-Schulz together like in the single-call
        step (at most eight rounds per pass); every round of a pass writes its own gather buffer,
        and two passes' worth of buffers let the next pass start while the rounds of the previous
        one are still being exchanged and applied."""
        lanes = self._plan(group, False)[0]
        rounds = -(-len(group["params"]) // self.world_size)
        per_pass = 1
        if self._rounds_per_pass > 0:
            per_pass = min(self._rounds_per_pass, rounds)
        elif self._overlap_updates and self._two_lanes and self._stock_device_ops() \
                and group["update_buffer"].is_cuda and os.environ.get("FM_MUON_LOOP_BATCH", "1") != "0":
            per_pass = max(1, min(8, self._plan(group, True)[1], rounds))
        if per_pass > 1:
            lanes = 2
        return lanes, per_pass, max(2 * lanes, 2 * per_pass)

    def _group_buffers(self, gi: int, count: int):
        """``count`` gather buffers of group ``gi`` in rotation order and their per-rank views: the
        group's own ``update_buffer`` first, the rest from a pool outside ``param_groups``."""
        group = self.param_groups[gi]
        first = group["update_buffer"]
        pool = self._pool.get(gi)
        if pool is None or any(b.shape != first.shape or b.device != first.device for b in pool):
            pool = self._pool[gi] = []
        while len(pool) < count - 1:
            pool.append(torch.empty_like(first))
        bufs = [first, *pool[:count - 1]]
        views = [group["update_buffer_views"]] + [[b[i] for i in range(self.world_size)]
                                                  for b in pool[:count - 1]]
        return bufs, views

    def _ns_workspace(self, rows: int, cols: int, device) -> Tensor:
        """Newton-Schulz scratch of the lane (stream) the current round runs on; grows to the
        largest matrix that lane has seen."""
        need = newtonschulz_workspace_bytes(rows, cols)
        ws = self._workspaces.get(self._lane)
        if ws is None or ws.numel() < need or ws.device != device:
            self._workspaces[self._lane] = ws = torch.empty(need, dtype=torch.uint8, device=device)
        return ws

    def _momentum(self, g: Tensor, buf: Tensor, momentum: float, nesterov: bool,
                  partials: int = 0) -> Tensor:
        # buf.lerp_(g, 1 - momentum); g.lerp_(buf, momentum)           (flash_muon/muon.py:99-100)
        # `partials`: device address that receives the partial sums of squares of the result
        assert g.is_contiguous(), "Muon gradients must be contiguous"
        check(lib.fm_momentum(g.data_ptr(), buf.data_ptr(), g.numel(), dtype_code(g.dtype),
                              float(momentum), 1 if nesterov else 0, partials or None,
                              current_stream_ptr(g.device)))
        return g if nesterov else buf

    def _orthogonalize(self, g: Tensor, out: Tensor, steps: int, sumsq_ready: bool = False) -> None:
        # fast_newtonschulz(g, steps).flatten() written into `out`     (flash_muon/muon.py:103)
        rows, cols = g.shape
        fast_newtonschulz(g, steps=steps, out=out.view(rows, cols),
                          workspace=self._ns_workspace(rows, cols, g.device), sumsq_ready=sumsq_ready)

    def _momentum_and_orthogonalize(self, items, group, fused: bool) -> None:
        """Momentum + Newton-Schulz of the matrices this rank owns in the rounds of one pass:
        ``items`` holds (gradient, momentum buffer, slot) per matrix.  Matrices that share their
        smaller and larger dimension go through ``fm_newtonschulz_batched`` together; anything
        else (one matrix, overridden device operations, mixed shapes) one at a time."""
        mom, nes, steps = group["momentum"], group["nesterov"], group["ns_steps"]
        dims = {(min(g.size(0), g.numel() // max(g.size(0), 1)), max(g.size(0), g.numel() // max(g.size(0), 1)),
                 g.dtype) for g, _, _ in items}
        native = fused and all(g.ndim in (2, 4) and g.numel() > 0 and g.dtype in _NATIVE_DTYPES
                               and g.is_contiguous() for g, _, _ in items)
        if not (native and len(items) > 1 and len(dims) == 1):
            for g, buf, slot in items:
                rows = g.size(0)
                cols = g.numel() // max(rows, 1)
                if native:
                    wsp = self._ns_workspace(rows, cols, g.device)
                    part = wsp.data_ptr() + int(lib.fm_ns_partials_offset(rows, cols))
                    g = self._momentum(g, buf, mom, nes, part)
                else:
                    g = self._momentum(g, buf, mom, nes)
                if g.ndim == 4:  # for the case of conv filters
                    g = g.view(len(g), -1)
                if native:
                    self._orthogonalize(g, slot, steps, True)
                else:
                    self._orthogonalize(g, slot, steps)
            return
        n = len(items)
        g0 = items[0][0]
        rows = [g.size(0) for g, _, _ in items]
        cols = [g.numel() // r for (g, _, _), r in zip(items, rows)]
        need = int(lib.fm_ns_batched_workspace_bytes(n, rows[0], cols[0]))
        wsp = self._workspaces.get(self._lane)
        if wsp is None or wsp.numel() < need or wsp.device != g0.device:
            self._workspaces[self._lane] = wsp = torch.empty(need, dtype=torch.uint8, device=g0.device)
        part = wsp.data_ptr() + int(lib.fm_ns_batched_partials_offset(n, rows[0], cols[0]))
        stride = 4 * int(lib.fm_norm_scratch_floats())
        srcs = [self._momentum(g, buf, mom, nes, part + j * stride) for j, (g, buf, _) in enumerate(items)]
        check(lib.fm_newtonschulz_batched(
            (ctypes.c_void_p * n)(*[t.data_ptr() for t in srcs]), (ctypes.c_int64 * n)(*rows),
            (ctypes.c_int64 * n)(*cols), n, dtype_code(g0.dtype), int(steps),
            (ctypes.c_void_p * n)(*[slot.data_ptr() for _, _, slot in items]), wsp.data_ptr(),
            wsp.numel(), _lib_flags_sumsq_ready, current_stream_ptr(g0.device)))

    def _all_gather(self, buffer: Tensor, slot: Tensor):
        # in place: `slot` is row `rank` of `buffer`                    (flash_muon/muon.py:108)
        return dist.all_gather_into_tensor(buffer, slot, async_op=True)

    # ------------------------------------------------------------------ checkpoints
    def load_state_dict(self, state_dict) -> None:
        """Loads a checkpoint of this class or of the reference (flash_muon/muon.py:68-73 writes
        one ``param_groups`` entry per numel with ``update_buffer`` of shape
        ``[world_size, numel]``, in the iteration order of a Python set).  Saved groups are matched
        to this optimizer's groups by that width, and gather buffers that come back on another
        device or for another world size are replaced."""
        saved = list(state_dict["param_groups"])
        ours = [g["params"][0].numel() for g in self.param_groups]
        if len(saved) == len(ours) and all(torch.is_tensor(g.get("update_buffer")) for g in saved):
            widths = [g["update_buffer"].size(-1) for g in saved]
            if widths != ours and sorted(widths) == sorted(ours):
                saved = [saved[widths.index(n)] for n in ours]
                state_dict = dict(state_dict, param_groups=saved)
        super().load_state_dict(state_dict)
        for gi, group in enumerate(self.param_groups):
            p0 = group["params"][0]
            want_dev = p0.device if p0.is_cuda else torch.device(self._buffer_device)
            b = group.get("update_buffer")
            ok = (torch.is_tensor(b) and b.dtype == torch.bfloat16 and b.is_contiguous()
                  and tuple(b.shape) == (self.world_size, p0.numel())
                  and b.device.type == want_dev.type
                  and (want_dev.index is None or b.device == want_dev))
            if not ok:
                group["update_buffer"] = b = torch.empty(self.world_size, p0.numel(),
                                                         dtype=torch.bfloat16, device=want_dev)
            group["update_buffer_views"] = [b[i] for i in range(self.world_size)]
        self._pool = {}
        self._peer_recheck = True

    def close(self) -> None:
        """Releases what the copy-engine exchange mapped from the peers (collective in spirit:
        call it on every rank, with no step in flight)."""
        if self._watchdog is not None:
            self._watchdog.stop()
            self._watchdog = None
        if self._peer:
            self._peer.close()
        self._peer = None

    # ------------------------------------------------------------------ exchange set-up
    def _replicas_identical(self, device) -> bool:
        """One all-reduce over a checksum of the raw bits of every parameter: the owner-pushes-
        the-parameter exchange equals the reference only if all replicas agree beforehand."""
        sums = []
        for group in self.param_groups:
            for p in group["params"]:
                bits = p.detach().reshape(-1).view(
                    {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[p.element_size()])
                sums.append(bits.sum(dtype=torch.int64))
        h = torch.stack(sums).to(device)
        lo, hi = h.clone(), h.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool(torch.equal(lo, hi))

    def _peer_pointers(self):
        bufs = [[b.data_ptr() for b in self._group_buffers(gi, self._loop_plan(g)[2])[0]]
                for gi, g in enumerate(self.param_groups)]
        pars = [[p.data_ptr() for p in g["params"]] for g in self.param_groups]
        return bufs, pars

    def _peer_gather(self):
        """The copy-engine all-gather, set up collectively on first use (None: use NCCL)."""
        if self._peer:
            # Addresses exported to the peers must still be the live ones.  Setting the exchange
            # up again is collective, so it may only be decided together: after load_state_dict
            # (which every rank calls) the ranks agree by all-reduce; a rank whose tensors moved
            # on its own cannot drag the others in and has to fail instead.
            bufs, pars = self._peer_pointers()
            stale = bufs != self._peer.buffer_ptrs or pars != self._peer.param_ptrs
            if self._peer_recheck:
                self._peer_recheck = False
                flag = torch.tensor([int(stale)], device=self.param_groups[0]["update_buffer"].device)
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                if int(flag.item()):
                    self.close()
            elif stale:
                raise RuntimeError(
                    "parameter or gather-buffer storage moved since the peer exchange was set up; "
                    "call load_state_dict (or close()) on every rank so that all ranks set it up again")
        if self._peer is None:
            self._peer = False
            self._peer_recheck = False
            want = os.environ.get("FM_MUON_GATHER", "peer") != "nccl"
            if want and self.world_size > 1 and self.param_groups[0]["update_buffer"].is_cuda:
                from .peer_gather import CudaOps, PeerGather, Watchdog
                ok, peer = 1, None
                device = self.param_groups[0]["update_buffer"].device
                timeout = float(os.environ.get("FM_MUON_PEER_TIMEOUT", self._peer_timeout_s or 0)) or None
                try:
                    bufs, pars = self._peer_pointers()
                    peer = PeerGather(self.rank, self.world_size, bufs, CudaOps(device),
                                      param_addrs=pars, timeout_s=timeout)
                except Exception as exc:  # same decision on every rank, taken below
                    ok = 0
                    warnings.warn(f"peer all-gather unavailable ({exc}); using NCCL")
                flag = torch.tensor([ok], device=device)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) == 1:
                    self._peer = peer
                    self._push_params = self._replicas_identical(device)
                    if not self._push_params:
                        warnings.warn("parameter replicas differ between ranks: every rank applies "
                                      "every update (as the reference does) instead of receiving "
                                      "the owner's updated parameter")
                    if timeout is not None:
                        self._watchdog = Watchdog(peer, device)
                        self._watchdog.start()
        return self._peer or None

    def _apply_updates(self, params_world, views, lr, weight_decay):
        # p *= 1 - lr*wd ; p += -lr*sqrt(max(1, rows/cols)) * g      (flash_muon/muon.py:87-89)
        stream_ptr = current_stream_ptr(views[0].device)
        by_dtype: dict = {}
        for p_world, g_world in zip(params_world, views):
            assert p_world.is_contiguous(), "Muon parameters must be contiguous"
            by_dtype.setdefault(p_world.dtype, []).append((p_world, g_world))
        decay = 1 - lr * weight_decay
        for dt, items in by_dtype.items():
            n = len(items)
            ptrs = (ctypes.c_void_p * n)(*[p.data_ptr() for p, _ in items])
            upds = (ctypes.c_void_p * n)(*[g.data_ptr() for _, g in items])
            nels = (ctypes.c_int64 * n)(*[p.numel() for p, _ in items])
            alphas = (ctypes.c_double * n)(
                *[-lr * max(1, p.size(-2) / p.size(-1)) ** 0.5 for p, _ in items])
            check(lib.fm_update_multi(ptrs, upds, nels, alphas, n, dtype_code(dt), decay,
                                      stream_ptr))

    # ------------------------------------------------------------------ step
    def _side_stream(self, device):
        st = getattr(self, "_side", None)
        if st is None or st.device != device:
            self._side = st = torch.cuda.Stream(device=device)
        return st

    def _land_stream(self, device):
        st = getattr(self, "_land", None)
        if st is None or st.device != device:
            self._land = st = torch.cuda.Stream(device=device)
        return st

    @torch.no_grad()
    def step(self, *, grad_ready=None, on_applied=None):
        """One optimizer step (flash_muon/muon.py:75-110; no closure, returns None).

        Two optional hooks let a caller stream tensors through the step instead of waiting for
        whole-model copies on either side of it:

        * ``grad_ready``: mapping parameter -> ``torch.cuda.Event``; the step waits for the event
          on its stream before it first touches that parameter's gradient (e.g. the event of a
          host-to-device copy still in flight).
        * ``on_applied(params, stream)``: called right after the decay + update of a round's
          parameters has been enqueued on ``stream``; work the callback enqueues behind an event
          of that stream (e.g. device-to-host copies) sees the updated parameters.
        """
        if len(self.param_groups) > 0 and self.param_groups[0]["update_buffer"].is_cuda:
            # kernels are launched on the device of the buffers, whatever device is current
            with torch.cuda.device(self.param_groups[0]["update_buffer"].device):
                return self._step(grad_ready, on_applied)
        return self._step(grad_ready, on_applied)

    def _stock_device_ops(self) -> bool:
        cls = type(self)
        return (cls._momentum is Muon._momentum and cls._orthogonalize is Muon._orthogonalize
                and cls._apply_updates is Muon._apply_updates)

    def _native_step(self) -> bool:
        """The whole step as one C call (``fm_muon_step``) when there is nothing for Python to do
        between rounds: one rank, no hooks, the stock device operations.  Returns False (having
        done nothing) when the round loop below has to run instead.  Same arithmetic per matrix
        as the loop, so the parameters come out bit-identical; what goes away is the per-round
        stream and event bookkeeping on the host, and narrow matrices share their launches."""
        if not (self._overlap_updates and self._two_lanes and self._stock_device_ops()
                and os.environ.get("FM_MUON_NATIVE", "1") != "0"):
            return False
        device = self.param_groups[0]["update_buffer"].device
        plan = []
        for gi, group in enumerate(self.param_groups):
            params = group["params"]
            if not params:
                continue
            p0 = params[0]
            for p in params:
                g = p.grad
                assert g is not None
                if (g.ndim not in (2, 4) or p.dtype != p0.dtype or g.dtype != p0.grad.dtype
                        or not g.is_contiguous() or not p.is_contiguous() or g.device != device
                        or p.dtype not in _NATIVE_DTYPES or g.dtype not in _NATIVE_DTYPES):
                    return False
            plan.append((gi, group))
        groups = (MuonGroup * max(len(plan), 1))()
        keep = []  # ctypes arrays must outlive the call
        need = 0
        nlanes = 1
        for gs, (gi, group) in zip(groups, plan):
            params = group["params"]
            n = len(params)
            lr, nes = group["lr"], group["nesterov"]
            bufs = []
            for p in params:
                state = self.state[p]
                if "momentum_buffer" not in state:
                    state["momentum_buffer"] = torch.zeros_like(p.grad)
                bufs.append(state["momentum_buffer"].data_ptr())
            rows = [p.grad.size(0) for p in params]
            cols = [p.grad.numel() // max(r, 1) for p, r in zip(params, rows)]
            lanes, batch = self._plan(group, True)
            batch = min(batch, n)
            nlanes = max(nlanes, lanes)
            need = max([need] + [int(lib.fm_ns_batched_workspace_bytes(batch, r, c))
                                 for r, c in set(zip(rows, cols))])
            slots, _ = self._group_buffers(gi, 2 * lanes * batch)
            arrays = (
                (ctypes.c_void_p * n)(*[p.data_ptr() for p in params]),
                (ctypes.c_void_p * n)(*[p.grad.data_ptr() for p in params]),
                (ctypes.c_void_p * n)(*bufs),
                (ctypes.c_int64 * n)(*rows),
                (ctypes.c_int64 * n)(*cols),
                (ctypes.c_double * n)(*[-lr * max(1, p.size(-2) / p.size(-1)) ** 0.5 for p in params]),
                (ctypes.c_void_p * len(slots))(*[b.data_ptr() for b in slots]),
            )
            keep.append(arrays)
            (gs.params, gs.grads, gs.momentum, gs.rows, gs.cols, gs.alphas, gs.slots) = arrays
            gs.count, gs.lanes, gs.batch = n, lanes, batch
            gs.p_dtype, gs.g_dtype = dtype_code(params[0].dtype), dtype_code(params[0].grad.dtype)
            gs.nesterov, gs.ns_steps = (1 if nes else 0), int(group["ns_steps"])
            gs.momentum_coef = float(group["momentum"])
            gs.decay = 1 - lr * group["weight_decay"]
        for lane in range(nlanes):
            ws = self._workspaces.get(lane)
            if ws is None or ws.numel() < need or ws.device != device:
                self._workspaces[lane] = torch.empty(need, dtype=torch.uint8, device=device)
        wptrs = (ctypes.c_void_p * nlanes)(*[self._workspaces[i].data_ptr() for i in range(nlanes)])
        wbytes = min(self._workspaces[i].numel() for i in range(nlanes))
        check(lib.fm_muon_step(groups, len(plan), wptrs, wbytes, current_stream_ptr(device)))
        return True

    def _step(self, grad_ready, on_applied):
        ws = self.world_size
        if (ws == 1 and grad_ready is None and on_applied is None and len(self.param_groups) > 0
                and self.param_groups[0]["update_buffer"].is_cuda and self._native_step()):
            return
        overlap = self._overlap_updates and len(self.param_groups) > 0 and \
            self.param_groups[0]["update_buffer"].is_cuda
        lanes = None
        if overlap:
            device = self.param_groups[0]["update_buffer"].device
            main = torch.cuda.current_stream(device)
            side = self._side_stream(device)
            land = self._land_stream(device)    # waits for what the peers push into this rank
            land.wait_stream(main)
            if self._two_lanes:
                extra = getattr(self, "_extra_lanes", None)
                if extra is None or extra[0].device != device:
                    self._extra_lanes = extra = [torch.cuda.Stream(device=device) for _ in range(3)]
                lanes = (main, *extra)
                for st in extra:
                    st.wait_stream(main)        # gradients produced on the caller's stream
        peer = self._peer_gather() if (ws > 1 and type(self)._all_gather is Muon._all_gather) else None
        # Owner-applies-and-pushes-the-parameter exchange (see peer_gather.py): needs the peer
        # set-up, the event-ordered update stream and replicas that agreed at set-up;
        # FM_MUON_EXCHANGE=updates keeps the reference's "gather the updates, every rank applies
        # all of them".
        push_params_ok = peer is not None and overlap and self._push_params and \
            os.environ.get("FM_MUON_EXCHANGE", "params") != "updates"
        # the fused momentum kernel can leave the partial sums of the norm for Newton-Schulz
        fused = self._stock_device_ops() and overlap
        if peer is not None:
            peer.begin_step(torch.cuda.current_stream(self.param_groups[0]["update_buffer"].device))
        for gi, group in enumerate(self.param_groups):
            nlanes, per_pass, nbuf_want = self._loop_plan(group)
            buffers, views = self._group_buffers(gi, nbuf_want)
            nbuf = len(buffers)
            params: list[Tensor] = group["params"]
            handle = None
            params_world = None
            prev = 0                   # which buffer the round in flight uses
            ns_done = [None] * nbuf    # per buffer: this rank's slot has been written
            upd_done = [None] * nbuf   # per buffer: its updates have been applied (side stream)
            # parameters wider than the bf16 updates would cost more link bytes than they save
            push_params = push_params_ok and all(p.element_size() <= 2 and p.is_contiguous()
                                                 for p in params)
            prev_base = 0

            def update_prev():
                if not overlap:
                    if handle is not None:
                        handle.wait()
                    self._apply_updates(params_world, views[prev], group["lr"], group["weight_decay"])
                    if hasattr(handle, "done"):
                        handle.done()
                    if on_applied is not None:
                        on_applied(params_world, torch.cuda.current_stream(views[prev][0].device))
                    return
                # The update only streams parameters through HBM; on its own stream it runs under
                # the tensor-core work of the following rounds instead of between them.
                if ns_done[prev] is not None:
                    side.wait_event(ns_done[prev])  # this rank's own slot is complete
                if push_params:
                    with torch.cuda.stream(side):
                        mine = prev_base + self.rank
                        if mine < len(params):  # apply my own update, then hand the result out
                            self._apply_updates([params[mine]], [views[prev][self.rank]],
                                                group["lr"], group["weight_decay"])
                        p_own = params[mine] if mine < len(params) else params[prev_base]
                        h = peer.publish(gi, prev, p_own.data_ptr(), p_own.numel() * p_own.element_size(),
                                         list(range(len(params_world))), param_index=mine)
                        # the slot is free again once my own update has read it: nothing of this
                        # rank's compute waits for a peer inside the step
                        upd_done[prev] = torch.cuda.Event()
                        upd_done[prev].record(side)
                    with torch.cuda.stream(land):
                        h.wait()            # the peers' parameters of this round have landed here
                        h.done()
                        if on_applied is not None:
                            land.wait_event(upd_done[prev])
                            on_applied(params_world, land)
                    return
                with torch.cuda.stream(side):
                    if handle is not None:
                        handle.wait()
                    self._apply_updates(params_world, views[prev], group["lr"], group["weight_decay"])
                    if hasattr(handle, "done"):
                        handle.done()  # peers may overwrite their slots of this buffer
                    if on_applied is not None:
                        on_applied(params_world, side)
                    upd_done[prev] = torch.cuda.Event()
                    upd_done[prev].record(side)

            bases = list(range(0, len(params), ws))
            for pass_idx, r0 in enumerate(range(0, len(bases), per_pass)):
                rounds = bases[r0: r0 + per_pass]
                # a pass travels on one lane; its rounds use consecutive gather buffers
                lane = lanes[pass_idx % nlanes] if lanes is not None else (main if overlap else None)
                self._lane = (pass_idx % nlanes) if lanes is not None else 0
                with (torch.cuda.stream(lane) if lanes is not None else contextlib.nullcontext()):
                    # -- this rank's matrices of the pass: momentum + Newton-Schulz into their slots
                    items, curs = [], []
                    for k, base_i in enumerate(rounds):
                        cur = (r0 + k) % nbuf
                        if overlap and upd_done[cur] is not None:
                            lane.wait_event(upd_done[cur])  # buffer `cur` is free to be overwritten
                            upd_done[cur] = None
                        if peer is not None:
                            peer.before_slot_write(gi, cur, torch.cuda.current_stream(views[cur][self.rank].device))
                        ns_done[cur] = None
                        if base_i + self.rank < len(params):
                            p = params[base_i + self.rank]
                            g = p.grad
                            assert g is not None
                            if grad_ready is not None and p in grad_ready:
                                torch.cuda.current_stream(g.device).wait_event(grad_ready[p])
                            state = self.state[p]
                            if "momentum_buffer" not in state:
                                state["momentum_buffer"] = torch.zeros_like(g)
                            items.append((g, state["momentum_buffer"], views[cur][self.rank]))
                            curs.append(cur)
                        # an idle rank contributes whatever its slot holds (muon.py:104-105)
                    if items:
                        self._momentum_and_orthogonalize(items, group, fused)
                        if overlap:
                            done = torch.cuda.Event()
                            done.record(lane)
                            for cur in curs:
                                ns_done[cur] = done
                    # -- the rounds of the pass, one exchange each, in the reference's order
                    for k, base_i in enumerate(rounds):
                        cur = (r0 + k) % nbuf
                        slot = views[cur][self.rank]
                        if params_world is not None:
                            update_prev()
                        if push_params:
                            handle = None  # published by update_prev, after the owner's update
                        elif peer is not None:
                            handle = peer.publish(gi, cur, slot.data_ptr(), slot.numel() * slot.element_size(),
                                                  list(range(min(ws, len(params) - base_i))))
                        elif ws > 1:
                            handle = self._all_gather(buffers[cur], slot)
                        params_world = params[base_i: base_i + ws]
                        prev = cur
                        prev_base = base_i
            if params_world is not None:
                update_prev()
        if overlap:
            main.wait_stream(side)  # the step's effects are ordered on the caller's stream
            main.wait_stream(land)
            if peer is not None:
                peer.end_step(main)
            if lanes is not None:
                for st in lanes[1:]:
                    main.wait_stream(st)
