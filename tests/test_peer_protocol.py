"""The flag protocol of the copy-engine all-gather (flash_muon_b200/peer_gather.py) under a
simulated set of CUDA streams: every rank's streams are queues of operations that a scheduler
executes in random order whenever their waits are satisfied.  The simulation checks what no GPU
run can show exhaustively -- that for every interleaving the protocol neither deadlocks, nor lets
a consumer read a slot before it has landed, nor lets a producer overwrite a slot (its own or a
peer's copy of it) that someone still has to read."""
import random

import pytest

from flash_muon_b200.peer_gather import PeerExchangeError, PeerGather


class Sim:
    """Shared world: memory words, streams of all ranks, exchange board."""

    def __init__(self, world_size, seed):
        self.ws = world_size
        self.mem = {}            # address -> int (flags) or ("slot", producer, round) payloads
        self.streams = []        # all SimStream objects
        self.board = {}
        self.rng = random.Random(seed)
        self.next_addr = 1 << 20
        self.clock = 0.0         # host time the deadline of the exchange is measured against
        self.relaxed = False     # after a forced release the data invariants no longer hold
        self.replica_of = {}     # address of a parameter replica -> rank that holds it
        self.used = {}           # rank -> last step whose pre-step use of the replicas is over

    def alloc(self, nbytes):
        a = self.next_addr
        self.next_addr += (nbytes + 255) // 256 * 256 + 256
        return a

    def run(self, allow_stuck=False):
        while True:
            ready = [s for s in self.streams if s.queue and s.queue[0].ready()]
            if not ready:
                break
            s = self.rng.choice(ready)
            s.queue.pop(0).run()
        stuck = [s.name for s in self.streams if s.queue]
        assert allow_stuck or not stuck, f"deadlock: streams with pending work {stuck}"
        return stuck


class Op:
    def __init__(self, ready, run):
        self.ready, self.run = ready, run


class SimStream:
    def __init__(self, sim, name):
        self.sim, self.name, self.queue = sim, name, []
        sim.streams.append(self)

    def push(self, ready, run):
        self.queue.append(Op(ready, run))


class SimEvent:
    def __init__(self):
        self.done = False


class SimOps:
    """Same interface as peer_gather.CudaOps; addresses are keys of Sim.mem."""

    def __init__(self, sim, rank):
        self.sim, self.rank = sim, rank
        self.cur = SimStream(sim, f"r{rank}.main")

    def alloc_flags(self, n):
        a = self.sim.alloc(4 * n)
        for i in range(n):
            self.sim.mem[a + 4 * i] = 0
        return None, a

    def export(self, addr):
        return ("h", addr)

    def import_(self, exported):
        return exported[1]          # one address space in the simulation

    def exchange(self, obj, world_size):
        self.sim.board[self.rank] = obj
        return None                 # filled in by the test once every rank has posted

    def barrier(self):
        pass

    def new_stream(self):
        return SimStream(self.sim, f"r{self.rank}.s{len(self.sim.streams)}")

    def current_stream(self):
        return self.cur

    def record(self, stream):
        ev = SimEvent()
        stream.push(lambda: True, lambda: setattr(ev, "done", True))
        return ev

    def wait_event(self, stream, event):
        stream.push(lambda: event.done, lambda: None)

    def query(self, event):
        return event.done

    def now(self):
        return self.sim.clock

    def wait32_geq(self, stream, addr, value):
        stream.push(lambda: self.sim.mem[addr] >= value, lambda: None)

    def write32(self, stream, addr, value):
        stream.push(lambda: True, lambda: self.sim.mem.__setitem__(addr, value))

    def copy(self, stream, dst, src, nbytes):
        def run():
            payload = self.sim.mem[src]
            old = self.sim.mem.get(dst)
            if self.sim.relaxed:
                self.sim.mem[dst] = payload
                return
            if dst in self.sim.replica_of:
                # live model state: its holder must have entered the step the value belongs to
                q = self.sim.replica_of[dst]
                assert self.sim.used.get(q, -1) >= payload[2], \
                    f"replica of rank {q} overwritten with step {payload[2]} while still in use"
                self.sim.mem[dst] = payload
                return
            # the slot being overwritten must have been consumed by its holder
            assert old is None or old[3], f"slot {dst} overwritten before it was read: {old}"
            self.sim.mem[dst] = (payload[0], payload[1], payload[2], False)
        stream.push(lambda: True, run)


def build_world(ws, nbuf, numel_bytes, seed, nparams=0, timeout_s=None):
    sim = Sim(ws, seed)
    opses = [SimOps(sim, r) for r in range(ws)]
    bufs = [[sim.alloc(ws * numel_bytes) for _ in range(nbuf)] for _ in range(ws)]
    pars = [[sim.alloc(numel_bytes) for _ in range(nparams)] for _ in range(ws)]
    # PeerGather's constructor is collective: post every rank's exports first, then construct
    gathers = []
    # phase 1: flags + exports per rank (mimic the constructor's first half)
    posted = {}
    for r, ops in enumerate(opses):
        keep, fa = ops.alloc_flags(1 * nbuf * 2 * ws + ws)
        posted[r] = {"flags": ops.export(fa), "bufs": [[ops.export(a) for a in bufs[r]]],
                     "params": [[ops.export(a) for a in pars[r]]]}
        ops._prealloc = (keep, fa)
    for r, ops in enumerate(opses):
        ops.alloc_flags = lambda n, o=ops: o._prealloc
        ops.exchange = lambda obj, w, p=posted: [p[i] for i in range(w)]
        gathers.append(PeerGather(r, ws, [bufs[r]], ops, param_addrs=[pars[r]], timeout_s=timeout_s))
    if nparams:
        return sim, opses, bufs, gathers, pars
    return sim, opses, bufs, gathers


@pytest.mark.parametrize("ws,nbuf,lanes", [(2, 2, 1), (3, 4, 2), (4, 8, 4), (3, 2, 1)])
@pytest.mark.parametrize("seed", range(12))
def test_protocol_is_safe_under_any_interleaving(ws, nbuf, lanes, seed):
    drive(ws, nbuf, lanes, seed)


def test_simulation_catches_a_protocol_without_acknowledgements():
    """Sanity of the simulation itself: a producer that does not wait for ACK before pushing
    must be caught overwriting a slot that its peer has not read yet (for some interleaving)."""
    caught = 0
    for seed in range(40):
        try:
            drive(3, 2, 1, seed, drop_ack_wait=True)
        except AssertionError as exc:
            assert "overwritten before it was read" in str(exc) or "holds" in str(exc)
            caught += 1
    assert caught > 0


def drive(ws, nbuf, lanes, seed, drop_ack_wait=False):
    nbytes = 64
    rounds = 9
    nparams = rounds * ws - (ws - 1)          # last round has a single producer
    sim, opses, bufs, gathers = build_world(ws, nbuf, nbytes, seed)
    consumed = []
    if drop_ack_wait:
        for ops in opses:
            real = ops.wait32_geq
            # ACK waits are the ones issued on the per-peer push streams (name "r<k>.s<n>")
            ops.wait32_geq = lambda st, a, v, real=real: None if ".s" in st.name else real(st, a, v)

    for r in range(ws):                        # host program of rank r, as Muon.step issues it
        ops, pg = opses[r], gathers[r]
        main = ops.cur
        lane_streams = [main] + [SimStream(sim, f"r{r}.lane{i}") for i in range(1, lanes)]
        side = SimStream(sim, f"r{r}.side")
        upd_done = [None] * nbuf
        ns_done = [None] * nbuf
        pending = None                         # (handle, b, producers, round)
        for i in range(rounds):
            b = i % nbuf
            lane = lane_streams[b % lanes]
            producers = list(range(min(ws, nparams - i * ws)))
            ops.cur = lane
            if upd_done[b] is not None:
                ops.wait_event(lane, upd_done[b])
                upd_done[b] = None
            pg.before_slot_write(0, b, lane)
            slot = bufs[r][b] + r * nbytes
            if r in producers:
                def ns(slot=slot, i=i, r=r):
                    old = sim.mem.get(slot)
                    assert old is None or old[3], f"own slot rewritten before its update read it: {old}"
                    sim.mem[slot] = ("slot", r, i, False)
                lane.push(lambda: True, ns)
                ns_done[b] = ops.record(lane)
            else:
                ns_done[b] = None
            if pending is not None:
                h, pb, pprod, pround = pending
                if ns_done[pb] is not None:
                    ops.wait_event(side, ns_done[pb])
                ops.cur = side
                h.wait()

                def update(pb=pb, pprod=pprod, pround=pround, r=r):
                    for q in pprod:
                        a = bufs[r][pb] + q * nbytes
                        v = sim.mem.get(a)
                        assert v is not None and v[1] == q and v[2] == pround, \
                            f"rank {r} round {pround}: slot of {q} holds {v}"
                        sim.mem[a] = (v[0], v[1], v[2], True)
                    consumed.append((r, pround))
                side.push(lambda: True, update)
                h.done()
                upd_done[pb] = ops.record(side)
                ops.cur = lane
            handle = pg.publish(0, b, slot, nbytes, producers)
            pending = (handle, b, producers, i)
        h, pb, pprod, pround = pending
        if ns_done[pb] is not None:
            ops.wait_event(side, ns_done[pb])
        ops.cur = side
        h.wait()

        def last(pb=pb, pprod=pprod, pround=pround, r=r):
            for q in pprod:
                v = sim.mem.get(bufs[r][pb] + q * nbytes)
                assert v is not None and v[1] == q and v[2] == pround
            consumed.append((r, pround))
        side.push(lambda: True, last)
        h.done()

    sim.run()
    assert sorted(consumed) == sorted((r, i) for r in range(ws) for i in range(rounds))


@pytest.mark.parametrize("ws,nbuf,lanes", [(2, 2, 1), (3, 4, 2), (4, 8, 4)])
@pytest.mark.parametrize("seed", range(10))
def test_parameter_push_exchange_over_two_steps(ws, nbuf, lanes, seed):
    drive_params(ws, nbuf, lanes, seed)


@pytest.mark.parametrize("streams", ["1", "2"])
@pytest.mark.parametrize("seed", range(6))
def test_shared_copy_streams_are_safe_and_finish(streams, seed, monkeypatch):
    """FM_MUON_PEER_STREAMS: the copies to several peers share a stream, so a wait for one peer's
    acknowledgement also holds back the copies to the others.  Both exchanges must still finish
    (the simulator raises when streams are stuck) and stay safe."""
    monkeypatch.setenv("FM_MUON_PEER_STREAMS", streams)
    drive(4, 4, 2, seed)
    drive_params(4, 4, 2, seed)


def test_simulation_catches_pushes_that_do_not_wait_for_the_step_flag():
    caught = 0
    for seed in range(40):
        try:
            drive_params(3, 4, 2, seed, drop_step_wait=True)
        except AssertionError as exc:
            assert "while still in use" in str(exc) or "holds" in str(exc)
            caught += 1
    assert caught > 0


def drive_params(ws, nbuf, lanes, seed, drop_step_wait=False, absent=(), timeout_s=None, steps=2):
    """The owner applies the update and pushes the parameter into its peers' replicas.  Between
    two steps every rank 'uses' its replicas (as a forward/backward pass would): no replica may
    change before its rank has entered the next step, every replica must carry the owner's value
    of the step when the step ends."""
    nbytes = 64
    rounds = 5
    nparams = rounds * ws - 1                      # last round: one rank idle
    sim, opses, bufs, gathers, pars = build_world(ws, nbuf, nbytes, seed, nparams=nparams,
                                                  timeout_s=timeout_s)
    for r in range(ws):
        for i in range(nparams):
            sim.mem[pars[r][i]] = ("param", i % ws, -1, True)    # identical replicas, step -1
            sim.replica_of[pars[r][i]] = r

    for r in range(ws):
        ops, pg = opses[r], gathers[r]
        main = ops.cur
        lane_streams = [main] + [SimStream(sim, f"r{r}.lane{i}") for i in range(1, lanes)]
        side = SimStream(sim, f"r{r}.side")
        land = SimStream(sim, f"r{r}.land")
        for step in range(steps):
            if (r, step) in absent:      # this rank left before the step: it enqueues nothing more
                break
            # the training loop reads the replicas before the step (all must be of step-1)
            def use(r=r, step=step):
                if sim.relaxed:
                    return
                for i in range(nparams):
                    v = sim.mem[pars[r][i]]
                    assert v[2] == step - 1, f"rank {r} before step {step}: param {i} holds {v}"
                sim.used[r] = step
            main.push(lambda: True, use)
            ops.cur = main
            pg.begin_step(main)
            if drop_step_wait:
                pg._step_waited = set(range(ws))   # pretend every peer was already waited for
            for st in lane_streams[1:] + [land]:
                ops.wait_event(st, ops.record(main))
            upd_done = [None] * nbuf
            pending = None
            for i in range(rounds):
                b = i % nbuf
                lane = lane_streams[b % lanes]
                base = i * ws
                world = list(range(base, min(base + ws, nparams)))
                if upd_done[b] is not None:
                    ops.wait_event(lane, upd_done[b])
                    upd_done[b] = None
                mine = base + r
                ns_done = None
                if mine < nparams:
                    lane.push(lambda: True, lambda: None)          # momentum + Newton-Schulz
                    ns_done = ops.record(lane)
                if pending is not None:
                    _flush(sim, ops, pg, side, land, pars, r, nbytes, pending, upd_done, step)
                pending = (b, base, world, mine, ns_done)
            _flush(sim, ops, pg, side, land, pars, r, nbytes, pending, upd_done, step)
            # join: side stream, landing stream and pushes, then the step is over on main
            ops.wait_event(main, ops.record(side))
            ops.wait_event(main, ops.record(land))
            pg.end_step(main)

            def check_end(r=r, step=step):
                for i in range(nparams):
                    v = sim.mem[pars[r][i]]
                    assert v[1] == i % ws and v[2] == step, f"rank {r} after step {step}: param {i} holds {v}"
            if not absent:
                main.push(lambda: True, check_end)
    if absent:
        return sim, opses, gathers
    sim.run()


def _flush(sim, ops, pg, side, land, pars, r, nbytes, pending, upd_done, step):
    """One round as Muon.step enqueues it: own update and pushes on the side stream (the slot is
    free once the update has read it), waiting for the peers' pushes on the landing stream."""
    b, base, world, mine, ns_done = pending
    if ns_done is not None:
        ops.wait_event(side, ns_done)
    ops.cur = side
    nparams = len(pars[r])
    if mine < nparams:
        def own_update(a=pars[r][mine], r=r, step=step):
            sim.mem[a] = ("param", r, step, True)
        side.push(lambda: True, own_update)
    src = pars[r][mine] if mine < nparams else pars[r][base]
    h = pg.publish(0, b, src, nbytes, list(range(len(world))), param_index=mine)
    upd_done[b] = ops.record(side)
    ops.cur = land
    h.wait()
    h.done()
    ops.cur = side


@pytest.mark.parametrize("ws,nbuf,lanes", [(2, 2, 1), (3, 4, 2), (4, 8, 4)])
@pytest.mark.parametrize("seed", range(4))
def test_a_rank_that_leaves_between_steps_is_detected_by_the_deadline(ws, nbuf, lanes, seed):
    """Rank ws-1 takes part in step 0 and never enters step 1.  The streams of the others park on
    flags nobody will write; past the deadline ``poll`` writes the awaited values itself, every
    parked stream drains, the exchange is marked failed and the next step raises.  Before the
    deadline nothing is touched."""
    gone = ws - 1
    sim, opses, gathers = drive_params(ws, nbuf, lanes, seed, absent={(gone, 1)}, timeout_s=30.0)
    stuck = sim.run(allow_stuck=True)
    assert stuck and not any(name.startswith(f"r{gone}.") for name in stuck)
    live = [r for r in range(ws) if r != gone]
    sim.clock = 29.0
    for r in live:
        assert gathers[r].poll() is True and gathers[r].failed is None
    assert sim.run(allow_stuck=True) == stuck              # still parked, nothing released
    sim.clock = 31.0
    sim.relaxed = True                                     # released streams carry no valid data
    for r in live:
        assert gathers[r].poll() is False
        assert "did not take part" in gathers[r].failed
    assert sim.run(allow_stuck=True) == []                 # every stream drained
    for r in live:
        with pytest.raises(PeerExchangeError):
            gathers[r].begin_step(opses[r].cur)
    # the rank that left has nothing in flight and is not declared failed by its own deadline
    assert gathers[gone].poll() is True


def test_a_healthy_exchange_never_trips_the_deadline():
    sim, opses, gathers = drive_params(3, 4, 2, 1, absent={(99, 99)}, timeout_s=5.0)
    sim.clock = 1000.0                                      # long after: steps that finished do not count
    assert sim.run(allow_stuck=True) == []
    for g in gathers:
        assert g.poll() is True and g.failed is None


def test_a_producer_that_never_publishes_is_detected():
    """Gather-of-updates exchange: rank 1 stops publishing after its second round (an exception in
    its step).  Its peers wait for READY flags that never come; the deadline releases them."""
    ws, nbuf, nbytes = 3, 2, 64
    sim, opses, bufs, gathers = build_world(ws, nbuf, nbytes, seed=3, timeout_s=10.0)
    for r in range(ws):
        ops, pg = opses[r], gathers[r]
        main, side = ops.cur, SimStream(sim, f"r{r}.side")
        pg.begin_step(main)
        pending = None

        def consume(h, ops=ops, side=side, main=main, r=r):
            ops.cur = side
            h.wait()

            def read(r=r, b=h.b):
                for q in range(ws):
                    a = bufs[r][b] + q * nbytes
                    v = sim.mem.get(a)
                    if v is not None:
                        sim.mem[a] = (v[0], v[1], v[2], True)
            side.push(lambda: True, read)
            h.done()
            ops.cur = main

        for i in range(4):
            if r == 1 and i == 2:
                break                                       # rank 1 dies here
            b = i % nbuf
            ops.cur = main
            pg.before_slot_write(0, b, main)
            slot = bufs[r][b] + r * nbytes
            main.push(lambda: True, lambda slot=slot, r=r, i=i: sim.mem.__setitem__(slot, ("slot", r, i, True)))
            if pending is not None:
                consume(pending)
            pending = pg.publish(0, b, slot, nbytes, list(range(ws)))
        if r != 1:
            consume(pending)
            ops.wait_event(main, ops.record(side))
            pg.end_step(main)
    assert sim.run(allow_stuck=True)
    sim.clock = 11.0
    sim.relaxed = True
    assert gathers[0].poll() is False and gathers[2].poll() is False
    assert [s for s in sim.run(allow_stuck=True) if not s.startswith("r1.")] == []
