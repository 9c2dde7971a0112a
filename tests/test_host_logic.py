"""Host-side behaviour of the operator interface that needs no GPU: the reference's error
behaviour (flash_muon/matmul_transpose_triton.py:79-86, flash_muon/muon.py:61-62) and the
round-robin ``Muon.step`` control flow among CPU ranks over gloo."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import flash_muon_b200 as fm

ROOT = Path(__file__).resolve().parent.parent


def test_public_names_match_reference():
    for name in ("matmul_transpose", "matmul_transpose_assign", "fast_newtonschulz", "Muon"):
        assert hasattr(fm, name)


def test_cpu_tensor_raises_like_reference():
    x = torch.randn(8, 8)
    with pytest.raises(AssertionError, match="Input `d_in` must be a CUDA tensor"):
        fm.matmul_transpose(x)
    with pytest.raises(AssertionError, match="must be a CUDA tensor"):
        fm.matmul_transpose_assign(x, torch.empty(8, 8))
    with pytest.raises(AssertionError):
        fm.fast_newtonschulz(x)
    with pytest.raises(AssertionError):
        fm.fast_newtonschulz(torch.randn(8))


def test_muon_requires_rank_and_world_size():
    p = [torch.nn.Parameter(torch.randn(4, 4))]
    with pytest.raises(Exception, match="world_size and rank params required"):
        fm.Muon(p)
    with pytest.raises(Exception, match="world_size and rank params required"):
        fm.Muon(p, rank=0)


def test_muon_signature_matches_reference():
    import inspect
    sig = inspect.signature(fm.Muon.__init__)
    names = list(sig.parameters)[1:]
    assert names == ["params", "lr", "weight_decay", "momentum", "nesterov", "ns_steps", "rank",
                     "world_size"]
    d = {k: v.default for k, v in sig.parameters.items()}
    assert (d["lr"], d["weight_decay"], d["momentum"], d["nesterov"], d["ns_steps"]) == \
        (0.02, 0.01, 0.95, True, 5)
    # step() takes no positional argument, like the reference; the two extras are keyword-only
    step = inspect.signature(fm.Muon.step).parameters
    assert list(step) == ["self", "grad_ready", "on_applied"]
    assert all(step[k].kind is inspect.Parameter.KEYWORD_ONLY and step[k].default is None
               for k in ("grad_ready", "on_applied"))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("ws,per_pass", [(1, 0), (2, 0), (3, 0), (1, 3), (2, 2), (3, 4)])
def test_muon_step_control_flow_over_gloo(ws, per_pass, tmp_path, golden):
    """The product's ``Muon.step`` loop (ownership, double-buffered gather, update order) with its
    device hooks replaced by the oracle, run as ``ws`` CPU ranks: all ranks must end with the
    reference's parameters, bit for bit, and momentum state must live on the owner only.
    ``per_pass`` > 0 makes a rank compute the matrices it owns in that many consecutive rounds
    before the first of those rounds is exchanged (what the loop does on the GPU when it sends
    them through Newton-Schulz together)."""
    port = _free_port()
    procs = []
    for r in range(ws):
        env = {**os.environ, "RANK": str(r), "WORLD_SIZE": str(ws), "MASTER_ADDR": "127.0.0.1",
               "MASTER_PORT": str(port), "OMP_NUM_THREADS": "2", "TEST_ROUNDS_PER_PASS": str(per_pass)}
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "gloo_muon_child.py"),
                                       str(tmp_path / "out")], env=env))
    for p in procs:
        assert p.wait(timeout=300) == 0
    key = {1: "muon_step/ws1/params", 2: "muon_step/ws2/params_rank0", 3: "muon_step/ws3/params_rank0"}[ws]
    for r in range(ws):
        res = torch.load(str(tmp_path / "out") + f".rank{r}")
        for p, ref in zip(res["params"], golden[key]):
            assert torch.equal(p, ref)
        if ws > 1:
            assert res["owned"] == golden[f"muon_step/ws{ws}/owned"][r]


def test_whole_step_call_receives_the_reference_step_arguments(monkeypatch):
    """What ``Muon.step`` hands to ``fm_muon_step`` at world_size 1: every parameter once, grouped
    by numel in the optimizer's order, with the 2-D view of conv filters (flash_muon/muon.py:101-
    102), the update scale of the ORIGINAL shape (muon.py:89), the decay of muon.py:87 and the
    momentum buffers created on first use (muon.py:96-97).  The C call itself is replaced by a
    recorder, so this runs without a GPU."""
    import ctypes
    from flash_muon_b200 import muon as M

    class CpuMuon(fm.Muon):
        _buffer_device = "cpu"

    torch.manual_seed(0)
    shapes = [(64, 32), (32, 64), (16, 8, 3, 3), (48, 48), (64, 32)]
    params = [torch.nn.Parameter(torch.randn(*s).bfloat16()) for s in shapes]
    for p in params:
        p.grad = torch.randn(*p.shape).bfloat16()
    opt = CpuMuon(params, lr=0.05, weight_decay=0.1, momentum=0.9, nesterov=False, ns_steps=3,
                  rank=0, world_size=1)
    seen = {}

    def recorder(groups, ngroups, wptrs, wbytes, stream):
        seen["ngroups"] = ngroups
        seen["groups"] = []
        for i in range(ngroups):
            g = groups[i]
            n = g.count
            seen["groups"].append(dict(
                params=[g.params[j] for j in range(n)], grads=[g.grads[j] for j in range(n)],
                momentum=[g.momentum[j] for j in range(n)], rows=[g.rows[j] for j in range(n)],
                cols=[g.cols[j] for j in range(n)], alphas=[g.alphas[j] for j in range(n)],
                slots=[g.slots[j] for j in range(2 * g.lanes * g.batch)], lanes=g.lanes,
                batch=g.batch, p_dtype=g.p_dtype,
                g_dtype=g.g_dtype, nesterov=g.nesterov, ns_steps=g.ns_steps, mu=g.momentum_coef,
                decay=g.decay))
        seen["wbytes"] = wbytes
        seen["lanes_with_workspace"] = [wptrs[i] for i in range(max(g["lanes"] for g in seen["groups"]))]
        return 0

    monkeypatch.setattr(M.lib, "fm_muon_step", recorder)
    monkeypatch.setattr(M, "current_stream_ptr", lambda device: None)
    assert opt._native_step() is True
    assert seen["ngroups"] == len(opt.param_groups) == 3
    flat = []
    # groups are walked from the largest numel down
    assert [g["params"][0].numel() for g in opt.param_groups] == [48 * 48, 64 * 32, 16 * 72]
    for gi, (got, group) in enumerate(zip(seen["groups"], opt.param_groups)):
        ps = group["params"]
        flat += ps
        assert got["params"] == [p.data_ptr() for p in ps]
        assert got["grads"] == [p.grad.data_ptr() for p in ps]
        assert got["momentum"] == [opt.state[p]["momentum_buffer"].data_ptr() for p in ps]
        assert all(torch.count_nonzero(opt.state[p]["momentum_buffer"]) == 0 for p in ps)
        assert got["rows"] == [p.shape[0] for p in ps]
        assert got["cols"] == [p.numel() // p.shape[0] for p in ps]
        assert got["alphas"] == [-0.05 * max(1, p.size(-2) / p.size(-1)) ** 0.5 for p in ps]
        # narrow matrices share a Newton-Schulz pass: as many as the group holds, 16 at most
        assert got["lanes"] == 2 and got["batch"] == min(len(ps), 16)
        bufs, _ = opt._group_buffers(gi, 2 * got["lanes"] * got["batch"])
        assert got["slots"] == [b.data_ptr() for b in bufs]
        assert len(set(got["slots"])) == len(got["slots"]) and bufs[0] is group["update_buffer"]
        assert (got["p_dtype"], got["g_dtype"], got["nesterov"], got["ns_steps"]) == (0, 0, 0, 3)
        assert got["mu"] == 0.9 and got["decay"] == 1 - 0.05 * 0.1
    assert sorted(id(p) for p in flat) == sorted(id(p) for p in params)
    # conv filter: 16 x 72 view, scale of the kernel dims (3 / 3 -> 1)
    conv = [g for g in seen["groups"] if g["rows"] == [16]][0]
    assert conv["cols"] == [72] and conv["alphas"] == [-0.05]
    need = max(M.lib.fm_ns_batched_workspace_bytes(g["batch"], r, c)
               for g in seen["groups"] for r, c in zip(g["rows"], g["cols"]))
    assert seen["wbytes"] >= need and all(seen["lanes_with_workspace"])

    # anything the C call cannot express goes back to the round loop: strided gradients,
    # overridden device operations, the environment switch
    monkeypatch.setenv("FM_MUON_NATIVE", "0")
    assert opt._native_step() is False
    monkeypatch.delenv("FM_MUON_NATIVE")
    params[3].grad = torch.randn(48, 48).bfloat16().t()       # not contiguous
    assert opt._native_step() is False
    params[3].grad = torch.randn(48, 48).bfloat16()
    assert opt._native_step() is True

    class Hooked(CpuMuon):
        def _momentum(self, g, buf, momentum, nesterov):
            return g
    assert Hooked(params, rank=0, world_size=1)._native_step() is False
    params[1].grad = None
    with pytest.raises(AssertionError):
        opt._native_step()


REFERENCE_GROUP_KEYS = {"params", "lr", "weight_decay", "momentum", "nesterov", "ns_steps",
                        "update_buffer", "update_buffer_views"}


def reference_format(sd):
    """The layout flash_muon/muon.py:68-73 gives a checkpoint: one group per numel in another
    order than this optimizer's (a Python set there, ascending here), parameter ids numbered along
    that order, the gather buffer as a CPU tensor (as ``torch.load(map_location="cpu")`` leaves it)."""
    groups = sorted((dict(g) for g in sd["param_groups"]), key=lambda g: g["update_buffer"].size(-1))
    renumber, nxt = {}, 0
    for g in groups:
        ids = []
        for pid in g["params"]:
            renumber[pid] = nxt
            ids.append(nxt)
            nxt += 1
        g["params"] = ids
        b = g["update_buffer"].cpu().clone()
        g["update_buffer"], g["update_buffer_views"] = b, [b[i] for i in range(b.size(0))]
    # state_dict() hands out the live tensors; a checkpoint read from disk would not alias them
    state = {renumber[k]: {n: (t.clone() if torch.is_tensor(t) else t) for n, t in v.items()}
             for k, v in sd["state"].items()}
    return {"state": state, "param_groups": groups}


def test_state_dict_has_the_reference_layout_and_reference_checkpoints_load():
    from oracle import muon_oracle as O

    class CpuMuon(fm.Muon):
        _buffer_device = "cpu"

        def _momentum(self, g, buf, momentum, nesterov):
            return O.momentum_update(g, buf, momentum, nesterov)

        def _orthogonalize(self, g, out, steps):
            out.copy_(O.newtonschulz(g, steps=steps).flatten())

        def _apply_updates(self, params_world, views, lr, weight_decay):
            for p, g in zip(params_world, views):
                O.apply_update(p, g, lr, weight_decay)

    torch.manual_seed(1)
    shapes = [(64, 32), (32, 64), (16, 8, 3, 3), (48, 48), (64, 32), (24, 48)]

    def make():
        g = torch.Generator().manual_seed(5)
        ps = [torch.nn.Parameter((torch.randn(*s, generator=g) * 0.02).bfloat16()) for s in shapes]
        for p in ps:
            p.grad = (torch.randn(*p.shape, generator=g) * 1e-3).bfloat16()
        return ps

    a = make()
    opt = CpuMuon(a, rank=0, world_size=1)
    opt.step()
    sd = opt.state_dict()
    for g in sd["param_groups"]:
        assert set(g) == REFERENCE_GROUP_KEYS            # nothing beyond what the reference saves
    ref_sd = reference_format(sd)
    assert [g["update_buffer"].size(-1) for g in ref_sd["param_groups"]] != \
        [g["update_buffer"].size(-1) for g in sd["param_groups"]]

    b = make()
    opt2 = CpuMuon(b, rank=0, world_size=1)
    opt2.load_state_dict(ref_sd)
    for pa, pb in zip(a, b):                             # every momentum buffer on its own parameter
        assert torch.equal(opt.state[pa]["momentum_buffer"], opt2.state[pb]["momentum_buffer"])
    for g in opt2.param_groups:
        n = g["params"][0].numel()
        assert tuple(g["update_buffer"].shape) == (1, n) and all(p.numel() == n for p in g["params"])
    # and the next step continues as if nothing had happened
    for pa, pb in zip(a, b):
        pb.data.copy_(pa.data)
        pa.grad = pb.grad.clone()
    opt.step()
    opt2.step()
    for pa, pb in zip(a, b):
        assert torch.equal(pa, pb)
    # a checkpoint taken at another world size brings a gather buffer of the wrong height
    wide = reference_format(opt.state_dict())
    for g in wide["param_groups"]:
        t = g["update_buffer"].repeat(4, 1)
        g["update_buffer"], g["update_buffer_views"] = t, [t[i] for i in range(4)]
    opt2.load_state_dict(wide)
    assert all(tuple(g["update_buffer"].shape) == (1, g["params"][0].numel()) for g in opt2.param_groups)
    opt2.step()


def test_matrices_per_pass_of_the_benchmark_shapes(monkeypatch):
    """How many matrices of a numel group share one Newton-Schulz pass in the single-call step:
    as many as fill two waves of 74 CTA pairs with the tiles of X @ X.T for narrow matrices
    (1024 rows: 10 tiles each -> 14), two at a time for matrices that fill the GPU alone, two
    lanes each; the environment overrides are honoured and clamped."""
    for name in ("FM_MUON_BATCH", "FM_MUON_BATCH_LARGE", "FM_MUON_LANES"):
        monkeypatch.delenv(name, raising=False)
    shapes = [(1024, 1024), (4096, 1024), (1024, 4096), (2048, 2048), (4096, 4096), (4096, 14336)]
    params = [torch.nn.Parameter(torch.empty(*s, dtype=torch.bfloat16)) for s in shapes]

    class CpuMuon(fm.Muon):
        _buffer_device = "cpu"      # the reference allocates on "cuda" (flash_muon/muon.py:69)

    opt = CpuMuon(params, rank=0, world_size=1)
    plans = {}
    for group in opt.param_groups:
        narrow = opt._narrow(group)
        plans[narrow] = opt._plan(group, True)
        assert opt._plan(group, False)[1] == 1            # the round loop's own plan: one per round
    assert plans[1024] == (2, 14)
    assert plans[2048] == (2, 4)
    assert plans[4096] == (2, 2)
    monkeypatch.setenv("FM_MUON_BATCH", "99")
    monkeypatch.setenv("FM_MUON_BATCH_LARGE", "1")
    monkeypatch.setenv("FM_MUON_LANES", "3")
    for group in opt.param_groups:
        lanes, batch = opt._plan(group, True)
        assert lanes == 3
        assert batch == (16 if opt._narrow(group) <= 2048 else 1)
