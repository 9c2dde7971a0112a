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


@pytest.mark.parametrize("ws", [1, 2, 3])
def test_muon_step_control_flow_over_gloo(ws, tmp_path, golden):
    """The product's ``Muon.step`` loop (ownership, double-buffered gather, update order) with its
    device hooks replaced by the oracle, run as ``ws`` CPU ranks: all ranks must end with the
    reference's parameters, bit for bit, and momentum state must live on the owner only."""
    port = _free_port()
    procs = []
    for r in range(ws):
        env = {**os.environ, "RANK": str(r), "WORLD_SIZE": str(ws), "MASTER_ADDR": "127.0.0.1",
               "MASTER_PORT": str(port), "OMP_NUM_THREADS": "2"}
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
                slots=[g.slots[j] for j in range(2 * g.lanes)], lanes=g.lanes, p_dtype=g.p_dtype,
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
    for got, group in zip(seen["groups"], opt.param_groups):
        ps = group["params"]
        flat += ps
        assert got["params"] == [p.data_ptr() for p in ps]
        assert got["grads"] == [p.grad.data_ptr() for p in ps]
        assert got["momentum"] == [opt.state[p]["momentum_buffer"].data_ptr() for p in ps]
        assert all(torch.count_nonzero(opt.state[p]["momentum_buffer"]) == 0 for p in ps)
        assert got["rows"] == [p.shape[0] for p in ps]
        assert got["cols"] == [p.numel() // p.shape[0] for p in ps]
        assert got["alphas"] == [-0.05 * max(1, p.size(-2) / p.size(-1)) ** 0.5 for p in ps]
        bufs, _ = opt._group_buffers(group)
        assert got["slots"] == [b.data_ptr() for b in bufs[:2 * got["lanes"]]]
        assert (got["p_dtype"], got["g_dtype"], got["nesterov"], got["ns_steps"]) == (0, 0, 0, 3)
        assert got["mu"] == 0.9 and got["decay"] == 1 - 0.05 * 0.1
    assert sorted(id(p) for p in flat) == sorted(id(p) for p in params)
    # conv filter: 16 x 72 view, scale of the kernel dims (3 / 3 -> 1)
    conv = [g for g in seen["groups"] if g["rows"] == [16]][0]
    assert conv["cols"] == [72] and conv["alphas"] == [-0.05]
    need = max(M.newtonschulz_workspace_bytes(r, c) for g in seen["groups"] for r, c in zip(g["rows"], g["cols"]))
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
