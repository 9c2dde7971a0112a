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
