"""Generates ``tests/golden/reference_outputs.pt`` by running the REFERENCE (a checkout of
nil0x9/flash-muon) on CPU.

Run from the repo root:  ``python tests/golden/make_golden.py <path-to-flash-muon-checkout>``

The reference cannot execute as shipped without a GPU, so three documented shims are applied to
the imported modules (none of them touches the arithmetic under test except the first):

1. ``flash_muon.muon.matmul_transpose_assign`` (a Triton launch) is replaced by a CPU product with
   the kernel's semantics: fp32 accumulation, one cast (matmul_transpose_triton.py:53, :63).
2. ``torch.empty(..., device="cuda")`` in ``Muon.__init__`` (muon.py:69) allocates on the CPU.
3. ``dist.all_gather_into_tensor(out, inp)`` (muon.py:108) gets ``out.view(-1)``, because gloo
   rejects the stacked ``[world_size, n]`` output that NCCL accepts; with world_size 1 and no
   process group the gather is a copy.

The Triton kernel itself is exercised in fp32 under ``TRITON_INTERPRET=1`` (a child process), which
pins the tile mapping, masking and mirroring of ``mmt_kernel``.
"""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import torch

REF = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(os.environ.get("FLASH_MUON_REFERENCE", "reference"))
OUT = Path(__file__).resolve().parent / "reference_outputs.pt"
sys.path.insert(0, str(Path(__file__).resolve().parent))
from inputs import (MUON_HP, muon_case, ns_input, syrk_input, NS_SHAPES, SYRK_CASES)  # noqa: E402


def load_reference():
    sys.path.insert(0, str(REF))
    import flash_muon.muon as rmuon  # noqa: E402
    spec = importlib.util.spec_from_file_location("ref_benchmark", REF / "benchmark.py")
    rbench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rbench)
    return rmuon, rbench


def cpu_mmt_assign(d_in, d_out):
    d_out.copy_((d_in.float() @ d_in.float().T).to(d_in.dtype))


class _Done:
    def wait(self):
        return None


def run_muon_single(rmuon, steps: int):
    """Reference ``Muon`` at world_size 1 in this process."""
    import torch.distributed as dist
    params, grads_per_step = muon_case(steps)
    real_empty, real_gather = torch.empty, dist.all_gather_into_tensor

    def empty_cpu(*a, **k):
        if k.get("device") == "cuda":
            k["device"] = "cpu"
        return real_empty(*a, **k)

    def gather_copy(out, inp, async_op=False):
        out.view(-1).copy_(inp)
        return _Done()

    torch.empty, dist.all_gather_into_tensor = empty_cpu, gather_copy
    try:
        opt = rmuon.Muon(params, rank=0, world_size=1, **MUON_HP)
        for t in range(steps):
            for p, g in zip(params, grads_per_step[t]):
                p.grad = g.clone()
            opt.step()
    finally:
        torch.empty, dist.all_gather_into_tensor = real_empty, real_gather
    bufs = [opt.state[p]["momentum_buffer"].clone() for p in params]
    return [p.detach().clone() for p in params], bufs


_WS2_CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[4]); sys.path.insert(0, sys.argv[1])
import flash_muon.muon as rmuon
from inputs import MUON_HP, muon_case
rank = int(os.environ["RANK"]); ws = int(os.environ["WORLD_SIZE"]); steps = int(sys.argv[2])
dist.init_process_group("gloo", rank=rank, world_size=ws)
rmuon.matmul_transpose_assign = lambda i, o: o.copy_((i.float() @ i.float().T).to(i.dtype))
real_empty, real_gather = torch.empty, dist.all_gather_into_tensor
def empty_cpu(*a, **k):
    if k.get("device") == "cuda": k["device"] = "cpu"
    return real_empty(*a, **k)
torch.empty = empty_cpu
dist.all_gather_into_tensor = lambda out, inp, async_op=False: real_gather(out.view(-1), inp.contiguous(), async_op=async_op)
params, grads = muon_case(steps)
opt = rmuon.Muon(params, rank=rank, world_size=ws, **MUON_HP)
for t in range(steps):
    for p, g in zip(params, grads[t]): p.grad = g.clone()
    opt.step()
owned = {i: opt.state[p]["momentum_buffer"] for i, p in enumerate(params) if "momentum_buffer" in opt.state[p]}
torch.save({"params": [p.detach() for p in params], "owned": owned}, sys.argv[3] + f".rank{rank}")
dist.destroy_process_group()
'''


def run_muon_ws(ws: int, steps: int):
    """Reference ``Muon`` among ``ws`` CPU ranks over gloo (child processes via torchrun)."""
    with tempfile.TemporaryDirectory() as td:
        child = Path(td) / "child.py"
        child.write_text(_WS2_CHILD)
        out = str(Path(td) / "res")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ws}",
               "--master-addr", "127.0.0.1", "--master-port", "29671", str(child),
               str(Path(__file__).resolve().parent), str(steps), out, str(REF)]
        subprocess.run(cmd, check=True, env={**os.environ, "OMP_NUM_THREADS": "2"})
        return [torch.load(out + f".rank{r}") for r in range(ws)]


_INTERP_CHILD = r'''
import os, sys, torch
os.environ["TRITON_INTERPRET"] = "1"
sys.path.insert(0, sys.argv[3]); sys.path.insert(0, sys.argv[1])
from flash_muon.matmul_transpose_triton import mmt_kernel
from inputs import syrk_input
x = syrk_input(96, 80, torch.float32)
y = torch.full((96, 96), float("nan"))
mmt_kernel.fn[(9,)](x, y, 96, 80, x.stride(0), x.stride(1), y.stride(0), y.stride(1),
                    BLOCK_SIZE_M=32, BLOCK_SIZE_K=32, GROUP_SIZE_M=8)
torch.save(y, sys.argv[2])
'''


def run_triton_interpreter():
    with tempfile.TemporaryDirectory() as td:
        child = Path(td) / "child.py"
        child.write_text(_INTERP_CHILD)
        out = str(Path(td) / "y.pt")
        subprocess.run([sys.executable, str(child), str(Path(__file__).resolve().parent), out,
                        str(REF)], check=True)
        return torch.load(out)


def main():
    torch.set_num_threads(4)
    rmuon, rbench = load_reference()
    rmuon.matmul_transpose_assign = cpu_mmt_assign
    gold = {"torch_version": str(torch.__version__)}

    for (m, k, dt) in SYRK_CASES:
        x = syrk_input(m, k, dt)
        gold[f"torch_matmul_transpose/{m}x{k}/{dt}"] = rbench.torch_matmul_transpose(x)
    gold["mmt_kernel_interpreter/96x80/torch.float32"] = run_triton_interpreter()

    for shape in NS_SHAPES:
        for steps in (0, 1, 5):
            G = ns_input(*shape)
            gold[f"fast_newtonschulz/{shape[0]}x{shape[1]}/steps{steps}"] = \
                rmuon.fast_newtonschulz(G, steps=steps).contiguous()
        gold[f"torch_zeropower_via_newtonschulz5/{shape[0]}x{shape[1]}"] = \
            rbench.torch_zeropower_via_newtonschulz5(ns_input(*shape), steps=5).contiguous()

    steps = 2
    p1, b1 = run_muon_single(rmuon, steps)
    gold["muon_step/ws1/params"] = p1
    gold["muon_step/ws1/momentum"] = b1
    res2 = run_muon_ws(2, steps)
    gold["muon_step/ws2/params_rank0"] = res2[0]["params"]
    gold["muon_step/ws2/params_rank1"] = res2[1]["params"]
    gold["muon_step/ws2/owned"] = [sorted(r["owned"].keys()) for r in res2]
    res3 = run_muon_ws(3, steps)
    gold["muon_step/ws3/params_rank0"] = res3[0]["params"]
    gold["muon_step/ws3/owned"] = [sorted(r["owned"].keys()) for r in res3]

    torch.save(gold, OUT)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.1f} KiB, {len(gold)} entries)")


if __name__ == "__main__":
    main()
