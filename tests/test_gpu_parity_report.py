"""Where the bf16 noise floor of Newton-Schulz lies, measured: for BASELINE.json's configs[1]
(4096 x 4096) and the four Llama-3-8B shapes of configs[4], the relative Frobenius distance after
1, 3 and 5 steps between

* the product and the CPU oracle (exact-fp32 sums),
* the product and the same formulation in torch CUDA ops (cuBLAS products),
* the torch CUDA formulation and the CPU oracle -- two orders of the same fp32 sums with the same
  rounding points, i.e. the floor no implementation can be expected to beat.

The numbers are written to ``parity_report.json`` in the report folder (``conftest.REPORT_DIR``,
when it can be created) and bounded here: BASELINE.json's 2e-2 after 5 steps against the reference formulation on the same
device, and the product never further from the CPU oracle than 1.5 x the floor + 2e-3.
"""
import json
from pathlib import Path

import pytest
import torch

import flash_muon_b200 as fm
from flash_muon_b200 import _lib
from conftest import REPORT_DIR, rel_fro
from oracle import muon_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]
STEPS = (1, 3, 5)


def staged(G, native):
    """flash_muon/muon.py:13-33 with the oracle's building blocks, keeping the iterate after the
    steps of interest (one pass instead of three)."""
    a, b, c = O.NS_COEFFS
    X = G.bfloat16()
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    out = {}
    for s in range(1, max(STEPS) + 1):
        buf1 = O.matmul_transpose(X, native)
        buf2 = O.matmul_transpose(buf1, native)
        B = b * buf1 + c * buf2
        X = a * X + B @ X
        if s in STEPS:
            out[s] = (X.mT if tall else X).clone()
    return out


@pytest.mark.parametrize("shape", SHAPES)
def test_record_and_bound_the_distance_to_the_reference_formulation(shape):
    G = torch.randn(*shape, generator=torch.Generator().manual_seed(shape[0] + shape[1])).bfloat16()
    cpu = staged(G, native=False)
    gpu_ref = staged(G.to(DEV), native=True)
    rec = {"shape": list(shape), "steps": {}}
    for s in STEPS:
        mine = fm.fast_newtonschulz(G.to(DEV), s)
        rec["steps"][str(s)] = {
            "product_vs_cpu_oracle": rel_fro(mine, cpu[s]),
            "product_vs_torch_cuda": rel_fro(mine, gpu_ref[s]),
            "torch_cuda_vs_cpu_oracle": rel_fro(gpu_ref[s], cpu[s]),
        }
    _lib.device_status()
    out = REPORT_DIR
    try:
        out.mkdir(exist_ok=True)
        f = out / "parity_report.json"
        allrec = json.loads(f.read_text()) if f.exists() else {}
        allrec["x".join(map(str, shape))] = rec
        f.write_text(json.dumps(allrec, indent=1))
    except OSError:
        pass
    print(json.dumps(rec))
    for s in STEPS:
        r = rec["steps"][str(s)]
        floor = r["torch_cuda_vs_cpu_oracle"]
        assert r["product_vs_torch_cuda"] <= 2e-2, (shape, s, r)          # BASELINE.json's bar
        assert r["product_vs_cpu_oracle"] <= 1.5 * floor + 2e-3, (shape, s, r)
    assert rec["steps"]["5"]["product_vs_cpu_oracle"] <= 2.5e-2
