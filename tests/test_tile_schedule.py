"""The static tile lists of the GEMM kernels, enumerated on the host.

The kernels are persistent: each CTA (or CTA pair) walks a list of output tiles computed from
its index, and the balanced tail cuts the last tiles by K blocks.  The arithmetic lives in
``flash_muon_b200/csrc/tile_schedule.cuh`` and compiles as plain C++, so the property the
reference gets from launching one program per tile pair
(flash_muon/matmul_transpose_triton.py:34-44: every upper-triangle tile exactly once) is checked
here exhaustively without a GPU by ``tests/schedule_check.cpp``.
"""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_every_tile_and_k_block_is_computed_exactly_once(tmp_path):
    exe = tmp_path / "schedule_check"
    build = subprocess.run(
        ["g++", "-O2", "-std=c++17", "-I", str(ROOT / "flash_muon_b200" / "csrc"),
         "-x", "c++", str(ROOT / "tests" / "schedule_check.cpp"), "-o", str(exe)],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr
    assert run.stdout.startswith("OK ")
