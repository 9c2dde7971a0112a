"""The parts of bench.py that run without a GPU: the reference arm's JSON line and the FLOP /
byte bookkeeping the roofline figures are computed from."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600,
                         env={**os.environ, "FM_BENCH_CPU_SAMPLE": "small"})  # two matrices, not a layer
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "muon_step_ms" and d["unit"] == "ms"
    assert d["higher_is_better"] is False and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert "scaled" in d["cpu_baseline"]["sample"] and d["cpu_baseline"]["sample_seconds"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_default_cpu_sample_is_one_whole_layer():
    shapes = bench.cpu_sample_shapes()
    assert shapes == list(bench.LLAMA_LAYER) and len(shapes) == 7
    _, full = bench.full_step_flops()
    fl = sum(bench.ns_flops(*s)[1] for s in shapes)
    assert abs(full / fl - bench.N_LAYERS) < 1e-9          # the extrapolation is exactly x32
    assert "x32.0" in bench.describe_sample(shapes, full / fl)


def test_flop_bookkeeping_of_the_llama_shaped_step():
    alg, full = bench.full_step_flops()
    assert abs(alg - 4.7181e14) / 4.7181e14 < 1e-3      # algorithmic FLOPs of one Llama-shaped step
    assert abs(full - 6.6589e14) / 6.6589e14 < 1e-3     # cuBLAS-equivalent FLOPs
    a, f = bench.ns_flops(4096, 4096)
    assert abs(a - 1.3746e12) / 1.3746e12 < 1e-3 and abs(f - 2.0616e12) / 2.0616e12 < 1e-3
    assert sum(r * c for r, c in bench.LLAMA_LAYER) * bench.N_LAYERS == 6979321856


def test_replica_checksum_sees_single_bit_and_position_changes():
    import torch
    g = torch.Generator().manual_seed(0)
    params = [torch.randn(300, 500, generator=g).bfloat16(), torch.randn(64, 64, generator=g)]
    base = bench.replica_checksum(params)
    assert torch.equal(base, bench.replica_checksum([p.clone() for p in params]))
    flipped = [p.clone() for p in params]
    flipped[0].view(torch.int16)[17, 33] ^= 1
    assert not torch.equal(base, bench.replica_checksum(flipped))
    swapped = [p.clone() for p in params]
    a, b = swapped[0].view(-1)[5].clone(), swapped[0].view(-1)[70000].clone()
    swapped[0].view(-1)[5], swapped[0].view(-1)[70000] = b, a
    assert a != b and not torch.equal(base, bench.replica_checksum(swapped))


def test_recorded_traffic_is_only_reported_for_the_sources_it_was_captured_from(monkeypatch):
    """`roofline.traffic` comes from a tracked capture stamped with a hash of the kernel sources:
    reported while the hash matches and no tuning switch is set, null otherwise."""
    rec = json.loads((ROOT / "profiles" / "gemm_tc2_kernel_syrk_traffic.json").read_text())
    assert rec["shape"] == [8192, 8192] and rec["dram_bytes_read"] > 0 and rec["dram_bytes_written"] > 0
    for v in ("FM_GEMM_IMPL", "FM_GEMM_BN", "FM_GEMM_STAGES", "FM_GEMM_BALANCE", "FM_GEMM_STRIP", "FM_PDL"):
        monkeypatch.delenv(v, raising=False)
    traffic, source = bench.recorded_traffic(8192, 8192)
    if rec["source_hash"] == bench.gemm_source_hash():
        assert traffic == rec["dram_bytes_read"] + rec["dram_bytes_written"] and rec["commit"] in source
    else:
        assert traffic is None and "predates" in source
    assert bench.recorded_traffic(4096, 4096)[0] is None
    monkeypatch.setenv("FM_GEMM_STRIP", "0")
    assert bench.recorded_traffic(8192, 8192)[0] is None
    monkeypatch.setattr(bench, "gemm_source_hash", lambda: "0" * 16)
    monkeypatch.delenv("FM_GEMM_STRIP")
    assert bench.recorded_traffic(8192, 8192)[0] is None
