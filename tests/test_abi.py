"""The C-ABI library loads and exports every symbol ``include/flash_muon_b200.h`` declares
(no compute calls: this runs without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "flash_muon_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fm_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path_entry_points():
    syms = declared_symbols()
    for name in ("fm_syrk", "fm_newtonschulz", "fm_newtonschulz_batched", "fm_momentum",
                 "fm_update_multi", "fm_gemm_nt", "fm_syrk_poly", "fm_normalize",
                 "fm_ns_workspace_bytes", "fm_device_status", "fm_muon_step"):
        assert name in syms


def test_library_builds_in_tree():
    import importlib.util
    spec = importlib.util.spec_from_file_location("_fm_build", ROOT / "flash_muon_b200" / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    path = build.build()
    assert path.exists() and path.parent == ROOT / "flash_muon_b200"


@pytest.mark.parametrize("name", declared_symbols())
def test_library_exports(name):
    from flash_muon_b200 import _lib
    assert hasattr(_lib.lib, name), f"{name} declared in the header but not exported"
    assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_integration_notes_name_every_entry_point():
    """Every function the header declares has a line in INTEGRATION.md saying what it replaces."""
    header = (ROOT / "include" / "flash_muon_b200.h").read_text()
    notes = (ROOT / "INTEGRATION.md").read_text()
    declared = sorted(set(re.findall(r"\b(fm_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    missing = [name for name in declared if name not in notes]
    assert not missing, f"not in INTEGRATION.md: {missing}"


def test_ctypes_table_has_no_undeclared_entry():
    from flash_muon_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_only_calls():
    """Entry points that touch no device."""
    from flash_muon_b200 import _lib
    lib = _lib.lib
    assert lib.fm_version() >= 200
    assert lib.fm_norm_scratch_floats() >= 1
    assert lib.fm_ns_workspace_bytes(0, 4) == 0
    m, k = 1024, 4096
    need = lib.fm_ns_workspace_bytes(m, k)
    assert need == lib.fm_ns_workspace_bytes(k, m)          # tall = wide transposed
    assert need >= (4 * m * k + 2 * m * m) * 2              # X, XT double-buffered + A + B
    # argument validation happens before any CUDA call
    assert lib.fm_syrk(None, None, 4, 4, 4, 4, 1, 0, None, 0, None) == -1
    assert b"null" in lib.fm_last_error()
    assert lib.fm_newtonschulz(None, 4, 4, 4, 0, 5, None, None, 0, 0, None) == -1
    assert lib.fm_momentum(None, None, 4, 0, 0.95, 1, None, None) == -1
    assert lib.fm_update_multi(None, None, None, None, -1, 0, 1.0, None) == -1
    assert lib.fm_newtonschulz_batched(None, None, None, 2, 0, 5, None, None, 0, 0, None) == -1
    assert lib.fm_ns_batched_workspace_bytes(0, 8, 8) == 0 == lib.fm_ns_batched_workspace_bytes(17, 8, 8)
    assert lib.fm_ns_batched_workspace_bytes(1, m, k) == need
    assert lib.fm_ns_batched_workspace_bytes(4, m, k) >= 4 * (4 * m * k + 2 * m * m) * 2
    assert lib.fm_ns_partials_offset(m, k) + 4 * lib.fm_norm_scratch_floats() <= need
    # tuning switches: unknown names are refused, known ones round-trip
    assert lib.fm_set_option(b"no_such_switch", 1) == -1
    v = ctypes.c_int(-5)
    assert lib.fm_get_option(b"gemm_balance", ctypes.byref(v)) == 0 and v.value in (0, 1)
    old = v.value
    assert lib.fm_set_option(b"gemm_balance", 0) == 0
    assert lib.fm_get_option(b"gemm_balance", ctypes.byref(v)) == 0 and v.value == 0
    assert lib.fm_set_option(b"gemm_balance", old) == 0
    assert lib.fm_newtonschulz_static(None, 0, 4, 4, 0, 5, None, 0, None) == -1
    assert lib.fm_newtonschulz_static(None, 2048, 2048, 2048, 0, 5, None, 0, None) == -5
    assert b"1024 x 4096" in lib.fm_last_error()
    assert lib.fm_ipc_export(None, None, None) == -1
    assert lib.fm_ipc_import(None, 0, None) == -1
    assert lib.fm_stream_write32(None, 1, None) == -1
    assert lib.fm_stream_wait32_geq(None, 1, None) == -1
    assert lib.fm_copy_async(None, None, 0, None) == 0      # nothing to copy
    assert lib.fm_copy_async(None, None, 16, None) == -1


def test_whole_step_call_validates_before_any_cuda_call():
    """fm_muon_step rejects malformed groups on the host; the struct layout is the header's."""
    import ctypes
    from flash_muon_b200 import _lib
    assert ctypes.sizeof(_lib.MuonGroup) == 6 * 8 + 8 * 4 + 2 * 8 + 8
    g = _lib.MuonGroup()
    g.count, g.lanes, g.batch = 1, 2, 1
    assert _lib.lib.fm_muon_step(g, 1, None, 0, None) == -1          # null workspace list
    w = (ctypes.c_void_p * 1)(0)
    assert _lib.lib.fm_muon_step(g, 1, w, 0, None) == -1             # null arrays in the group
    assert b"null array" in _lib.lib.fm_last_error()
    assert _lib.lib.fm_muon_step(None, 0, None, 0, None) == 0        # nothing to do
    g.count = -1
    assert _lib.lib.fm_muon_step(g, 1, w, 0, None) == -1


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    """No fallback: pointing the loader at a missing file raises ImportError."""
    import importlib
    import flash_muon_b200._lib as L
    monkeypatch.setenv("FLASH_MUON_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or Triton fallback"):
        importlib.reload(L)
    monkeypatch.delenv("FLASH_MUON_B200_LIB")
    importlib.reload(L)
