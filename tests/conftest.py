"""pytest configuration: the ``gpu`` marker, import paths and shared fixtures."""
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return torch.load(ROOT / "tests" / "golden" / "reference_outputs.pt")


@pytest.fixture
def options():
    """Sets tuning switches of the library (``fm_set_option``) for one test and restores them."""
    from flash_muon_b200 import _lib
    saved = {}

    def set_option(name: str, value: int) -> None:
        if name not in saved:
            saved[name] = _lib.get_option(name)
        _lib.set_option(name, value)

    yield set_option
    for name, value in saved.items():
        _lib.set_option(name, value)


# Where GPU sessions leave their measured records (parity distances): FM_REPORT_DIR, or the
# scratch output folder at the repository root.
REPORT_DIR = Path(os.environ.get("FM_REPORT_DIR", ROOT / "gpurun_out"))
_OBSERVED: dict = {}


def observe(name: str, value: float) -> float:
    """Remembers a measured distance under ``name`` (largest value wins) and returns it; at the end
    of a GPU session everything observed is written to ``parity_observed.json`` in the report
    folder, the record the tolerances in these tests are set from."""
    _OBSERVED[name] = max(float(value), _OBSERVED.get(name, 0.0))
    return value


def pytest_sessionfinish(session, exitstatus):
    if not _OBSERVED:
        return
    import json
    try:
        out = REPORT_DIR
        out.mkdir(exist_ok=True)
        (out / "parity_observed.json").write_text(json.dumps(dict(sorted(_OBSERVED.items())), indent=1))
    except OSError:
        pass


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b||_F / ||b||_F in float64."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-300)).item()
