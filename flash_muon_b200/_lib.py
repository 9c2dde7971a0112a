"""ctypes binding of ``libflash_muon_b200.so`` (declared in ``include/flash_muon_b200.h``).

There is no fallback: if the shared library is missing or fails to load, importing this module
raises, and every operator of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("FLASH_MUON_B200_LIB", _PKG_DIR / "libflash_muon_b200.so"))

FM_OK = 0
FM_BF16, FM_F16, FM_F32 = 0, 1, 2
FM_NS_FAITHFUL, FM_NS_PRECISE, FM_NS_SUMSQ_READY = 0, 1, 2

_DTYPES = {torch.bfloat16: FM_BF16, torch.float16: FM_F16, torch.float32: FM_F32}

c_void_p, c_int, c_int64, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
c_float, c_double = ctypes.c_float, ctypes.c_double

class MuonGroup(ctypes.Structure):
    """``fm_muon_group`` of include/flash_muon_b200.h."""
    _fields_ = [("params", ctypes.POINTER(c_void_p)), ("grads", ctypes.POINTER(c_void_p)),
                ("momentum", ctypes.POINTER(c_void_p)), ("rows", ctypes.POINTER(c_int64)),
                ("cols", ctypes.POINTER(c_int64)), ("alphas", ctypes.POINTER(c_double)),
                ("count", ctypes.c_int32), ("p_dtype", ctypes.c_int32), ("g_dtype", ctypes.c_int32),
                ("nesterov", ctypes.c_int32), ("ns_steps", ctypes.c_int32), ("lanes", ctypes.c_int32),
                ("batch", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("momentum_coef", c_double), ("decay", c_double),
                ("slots", ctypes.POINTER(c_void_p))]


# name -> (restype, argtypes); mirrors include/flash_muon_b200.h one to one
SIGNATURES = {
    "fm_version": (c_int, []),
    "fm_last_error": (ctypes.c_char_p, []),
    "fm_device_status": (c_int, [ctypes.POINTER(ctypes.c_uint)]),
    "fm_set_option": (c_int, [ctypes.c_char_p, c_int]),
    "fm_get_option": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_int)]),
    "fm_syrk_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int]),
    "fm_syrk": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int,
                        c_void_p, c_size_t, c_void_p]),
    "fm_gemm_nt": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64,
                           c_void_p, c_int64, c_float, c_float, c_void_p, c_int64, c_void_p,
                           c_int64, c_int, c_int, c_void_p]),
    "fm_syrk_poly": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_float,
                             c_float, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "fm_ns_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "fm_ns_partials_offset": (c_size_t, [c_int64, c_int64]),
    "fm_ns_batched_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64]),
    "fm_ns_batched_partials_offset": (c_size_t, [c_int, c_int64, c_int64]),
    "fm_newtonschulz_batched": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64),
                                        ctypes.POINTER(c_int64), c_int, c_int, c_int,
                                        ctypes.POINTER(c_void_p), c_void_p, c_size_t, c_int,
                                        c_void_p]),
    "fm_newtonschulz": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p,
                                c_void_p, c_size_t, c_int, c_void_p]),
    "fm_newtonschulz_static": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p,
                                       c_int, c_void_p]),
    "fm_normalize": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_int64,
                             c_void_p, c_int64, c_void_p, c_void_p]),
    "fm_norm_scratch_floats": (c_size_t, []),
    "fm_momentum": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_double, c_int, c_void_p,
                            c_void_p]),
    "fm_ipc_export": (c_int, [c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64)]),
    "fm_ipc_import": (c_int, [ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(c_void_p)]),
    "fm_ipc_close_all": (c_int, []),
    "fm_copy_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "fm_stream_write32": (c_int, [c_void_p, ctypes.c_uint32, c_void_p]),
    "fm_stream_wait32_geq": (c_int, [c_void_p, ctypes.c_uint32, c_void_p]),
    "fm_update_multi": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                ctypes.POINTER(c_int64), ctypes.POINTER(c_double), c_int, c_int,
                                c_double, c_void_p]),
    "fm_muon_step": (c_int, [ctypes.POINTER(MuonGroup), c_int, ctypes.POINTER(c_void_p),
                             ctypes.c_size_t, c_void_p]),
}


class FlashMuonError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"flash_muon_b200 status {status}: {message}")
        self.status = status


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python flash_muon_b200/build.py` "
            "(there is no CPU or Triton fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export the symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int) -> None:
    if status != FM_OK:
        raise FlashMuonError(status, lib.fm_last_error().decode("utf-8", "replace"))


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"flash_muon_b200 supports bfloat16, float16 and float32, got {dtype}")


def current_stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


on_option_change: list = []  # callbacks of modules that cache plans depending on the options


def set_option(name: str, value: int) -> None:
    """Process-wide tuning switch of the library (``fm_set_option``)."""
    check(lib.fm_set_option(name.encode(), int(value)))
    for fn in on_option_change:
        fn()


def get_option(name: str) -> int:
    v = c_int(0)
    check(lib.fm_get_option(name.encode(), ctypes.byref(v)))
    return v.value


def device_status() -> int:
    """Synchronise and raise if any kernel abandoned a bounded wait; returns 0 otherwise."""
    code = ctypes.c_uint(0)
    check(lib.fm_device_status(ctypes.byref(code)))
    return code.value
