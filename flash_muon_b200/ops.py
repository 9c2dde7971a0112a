"""Operator interface of the reference (``flash_muon/__init__.py:1-4``) over the C-ABI library.

Same names, argument meaning and error behaviour as
``flash_muon/matmul_transpose_triton.py:78-107`` and ``flash_muon/muon.py:6-33``; the device work
is done by hand-written sm_100a kernels.  CPU tensors raise the same ``AssertionError`` as the
reference: there is no CPU path.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from ._lib import check, dtype_code, lib

__all__ = ["matmul_transpose", "matmul_transpose_assign", "fast_newtonschulz",
           "newtonschulz_workspace_bytes"]

# Host-side cost matters for small products (a 1024 x 1024 product is ~10 us of GPU time), so the
# wrappers look the raw stream handle up directly and enter a device guard only when the tensor
# does not live on the current device.
_raw_stream = torch._C._cuda_getCurrentRawStream
_current_device = torch._C._cuda_getDevice

# Scratch for the balanced tail of long tile lists, one per (device, stream): kernels of one
# stream run in order and may share it, kernels of different streams may overlap and may not.
_syrk_scratch: dict = {}
_syrk_need: dict = {}


def _syrk_workspace(device: torch.device, stream: int, M: int, K: int, code: int):
    key = (M, K, code)
    need = _syrk_need.get(key)
    if need is None:
        need = _syrk_need[key] = int(lib.fm_syrk_workspace_bytes(M, K, code))
    if need == 0:
        return 0, 0
    ws = _syrk_scratch.get((device.index, stream))
    if ws is None or ws.numel() < need:
        ws = _syrk_scratch[(device.index, stream)] = torch.empty(need, dtype=torch.uint8, device=device)
    return ws.data_ptr(), ws.numel()


def _forget_plans() -> None:
    """Sizes cached above depend on the library's options (``_lib.set_option``)."""
    _syrk_need.clear()


_lib.on_option_change.append(_forget_plans)


def matmul_transpose_assign(d_in: Tensor, d_out: Tensor) -> None:
    """``d_out[:] = d_in @ d_in.T`` with a bitwise-symmetric result.

    Mirrors ``matmul_transpose_assign`` (flash_muon/matmul_transpose_triton.py:78-101): same
    assertions and messages; ``d_out`` may have arbitrary strides.  The size check also covers
    ``d_out.size(1)``, which the reference's assert names but never compares.
    """
    assert d_in.is_cuda, "Input `d_in` must be a CUDA tensor"
    assert d_out.is_cuda, "Input `d_out` must be a CUDA tensor"
    assert d_in.device == d_out.device, "Inputs `d_in` and `d_out` must be on the same CUDA device"
    assert d_in.dtype == d_out.dtype, "Inputs must have the same data type"
    assert d_in.ndim == 2, "Input `d_in` must be a 2D tensor"
    assert d_out.ndim == 2, "Input `d_out` must be a 2D tensor"
    assert d_in.size(0) == d_out.size(0) == d_out.size(1), \
        "First dimension of `d_in` must match first and second dimension of `d_out`"

    M, K = d_in.shape
    if M == 0:
        return
    if K == 0:
        d_out.zero_()
        return
    if d_in.stride(1) != 1 or d_in.stride(0) < K:
        d_in = d_in.contiguous()
    device = d_in.device
    code = dtype_code(d_in.dtype)
    if device.index != _current_device():
        with torch.cuda.device(device):
            return _syrk(d_in, d_out, M, K, code, device)
    _syrk(d_in, d_out, M, K, code, device)


def _syrk(d_in: Tensor, d_out: Tensor, M: int, K: int, code: int, device: torch.device) -> None:
    stream = _raw_stream(device.index)
    ws, ws_bytes = _syrk_workspace(device, stream, M, K, code)
    rc = lib.fm_syrk(d_in.data_ptr(), d_out.data_ptr(), M, K, d_in.stride(0), d_out.stride(0),
                     d_out.stride(1), code, ws, ws_bytes, stream)
    if rc:
        check(rc)


def matmul_transpose(d_in: Tensor) -> Tensor:
    """Returns ``d_in @ d_in.T`` (flash_muon/matmul_transpose_triton.py:103-107)."""
    M, _ = d_in.shape
    d_out = torch.empty((M, M), device=d_in.device, dtype=d_in.dtype)
    matmul_transpose_assign(d_in, d_out)
    return d_out


def newtonschulz_workspace_bytes(rows: int, cols: int) -> int:
    """Device scratch ``fast_newtonschulz`` needs for a ``rows x cols`` input."""
    return int(lib.fm_ns_workspace_bytes(rows, cols))


def fast_newtonschulz(G: Tensor, steps: int = 5, *, out: Tensor | None = None,
                      workspace: Tensor | None = None, precise: bool = False,
                      sumsq_ready: bool = False) -> Tensor:
    """Newton-Schulz orthogonalisation of ``G`` (flash_muon/muon.py:6-33).

    Returns a bfloat16 tensor of ``G``'s shape.  The whole iteration is enqueued by one C-ABI call
    on the current stream.  ``out`` (bf16, contiguous, G's shape) and ``workspace`` (uint8, at
    least ``newtonschulz_workspace_bytes`` bytes) let a caller run without any allocation;
    ``precise=True`` selects single-rounding epilogues instead of the reference's rounding points;
    ``sumsq_ready=True`` says that ``fm_momentum`` already left the partial sums of the norm in
    ``workspace`` (at ``fm_ns_partials_offset``), so the pass that computes them is skipped.
    """
    assert G.ndim >= 2
    assert G.ndim == 2, "fast_newtonschulz handles 2D matrices (flatten conv filters first)"
    assert G.is_cuda, "Input `G` must be a CUDA tensor"
    rows, cols = G.shape
    if out is None:
        out = torch.empty((rows, cols), device=G.device, dtype=torch.bfloat16)
    else:
        assert out.is_cuda and out.device == G.device and out.dtype == torch.bfloat16
        assert out.numel() == rows * cols and out.is_contiguous()
    if rows == 0 or cols == 0:
        return out
    if G.stride(1) != 1 or G.stride(0) < cols:
        G = G.contiguous()
    need = newtonschulz_workspace_bytes(rows, cols)
    if workspace is None:
        workspace = torch.empty(need, device=G.device, dtype=torch.uint8)
    else:
        assert workspace.is_cuda and workspace.device == G.device and workspace.is_contiguous()
        assert workspace.numel() * workspace.element_size() >= need, "workspace too small"
    flags = (_lib.FM_NS_PRECISE if precise else _lib.FM_NS_FAITHFUL) | \
        (_lib.FM_NS_SUMSQ_READY if sumsq_ready else 0)
    with torch.cuda.device(G.device):
        check(lib.fm_newtonschulz(G.data_ptr(), rows, cols, G.stride(0), dtype_code(G.dtype),
                                  int(steps), out.data_ptr(), workspace.data_ptr(),
                                  workspace.numel() * workspace.element_size(), flags,
                                  _raw_stream(G.device.index)))
    return out.view(rows, cols)
