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
from ._lib import check, current_stream_ptr, dtype_code, lib

__all__ = ["matmul_transpose", "matmul_transpose_assign", "fast_newtonschulz",
           "newtonschulz_workspace_bytes"]


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
    with torch.cuda.device(d_in.device):
        check(lib.fm_syrk(d_in.data_ptr(), d_out.data_ptr(), M, K, d_in.stride(0),
                          d_out.stride(0), d_out.stride(1), dtype_code(d_in.dtype),
                          current_stream_ptr(d_in.device)))


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
                      workspace: Tensor | None = None, precise: bool = False) -> Tensor:
    """Newton-Schulz orthogonalisation of ``G`` (flash_muon/muon.py:6-33).

    Returns a bfloat16 tensor of ``G``'s shape.  The whole iteration is enqueued by one C-ABI call
    on the current stream.  ``out`` (bf16, contiguous, G's shape) and ``workspace`` (uint8, at
    least ``newtonschulz_workspace_bytes`` bytes) let a caller run without any allocation;
    ``precise=True`` selects single-rounding epilogues instead of the reference's rounding points.
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
    with torch.cuda.device(G.device):
        check(lib.fm_newtonschulz(G.data_ptr(), rows, cols, G.stride(0), dtype_code(G.dtype),
                                  int(steps), out.data_ptr(), workspace.data_ptr(),
                                  workspace.numel() * workspace.element_size(),
                                  _lib.FM_NS_PRECISE if precise else _lib.FM_NS_FAITHFUL,
                                  current_stream_ptr(G.device)))
    return out.view(rows, cols)
