"""``fm_newtonschulz_static``: Newton-Schulz for callers that must not allocate device memory
(plugins inside a host that owns the allocator, code inside a stream capture).  Its scratch is a
fixed array inside the library, so the test checks three things through the C ABI: the result
equals the workspace-taking entry point's on two calls in a row (the shared array keeps the first
call's contents), nothing is allocated through torch while it runs, and inputs beyond the stated
limit are refused before any launch.  Collected last on purpose: a failure here cannot hide
another test's result in a run that stops at the first failure."""
import pytest
import torch

from flash_muon_b200 import _lib
from flash_muon_b200._lib import lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rel(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm()).item()


def _with_workspace(G, steps):
    rows, cols = G.shape
    out = torch.empty(rows, cols, device=DEV, dtype=torch.bfloat16)
    ws = torch.empty(lib.fm_ns_workspace_bytes(rows, cols), device=DEV, dtype=torch.uint8)
    _lib.check(lib.fm_newtonschulz(G.data_ptr(), rows, cols, cols, _lib.dtype_code(G.dtype), steps,
                                   out.data_ptr(), ws.data_ptr(), ws.numel(), 0, 0))
    return out


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    """Same kernels, same layout, other scratch: the outputs must be the workspace entry point's
    bit for bit -- anything left over from the previous call in the shared array, a wrong region
    offset or an overlap between regions would show up as a difference.  Calls go out on a
    stream of their own, as a plugin would issue them."""
    torch.cuda.set_device(0)
    gen = torch.Generator(device=DEV).manual_seed(11)
    inputs = [torch.randn(1024, 4096, device=DEV, generator=gen).bfloat16(),   # the largest allowed
              torch.randn(520, 300, device=DEV, generator=gen),                # tall, f32, odd sizes
              torch.randn(4096, 1024, device=DEV, generator=gen).bfloat16(),   # the largest, tall
              torch.randn(1023, 4095, device=DEV, generator=gen).half()]       # off the grid, near the limit
    expected = [_with_workspace(G, 5) for G in inputs]
    outs = [torch.full_like(e, float("nan")) for e in expected]
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    for G, out in zip(inputs, outs):                                           # back to back
        rows, cols = G.shape
        rc = lib.fm_newtonschulz_static(G.data_ptr(), rows, cols, cols, _lib.dtype_code(G.dtype), 5,
                                        out.data_ptr(), 0, stream.cuda_stream)
        assert rc == 0, lib.fm_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    for out, exp in zip(outs, expected):
        assert torch.equal(out, exp)
        assert _rel(out, exp) <= 2e-2            # the tolerance of the Newton-Schulz parity tests
    _lib.device_status()


def test_static_scratch_rejects_sizes_beyond_its_limit():
    G = torch.zeros(2048, 2048, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(G)
    rc = lib.fm_newtonschulz_static(G.data_ptr(), 2048, 2048, 2048, 0, 5, out.data_ptr(), 0, 0)
    assert rc == -5
    msg = lib.fm_last_error().decode()
    assert "1024 x 4096" in msg and "2048 x 2048" in msg
    rc = lib.fm_newtonschulz_static(G.data_ptr(), 512, 8192, 8192, 0, 5, out.data_ptr(), 0, 0)
    assert rc == -5
