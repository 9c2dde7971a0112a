"""The HBM-bound kernels against torch's own CUDA element kernels (what the reference launches at
flash_muon/muon.py:23, :87-89, :99-100): bit-exact, and against the CPU oracle."""
import ctypes

import pytest
import torch

from flash_muon_b200 import _lib
from flash_muon_b200._lib import check, dtype_code, lib
from oracle import muon_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def _rand(n, dt, scale, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(n, device=DEV, generator=g) * scale).to(dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nesterov", [True, False])
@pytest.mark.parametrize("n,offset", [(1 << 20, 0), (12345, 0), (4099, 1), (1, 0), (7, 3)])
def test_momentum_bit_exact(dt, nesterov, n, offset):
    g = _rand(n + offset, dt, 1e-3, 1)[offset:]
    b = _rand(n + offset, dt, 1e-3, 2)[offset:]
    g_ref, b_ref = g.clone(), b.clone()
    used = O.momentum_update(g_ref, b_ref, 0.95, nesterov)   # torch CUDA lerp_
    check(lib.fm_momentum(g.data_ptr(), b.data_ptr(), n, dtype_code(dt), 0.95, int(nesterov), None, 0))
    assert torch.equal(b, b_ref)
    assert torch.equal(g, g_ref)
    assert used.data_ptr() == (g_ref if nesterov else b_ref).data_ptr()
    # CPU oracle: same formula, torch's CPU kernel may differ in the last bit of a few elements
    gc, bc = _rand(n + offset, dt, 1e-3, 1)[offset:].cpu(), _rand(n + offset, dt, 1e-3, 2)[offset:].cpu()
    O.momentum_update(gc, bc, 0.95, nesterov)
    assert torch.allclose(b.cpu().float(), bc.float(), rtol=2 ** -7, atol=1e-9)
    assert torch.allclose(g.cpu().float(), gc.float(), rtol=2 ** -7, atol=1e-9)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nesterov", [True, False])
@pytest.mark.parametrize("rows,cols,offset", [(1024, 1024, 0), (256, 384, 0), (100, 72, 0),
                                              (65, 63, 0), (33, 7, 1), (4096, 1024, 0)])
def test_momentum_leaves_the_partial_sums_of_the_norm(dt, nesterov, rows, cols, offset):
    """With a partials pointer fm_momentum also produces the partial sums of squares that
    fm_normalize computes in its first pass -- the same floats, whether the fused kernel ran
    (aligned tensors of a vector multiple) or the separate pass (anything else): Newton-Schulz
    with FM_NS_SUMSQ_READY then equals the plain call bit for bit."""
    n = rows * cols
    g = _rand(n + offset, dt, 1e-3, 3)[offset:]
    b = _rand(n + offset, dt, 1e-3, 4)[offset:]
    g2, b2 = g.clone(), b.clone()
    need = lib.fm_ns_workspace_bytes(rows, cols)
    off = lib.fm_ns_partials_offset(rows, cols)
    ws = torch.zeros(need, device=DEV, dtype=torch.uint8)
    ws2 = torch.zeros(need, device=DEV, dtype=torch.uint8)
    check(lib.fm_momentum(g.data_ptr(), b.data_ptr(), n, dtype_code(dt), 0.95, int(nesterov),
                          ws.data_ptr() + off, 0))
    check(lib.fm_momentum(g2.data_ptr(), b2.data_ptr(), n, dtype_code(dt), 0.95, int(nesterov), None, 0))
    assert torch.equal(g, g2) and torch.equal(b, b2)
    src, src2 = (g, g2) if nesterov else (b, b2)
    out = torch.empty(rows, cols, device=DEV, dtype=torch.bfloat16)
    out2 = torch.empty(rows, cols, device=DEV, dtype=torch.bfloat16)
    check(lib.fm_newtonschulz(src.data_ptr(), rows, cols, cols, dtype_code(dt), 2, out.data_ptr(),
                              ws.data_ptr(), need, _lib.FM_NS_SUMSQ_READY, 0))
    check(lib.fm_newtonschulz(src2.data_ptr(), rows, cols, cols, dtype_code(dt), 2, out2.data_ptr(),
                              ws2.data_ptr(), need, 0, 0))
    nparts = max(1, min(1024, (n + 8191) // 8192))
    p1 = ws[off:off + 4 * nparts].view(torch.float32)
    p2 = ws2[off:off + 4 * nparts].view(torch.float32)
    assert torch.equal(p1, p2)
    assert torch.equal(out, out2)
    _lib.device_status()


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("count", [1, 8, 40])
def test_update_multi_bit_exact(dt, count):
    lr, wd = 0.02, 0.01
    shapes = [(64, 24), (24, 64), (40, 40)]
    ps = [_rand(s[0] * s[1], dt, 0.02, 10 + i).view(*s) for i in range(count) for s in [shapes[i % 3]]]
    us = [_rand(p.numel(), torch.bfloat16, 1.0, 100 + i) for i, p in enumerate(ps)]
    refs = [p.clone() for p in ps]
    for p, u in zip(refs, us):
        O.apply_update(p, u, lr, wd)                          # torch CUDA mul_ / add_
    n = len(ps)
    ptrs = (ctypes.c_void_p * n)(*[p.data_ptr() for p in ps])
    upds = (ctypes.c_void_p * n)(*[u.data_ptr() for u in us])
    nels = (ctypes.c_int64 * n)(*[p.numel() for p in ps])
    alphas = (ctypes.c_double * n)(*[-lr * max(1, p.size(-2) / p.size(-1)) ** 0.5 for p in ps])
    check(lib.fm_update_multi(ptrs, upds, nels, alphas, n, dtype_code(dt), 1 - lr * wd, 0))
    for p, r in zip(ps, refs):
        assert torch.equal(p, r)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("rows,cols", [(256, 512), (512, 256), (100, 72), (1, 8), (65, 63), (1024, 4096)])
def test_normalize_bit_exact(dt, rows, cols):
    G = _rand(rows * cols, dt, 1.0, rows + cols).view(rows, cols)
    X = G.bfloat16()
    ref = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)     # flash_muon/muon.py:15, :23
    ldd, ldt = cols + 8, rows + 16                            # padded pitches
    xd = torch.full((rows, ldd), float("nan"), device=DEV, dtype=torch.bfloat16)
    xt = torch.full((cols, ldt), float("nan"), device=DEV, dtype=torch.bfloat16)
    part = torch.empty(lib.fm_norm_scratch_floats(), device=DEV, dtype=torch.float32)
    check(lib.fm_normalize(G.data_ptr(), rows, cols, cols, dtype_code(dt), xd.data_ptr(), ldd,
                           xt.data_ptr(), ldt, part.data_ptr(), 0))
    # the norm is reduced in another order than torch's: allow the rare last-bit flip of the
    # bf16 denominator, which moves every quotient by at most one bf16 ulp
    assert torch.allclose(xd[:, :cols].float(), ref.float(), rtol=2 ** -7, atol=0)
    assert torch.equal(xt[:, :rows], xd[:, :cols].T)
    assert torch.isnan(xd[:, cols:]).all() and torch.isnan(xt[:, rows:]).all()
    _lib.device_status()


@pytest.mark.parametrize("rows,cols", [(192, 320), (2048, 2048), (4096, 1024), (64, 8192)])
def test_normalize_quotients_are_correctly_rounded_divisions(rows, cols):
    """The 16-byte path multiplies by the reciprocal of the denominator and divides only where the
    product lies near a bf16 rounding boundary.  Every element must still be the fp32 quotient
    rounded to bf16, as torch's division gives it (flash_muon/muon.py:23), for the bf16 denominator
    the kernel derived: torch's own, or its neighbour when the sum order moved the last bit."""
    X = _rand(rows * cols, torch.bfloat16, 1.0, 7 * rows + cols).view(rows, cols)
    xd = torch.empty_like(X)
    xt = torch.empty(cols, rows, device=DEV, dtype=torch.bfloat16)
    part = torch.empty(lib.fm_norm_scratch_floats(), device=DEV, dtype=torch.float32)
    check(lib.fm_normalize(X.data_ptr(), rows, cols, cols, dtype_code(torch.bfloat16), xd.data_ptr(), cols,
                           xt.data_ptr(), rows, part.data_ptr(), 0))
    norm = X.norm(dim=(-2, -1), keepdim=True)
    bits = norm.view(torch.int16)
    hits = []
    for delta in (0, -1, 1):
        d = (bits + delta).view(torch.bfloat16)
        hits.append(torch.equal(xd, X / (d + 1e-7)))
    assert any(hits), "no bf16 denominator next to torch's reproduces the kernel's quotients"
    assert torch.equal(xt, xd.T)
    _lib.device_status()
