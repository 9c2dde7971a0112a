"""Parity of the CUDA symmetric product (through the C ABI) with the oracle, the reference's golden
outputs and a plain torch product, on BASELINE's configs and on the edge cases the reference's
kernel handles (sizes off the tile grid, strided outputs, other dtypes)."""
import pytest
import torch

import flash_muon_b200 as fm
from flash_muon_b200 import _lib
from conftest import rel_fro
from inputs import SYRK_CASES, syrk_input
from oracle import muon_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2}  # tolerances BASELINE.json states for fp32 / 16-bit products


def check_syrk(x, y):
    assert not torch.isnan(y).any()
    assert torch.equal(y, y.T), "upper and lower triangles must be bit-identical mirrors"
    ref = x.double() @ x.double().T
    assert rel_fro(y, ref) <= TOL[x.dtype]
    _lib.device_status()


@pytest.mark.parametrize("m,k,dt", SYRK_CASES)
def test_golden_cases(golden, m, k, dt):
    x = syrk_input(m, k, dt)
    y = fm.matmul_transpose(x.to(DEV))
    check_syrk(x.to(DEV), y)
    assert rel_fro(y, golden[f"torch_matmul_transpose/{m}x{k}/{dt}"]) <= TOL[dt]
    assert rel_fro(y, O.matmul_transpose(x)) <= TOL[dt]
    if dt == torch.float32:
        assert rel_fro(y, golden["mmt_kernel_interpreter/96x80/torch.float32"]) <= 1e-5


def test_config0_fp32_1024():
    """configs[0]: X 1024x1024 fp32 N(0,1), seed 0; symmetric and equal to torch.matmul."""
    x = torch.randn(1024, 1024, generator=torch.Generator().manual_seed(0))
    y = fm.matmul_transpose(x.to(DEV))
    assert torch.equal(y, y.T)
    assert rel_fro(y, torch.matmul(x, x.T)) <= 1e-5
    assert rel_fro(y, O.matmul_transpose(x)) <= 1e-5


@pytest.mark.parametrize("m,k", [(1024, 1024), (2048, 2048), (4096, 4096), (8192, 8192),
                                 (4096, 16384), (16384, 4096)])
def test_config2_bf16_sweep(m, k):
    """configs[2]: bf16, entries N(0,1)/sqrt(k); the tall case is transposed first, as in Muon."""
    g = torch.Generator(device=DEV).manual_seed(m + k)
    x = (torch.randn(m, k, device=DEV, generator=g) / k ** 0.5).bfloat16()
    if m > k:
        x = x.T  # non-contiguous view: the wrapper makes it contiguous like the reference (:88)
    y = fm.matmul_transpose(x)
    assert y.shape == (x.shape[0], x.shape[0])
    assert torch.equal(y, y.T)
    ref = torch.matmul(x, x.T)  # cuBLAS, the reference's own baseline (benchmark.py:20-21)
    assert rel_fro(y, ref) <= 1e-2
    # size-independent properties: the diagonal holds the squared row norms, and a slice agrees
    # with the CPU oracle
    diag = (x.double() ** 2).sum(dim=1)
    assert torch.allclose(y.diagonal().double(), diag, rtol=1e-2, atol=1e-3)
    rows = slice(0, 64)
    blk = (x[rows].float().cpu() @ x.float().cpu().T).bfloat16()
    assert rel_fro(y[rows], blk) <= 1e-2
    _lib.device_status()


ODD = [(1, 8), (7, 8), (8, 1), (100, 72), (129, 64), (257, 136), (130, 1000), (33, 17), (300, 5),
       (384, 320), (640, 64), (1000, 520)]


@pytest.mark.parametrize("bn", ["64", "128", "256", "pair"])
@pytest.mark.parametrize("m,k", ODD)
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_sizes_off_the_tile_grid(m, k, dt, bn, options):
    """Every tile shape of the tensor-core family (single CTA 128x64 / 128x128 / 128x256, CTA
    pair 256x256) on sizes that are not multiples of any of them."""
    if bn == "pair":
        options("gemm_impl", 2)
    else:
        options("gemm_impl", 1)
        options("gemm_bn", int(bn))
    x = torch.randn(m, k, device=DEV, generator=torch.Generator(device=DEV).manual_seed(m * k)).to(dt)
    y = torch.full((m, m), float("nan"), device=DEV, dtype=dt)  # canary: every element written
    fm.matmul_transpose_assign(x, y)
    check_syrk(x, y)
    assert rel_fro(y, O.matmul_transpose(x.cpu())) <= TOL[dt]


def test_strided_output_and_input():
    x = torch.randn(200, 72, device=DEV).bfloat16()
    ref = O.matmul_transpose(x.cpu()).to(DEV)
    big = torch.full((200, 512), float("nan"), device=DEV, dtype=torch.bfloat16)
    out = big[:, 8:208]                                   # row pitch 512
    fm.matmul_transpose_assign(x, out)
    assert rel_fro(out, ref) <= 1e-2 and torch.equal(out, out.T)
    assert torch.isnan(big[:, :8]).all() and torch.isnan(big[:, 208:]).all()
    outT = torch.empty(200, 200, device=DEV, dtype=torch.bfloat16).T  # column-major view
    fm.matmul_transpose_assign(x, outT)
    assert torch.equal(outT, out)
    every2 = torch.full((200, 400), float("nan"), device=DEV, dtype=torch.bfloat16)[:, ::2]
    fm.matmul_transpose_assign(x, every2)                 # column stride 2
    assert torch.equal(every2, out)
    xbig = torch.randn(200, 128, device=DEV).bfloat16()
    xs = xbig[:, :72]                                     # row pitch 128 > K
    assert torch.equal(fm.matmul_transpose(xs), fm.matmul_transpose(xs.contiguous()))
    xt = torch.randn(72, 200, device=DEV).bfloat16().T    # transposed view of a [72, 200] tensor
    assert torch.equal(fm.matmul_transpose(xt), fm.matmul_transpose(xt.contiguous()))
    _lib.device_status()


def test_run_to_run_determinism():
    x = torch.randn(1000, 520, device=DEV).bfloat16()
    assert torch.equal(fm.matmul_transpose(x), fm.matmul_transpose(x))


def test_balanced_tail_schedule(options):
    """A tile list of several waves with a short last wave and a long K is finished by cutting
    the last tiles by K blocks (partial accumulators through fp32 scratch): same tolerance, exact
    symmetry, run-to-run determinism, and within rounding of the whole-tile schedule."""
    m, k = 3328, 5120   # 91 tiles of 256 x 256 on 74 CTA pairs, 80 K blocks
    x = (torch.randn(m, k, device=DEV, generator=torch.Generator(device=DEV).manual_seed(5)) / k ** 0.5).bfloat16()
    options("gemm_balance", 1)
    assert _lib.lib.fm_syrk_workspace_bytes(m, k, 0) > 0      # this shape takes the balanced tail
    y = torch.full((m, m), float("nan"), device=DEV, dtype=torch.bfloat16)
    fm.matmul_transpose_assign(x, y)
    check_syrk(x, y)
    assert torch.equal(y, fm.matmul_transpose(x))
    assert torch.equal(y, fm.matmul_transpose(x))
    options("gemm_balance", 0)
    assert _lib.lib.fm_syrk_workspace_bytes(m, k, 0) == 0
    whole = fm.matmul_transpose(x)
    # the C entry point without scratch deals whole tiles whatever the switch says
    options("gemm_balance", 1)
    bare = torch.empty_like(whole)
    _lib.check(_lib.lib.fm_syrk(x.data_ptr(), bare.data_ptr(), m, k, k, m, 1, 0, None, 0, 0))
    assert torch.equal(bare, whole)
    assert rel_fro(y, whole) <= 2e-3
    assert rel_fro(whole, torch.matmul(x, x.T)) <= 2e-3
    _lib.device_status()


@pytest.mark.parametrize("w", [3, 8])
def test_strip_tile_order_gives_the_same_product(w, options):
    """The strip order walks the same tiles in column strips: with whole tiles (short K, no balanced
    tail) every tile is computed by the same instructions, so the product is bit-identical."""
    torch.manual_seed(4)
    x = (torch.randn(4700, 320, device=DEV) / 18).bfloat16()     # 19 tile columns, ragged edge
    options("gemm_impl", 2)
    options("gemm_strip", 0)
    y0 = fm.matmul_transpose(x)
    options("gemm_strip", w)
    y1 = fm.matmul_transpose(x)
    assert torch.equal(y0, y1) and torch.equal(y1, y1.T)
    assert rel_fro(y1, x.float() @ x.float().T) <= 1e-2
    _lib.device_status()


def test_concurrent_streams_keep_their_own_scratch():
    """Two streams running the balanced schedule at the same time each use the scratch of their
    own stream: both results equal the single-stream result bit for bit."""
    m, k = 3328, 5120
    x = (torch.randn(m, k, device=DEV, generator=torch.Generator(device=DEV).manual_seed(6)) / k ** 0.5).bfloat16()
    ref = fm.matmul_transpose(x)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    torch.cuda.synchronize()
    for _ in range(3):
        for st in (s1, s2):
            with torch.cuda.stream(st):
                outs.append(fm.matmul_transpose(x))
    torch.cuda.synchronize()
    assert all(torch.equal(o, ref) for o in outs)
    _lib.device_status()


@pytest.mark.parametrize("pdl", [0, 1])
def test_dependent_launches_see_their_predecessor(pdl, options):
    """A chain of products, each reading the previous one's output, with and without programmatic
    dependent launch: the early-started kernel must not read before its predecessor is done."""
    options("pdl", pdl)
    x = (torch.randn(768, 768, device=DEV, generator=torch.Generator(device=DEV).manual_seed(8)) / 28).bfloat16()
    ref = x
    for _ in range(6):
        ref = (ref.float() @ ref.float().T).bfloat16()
        ref = ref / ref.abs().max().clamp_min(1e-30).bfloat16()
    cur = x
    bufs = [torch.empty(768, 768, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    # no host synchronisation inside the chain; the scaling is a torch kernel between two of ours
    for i in range(6):
        fm.matmul_transpose_assign(cur, bufs[i % 2])
        cur = bufs[i % 2]
        cur.div_(cur.abs().max().clamp_min(1e-30))
    torch.cuda.synchronize()
    assert rel_fro(cur, ref) <= 2e-2
    chain = []
    for _ in range(2):      # back-to-back products without anything in between
        a = fm.matmul_transpose(x)
        b = fm.matmul_transpose(a)
        chain.append(fm.matmul_transpose(b))
    torch.cuda.synchronize()
    assert torch.equal(chain[0], chain[1])
    a = fm.matmul_transpose(x)
    torch.cuda.synchronize()
    b = fm.matmul_transpose(a)
    torch.cuda.synchronize()
    assert torch.equal(chain[0], fm.matmul_transpose(b))
    _lib.device_status()


@pytest.mark.parametrize("name,value", [("gemm_kb_per_stage", 1), ("gemm_kb_per_stage", 3), ("gemm_stages", 4),
                                        ("gemm_stages", 7), ("gemm_tma_store", 0), ("pdl_trigger", 1),
                                        ("pdl_trigger", 2), ("pdl", 0), ("gemm_l2_promotion", 0), ("gemm_tma_d", 0)])
def test_pipeline_and_store_switches_change_no_bit(name, value, options):
    """Ring depth, K blocks per stage, TMA or per-lane stores, dependent-launch trigger: all of
    them change how a tile is fed and written, none the order of any sum.  Symmetric product with
    ragged edges and a general product with addend and both outputs, against the defaults."""
    lib = _lib.lib
    g = torch.Generator(device=DEV).manual_seed(31)
    x = (torch.randn(2500, 1100 + 8, device=DEV, generator=g) / 33).bfloat16()[:, :1096]   # pitch 1104
    M, N, K = 1000, 1800, 520
    A = (torch.randn(M, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    B = torch.randn(N, K, device=DEV, generator=g).bfloat16()
    D = torch.randn(M, N, device=DEV, generator=g).bfloat16()

    def run():
        y = fm.matmul_transpose(x)
        C = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        CT = torch.full((N, M), float("nan"), device=DEV, dtype=torch.bfloat16)
        _lib.check(lib.fm_gemm_nt(A.data_ptr(), K, B.data_ptr(), K, M, N, K, D.data_ptr(), N, 3.4445, 1.0,
                                  C.data_ptr(), N, CT.data_ptr(), M, 0, 0, 0))
        return y, C, CT

    options("gemm_impl", 2)
    ref = run()
    options(name, value)
    got = run()
    for a, b in zip(ref, got):
        assert not torch.isnan(a).any() and torch.equal(a, b)
    assert torch.equal(got[2], got[1].T)
    _lib.device_status()


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_tile_shapes_change_no_bit(bn, options):
    """A tile's shape decides who computes an output element, not the order of its sum over K:
    the single-CTA kernel with 128 x 64, 128 x 128 and 128 x 256 tiles gives the bits of the
    CTA-pair kernel, for a symmetric product and a general one with addend and both outputs."""
    lib = _lib.lib
    g = torch.Generator(device=DEV).manual_seed(37)
    x = (torch.randn(900, 1096, device=DEV, generator=g) / 33).bfloat16()
    M, N, K = 520, 712, 328
    A = (torch.randn(M, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    B = torch.randn(N, K, device=DEV, generator=g).bfloat16()
    D = torch.randn(M, N, device=DEV, generator=g).bfloat16()

    def run():
        y = fm.matmul_transpose(x)
        C = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        CT = torch.full((N, M), float("nan"), device=DEV, dtype=torch.bfloat16)
        _lib.check(lib.fm_gemm_nt(A.data_ptr(), K, B.data_ptr(), K, M, N, K, D.data_ptr(), N, 3.4445, 1.0,
                                  C.data_ptr(), N, CT.data_ptr(), M, 0, 0, 0))
        return y, C, CT

    options("gemm_impl", 2)
    ref = run()
    options("gemm_impl", 1)
    options("gemm_bn", bn)
    got = run()
    for a, b in zip(ref, got):
        assert not torch.isnan(a).any() and torch.equal(a, b)
    _lib.device_status()


def test_empty_and_degenerate():
    assert fm.matmul_transpose(torch.empty(0, 16, device=DEV, dtype=torch.bfloat16)).shape == (0, 0)
    y = fm.matmul_transpose(torch.empty(5, 0, device=DEV, dtype=torch.bfloat16))
    assert y.shape == (5, 5) and (y == 0).all()


def test_assertions_like_reference():
    x = torch.randn(16, 16, device=DEV).bfloat16()
    with pytest.raises(AssertionError, match="same data type"):
        fm.matmul_transpose_assign(x, torch.empty(16, 16, device=DEV))
    with pytest.raises(AssertionError, match="must be a 2D tensor"):
        fm.matmul_transpose_assign(x[0], torch.empty(16, 16, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="First dimension"):
        fm.matmul_transpose_assign(x, torch.empty(8, 8, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="First dimension"):
        fm.matmul_transpose_assign(x, torch.empty(16, 8, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(AssertionError, match="must be a CUDA tensor"):
        fm.matmul_transpose_assign(x, torch.empty(16, 16, dtype=torch.bfloat16))


def test_gemm_nt_epilogue_matches_torch_rounding_points():
    """C = round(round(a*D) + round(acc)) and its transposed copy, as `a*X + B@X` rounds."""
    lib = _lib.lib
    for (M, N, K) in ((128, 128, 64), (384, 200, 136), (1024, 2048, 1024)):
        A = (torch.randn(M, K, device=DEV) / K ** 0.5).bfloat16()
        B = torch.randn(N, K, device=DEV).bfloat16()
        D = torch.randn(M, N, device=DEV).bfloat16()
        C = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        CT = torch.full((N, M), float("nan"), device=DEV, dtype=torch.bfloat16)
        _lib.check(lib.fm_gemm_nt(A.data_ptr(), K, B.data_ptr(), K, M, N, K, D.data_ptr(), N, 3.4445,
                                  1.0, C.data_ptr(), N, CT.data_ptr(), M, 0, 0, 0))
        ref = 3.4445 * D + A @ B.T          # torch: three bf16 results
        assert torch.equal(CT, C.T)
        assert rel_fro(C, ref) <= 2e-3
        assert (C != ref).float().mean().item() < 1e-3
    _lib.device_status()
