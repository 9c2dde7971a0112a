// Tensor-core GEMM family of the Muon hot path for sm_100a:
//   C[M,N] = A[M,K] * B[N,K]^T  (both operands row-major = K-major), fp32 accumulation in TMEM,
//   fused epilogue  out = round(round(alpha*D) + round(beta*round(acc)))  and an optional
//   transposed second store.
// With sym != 0 the kernel is the symmetric rank-k update X X^T: a persistent scheduler walks
// only the tile pairs on or above the diagonal and the epilogue writes every tile twice
// (direct + mirrored) from the same rounded registers, so the result is bitwise symmetric.
// It stands in for the reference's Triton kernel (flash_muon/matmul_transpose_triton.py:19-75)
// and for the cuBLAS call + elementwise kernels of flash_muon/muon.py:27-29.
//
// Structure of one CTA (192 threads, one CTA per SM, persistent over a static tile list):
//   warp 0     : TMA producer  (one lane) -- 64-column operand slabs into a ring of smem stages
//   warp 1     : MMA issuer    (one lane) -- tcgen05.mma 128 x ncols x 16, accumulators in TMEM,
//                double-buffered so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..5 : epilogue -- tcgen05.ld 32 lanes x 32 columns, rounding-faithful arithmetic,
//                global stores (direct rows + transposed columns)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "tile_schedule.cuh"

namespace fm {

namespace {

constexpr int BM = 128;          // rows of an output tile = UMMA M
constexpr int BK = 64;           // K extent of one smem stage: 64 x 2 B = one 128-byte swizzle row
constexpr int UMMA_K = 16;       // K of one tcgen05.mma for 16-bit operands
constexpr int kThreads = 192;
constexpr int kSlabBytes = 128 * BK * 2;  // one 128-row operand slab = one TMA box (16 KiB)

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kStageBytes = kSlabBytes + BN * BK * 2;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators of BN fp32 columns
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kNumBars * 8 + 16 + 1024;
};

template <typename T, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t bar_base = smem_base + C::kStages * C::kStageBytes;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::kStages * C::kStageBytes + C::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * C::kStages + 2 + a); };
  auto a_smem = [&](int s) { return smem_base + s * C::kStageBytes; };
  auto b_smem = [&](int s) { return smem_base + s * C::kStageBytes + kSlabBytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 128);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Nothing above touches global memory: with programmatic stream serialization the set-up runs
  // while the previous kernel of the stream drains; from here on its results are visible.
  ptx::grid_dep_wait();
  const EpiPtrs ep = epilogue_ptrs(p, 0, (int)sizeof(T));

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      if ((int)blockIdx.x >= p.num_tiles) ptx::grid_dep_launch();
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        if (t + (int)gridDim.x >= p.num_tiles) ptx::grid_dep_launch();  // this CTA's last tile
        const Tile tl = decode_tile<BN>(p, t);
        // B arrives in boxes of min(BN, 128) rows (the box of tmB)
        const int nb = BN < 128 ? 1 : (tl.ncols >> 7);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          ptx::mbar_expect_tx(full_bar(s), (uint32_t)(kSlabBytes + tl.ncols * BK * 2));
          ptx::tma_load_2d(a_smem(s), &tmA, full_bar(s), kb * BK, tl.m0);
          for (int q = 0; q < nb; ++q)
            ptx::tma_load_2d(b_smem(s) + q * kSlabBytes, &tmB, full_bar(s), kb * BK,
                             tl.n0 + q * 128);
          if (++s == C::kStages) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        const Tile tl = decode_tile<BN>(p, t);
        if (!ptx::mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        const uint32_t idesc = ptx::make_idesc_f16(Num<T>::kFormat, BM, (uint32_t)tl.ncols);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t a_desc = ptx::make_kmajor_sw128_desc(a_smem(s));
          const uint64_t b_desc = ptx::make_kmajor_sw128_desc(b_smem(s));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 elements = 32 bytes inside the swizzled row = +2 in the
            // (address >> 4) field of the descriptor
            ptx::umma_f16(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                          (uint32_t)((kb | k) != 0));
          }
          ptx::umma_commit(empty_bar(s));  // frees the stage when these MMAs have read it
          if (++s == C::kStages) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(tfull_bar(acc));  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_ph = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      const Tile tl = decode_tile<BN>(p, t);
      const int row = tl.m0 + q * 32 + lane;
      const int nchunks = tl.ncols >> 5;
      // the addend does not depend on the accumulator: fetch the first chunk before waiting
      alignas(16) T dcur[32], dnext[32];
      epilogue_load_d<T>(p, ep, row, tl.n0, dcur);
      bool ok = ptx::mbar_wait(tfull_bar(acc), acc_ph, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      for (int ch = 0; ch < nchunks; ++ch) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + ch * 32),
                           raw);
        if (ch + 1 < nchunks) epilogue_load_d<T>(p, ep, row, tl.n0 + (ch + 1) * 32, dnext);
        ptx::tmem_ld_wait();
        epilogue_store<T>(p, ep, raw, dcur, row, tl.n0 + ch * 32, tl.bi);
        if (p.D != nullptr) {
#pragma unroll
          for (int v = 0; v < 4; ++v)
            reinterpret_cast<uint4*>(dcur)[v] = reinterpret_cast<const uint4*>(dnext)[v];
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    // Some wait ran out: give copies and MMAs still in flight a bounded time to land before the
    // shared memory and TMEM of this CTA are released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.err, 0x47450000u | (unsigned)blockIdx.x);
}

template <typename T, int BN>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  FM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    FM_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel<T, BN>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured[dev] = true;
  }
  p.num_tiles = count_tiles<BN>(p.M, p.N, p.sym);
  const int sms = sm_count();
  if (sms <= 0) return fail(FM_ERR_CUDA, "could not query the SM count");
  const int grid = p.num_tiles < sms ? p.num_tiles : sms;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().pdl ? 1 : 0;
  FM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<T, BN>, tmA, tmB, p));
  return FM_OK;
}

}  // namespace

int gemm_tc(const GemmArgs& a, cudaStream_t stream) {
  if (a.dtype != FM_BF16 && a.dtype != FM_F16)
    return fail(FM_ERR_UNSUPPORTED, "tensor-core GEMM covers bf16 and f16 only");
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.M > (1 << 30) || a.N > (1 << 30) || a.K > (1 << 30))
    return fail(FM_ERR_INVALID, "bad GEMM extents M=%lld N=%lld K=%lld", (long long)a.M,
                (long long)a.N, (long long)a.K);
  if (!a.A || !a.B || (!a.C && !a.CT)) return fail(FM_ERR_INVALID, "null operand or no output");
  if (a.sym && (a.M != a.N)) return fail(FM_ERR_INVALID, "symmetric mode needs M == N");
  if (a.batch < 1 || a.batch > kMaxGemmBatch)
    return fail(FM_ERR_INVALID, "batch must be 1..%d, got %d", kMaxGemmBatch, a.batch);
  if (a.batch > 1 && (a.a_batch_rows < a.M || a.b_batch_rows < a.N))
    return fail(FM_ERR_INVALID, "stacked operands overlap: batch rows smaller than the extents");

  // operands of a batch are stacked along the rows: one tensor map covers all of them, rows
  // past the last problem read as zeros
  const uint64_t rows_a = (uint64_t)(a.batch - 1) * (uint64_t)a.a_batch_rows + (uint64_t)a.M;
  const uint64_t rows_b = (uint64_t)(a.batch - 1) * (uint64_t)a.b_batch_rows + (uint64_t)a.N;
  CUtensorMap tmA, tmB;
  int rc = encode_tmap_2d(&tmA, a.dtype, a.A, (uint64_t)a.K, rows_a, (uint64_t)a.lda, BK, 128);
  if (rc != FM_OK) return rc;
  rc = encode_tmap_2d(&tmB, a.dtype, a.B, (uint64_t)a.K, rows_b, (uint64_t)a.ldb, BK, 128);
  if (rc != FM_OK) return rc;

  GemmParams p;
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.sym = a.sym;
  p.tiles_m = (p.M + 127) / 128;
  p.tiles_n = 0;
  p.num_kb = (p.K + BK - 1) / BK;
  p.num_tiles = 0;
  p.D = a.D; p.ldd = a.ldd;
  p.C = a.C; p.ldc_r = a.ldc_r; p.ldc_c = a.ldc_c;
  p.CT = a.CT; p.ldt_r = a.ldt_r; p.ldt_c = a.ldt_c;
  p.alpha = a.alpha; p.beta = a.beta;
  p.precise = a.precise;
  p.d_vec = (a.D != nullptr) && ((reinterpret_cast<uintptr_t>(a.D) & 15u) == 0) && (a.ldd % 8 == 0);
  p.c_vec = (a.C != nullptr) && ((reinterpret_cast<uintptr_t>(a.C) & 15u) == 0) &&
            (a.ldc_c == 1) && (a.ldc_r % 8 == 0);
  p.t_pack = (a.CT != nullptr) && (a.ldt_c == 1) && (a.ldt_r % 2 == 0) &&
             ((reinterpret_cast<uintptr_t>(a.CT) & 3u) == 0);
  p.stages = 0;
  p.kb_per_stage = 1;
  p.early_trigger = 1;
  p.strip_w = 0;
  p.sk_dp_tiles = 0; p.sk_per = 0; p.sk_total = 0; p.sk_ws = nullptr; p.sk_cnt = nullptr;
  p.batch = a.batch;
  p.tiles_per_batch = 0;
  p.a_batch_rows = (int)a.a_batch_rows; p.b_batch_rows = (int)a.b_batch_rows;
  p.d_batch = a.d_batch; p.c_batch = a.c_batch; p.t_batch = a.t_batch;
  p.use_c_tab = (a.batch > 1 && a.c_tab != nullptr) ? 1 : 0;
  for (int g = 0; g < kMaxGemmBatch; ++g) p.c_tab[g] = (p.use_c_tab && g < a.batch) ? a.c_tab[g] : nullptr;
  if (p.use_c_tab) {  // the fast store path must hold for every problem's output
    p.c_vec = (a.ldc_c == 1) && (a.ldc_r % 8 == 0);
    for (int g = 0; g < a.batch; ++g) {
      if (!a.c_tab[g]) return fail(FM_ERR_INVALID, "null output pointer for problem %d", g);
      if ((reinterpret_cast<uintptr_t>(a.c_tab[g]) & 15u) != 0) p.c_vec = 0;
    }
  } else if (a.batch > 1) {  // per-problem offsets must keep the alignment the fast paths assume
    if (a.D && a.d_batch % 8 != 0) p.d_vec = 0;
    if (a.C && a.c_batch % 8 != 0) p.c_vec = 0;
    if (a.CT && a.t_batch % 2 != 0) p.t_pack = 0;
  }
  if (a.batch > 1 && p.use_c_tab && a.D && a.d_batch % 8 != 0) p.d_vec = 0;
  if (a.batch > 1 && p.use_c_tab && a.CT && a.t_batch % 2 != 0) p.t_pack = 0;
  p.tma_store = 0;
  p.tma_d = 0;
  p.c_batch_rows = p.t_batch_rows = p.d_batch_rows = 0;
  p.err = device_error_word();
  if (!p.err) return fail(FM_ERR_CUDA, "no current CUDA device");

  // CTA pairs on 256 x 256 tiles when there are enough tiles to occupy most of the pairs;
  // otherwise single CTAs on 128 x 256 or 128 x 128 tiles (more, smaller units of work).
  // A batch always runs on pairs (the single-CTA kernel has no batch dimension).
  int impl = 1;
  {
    const int tiles2 = gemm_tc2_tiles(a.M, a.N, a.sym) * a.batch;
    const int pairs = gemm_tc2_max_pairs(a.dtype);
    if (pairs > 0 && tiles2 * 10 >= pairs * 6) impl = 2;
    const int v = options().gemm_impl;
    if (v == 1 || (v == 2 && pairs > 0)) impl = v;
    if (a.batch > 1) {
      if (pairs <= 0) return fail(FM_ERR_CUDA, "no resident CTA pair possible for a batched GEMM");
      impl = 2;
    }
  }
  if (impl == 2) {
    // Outputs through TMA tile stores when every output is a matrix TMA can address: unit column
    // stride, 16-byte aligned base and pitch, one base for the whole batch, and (batch > 1) no
    // tile hanging over the edge of a problem into the rows of the next one.
    auto addressable = [](const void* ptr, int64_t ld_r, int64_t ld_c) {
      return ptr == nullptr || (ld_c == 1 && ld_r % 8 == 0 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0);
    };
    CUtensorMap tmC = tmA, tmT = tmA;  // placeholders unless the stores use them
    p.tma_store = 0;
    p.c_batch_rows = p.t_batch_rows = 0;
    bool ok = options().gemm_tma_store && !p.use_c_tab && addressable(a.C, a.ldc_r, a.ldc_c) &&
              addressable(a.CT, a.ldt_r, a.ldt_c);
    if (ok && a.batch > 1) {
      ok = (a.M % 256 == 0) && (a.N % 256 == 0) && (!a.C || a.c_batch % a.ldc_r == 0) &&
           (!a.CT || a.t_batch % a.ldt_r == 0);
      if (ok) {
        p.c_batch_rows = a.C ? (int)(a.c_batch / a.ldc_r) : 0;
        p.t_batch_rows = a.CT ? (int)(a.t_batch / a.ldt_r) : 0;
      }
    }
    if (ok && a.C)
      ok = encode_tmap_2d(&tmC, a.dtype, a.C, (uint64_t)a.N,
                          (uint64_t)(a.batch - 1) * (uint64_t)p.c_batch_rows + (uint64_t)a.M,
                          (uint64_t)a.ldc_r, 64, 32, true) == FM_OK;
    if (ok && a.CT)
      ok = encode_tmap_2d(&tmT, a.dtype, a.CT, (uint64_t)a.M,
                          (uint64_t)(a.batch - 1) * (uint64_t)p.t_batch_rows + (uint64_t)a.N,
                          (uint64_t)a.ldt_r, 32, 64, false) == FM_OK;
    clear_error();
    p.tma_store = ok ? 1 : 0;
    // The addend by TMA tile loads as well (into the staging tiles of the stores, which then
    // carry C only; the transposed output goes back to per-lane stores): needs the tile stores
    // and an addend TMA can address, stacked like C when the launch is a batch.
    CUtensorMap tmD = tmA;
    p.tma_d = 0;
    p.d_batch_rows = 0;
    bool okd = ok && options().gemm_tma_d && a.D != nullptr && addressable(a.D, a.ldd, 1) &&
               (a.batch == 1 || a.d_batch % a.ldd == 0);
    if (okd) {
      p.d_batch_rows = a.batch > 1 ? (int)(a.d_batch / a.ldd) : 0;
      okd = encode_tmap_2d(&tmD, a.dtype, a.D, (uint64_t)a.N,
                           (uint64_t)(a.batch - 1) * (uint64_t)p.d_batch_rows + (uint64_t)a.M,
                           (uint64_t)a.ldd, 64, 32, true) == FM_OK;
      clear_error();
    }
    p.tma_d = okd ? 1 : 0;
    return gemm_tc2_launch(a.dtype, tmA, tmB, tmC, tmT, tmD, p, a.sk_ws, a.sk_bytes, stream);
  }

  // Tile width: 256 columns (less operand traffic per FLOP) unless that leaves most SMs idle;
  // 64 columns when even 128 x 128 tiles occupy less than half of the SMs (what bounds such a
  // launch is what one SM can load and store, so more, smaller units of work finish sooner).
  int bn = 256;
  const int sms = sm_count();
  if (count_tiles<256>(p.M, p.N, p.sym) < sms) bn = 128;
  if (bn == 128 && 2 * count_tiles<128>(p.M, p.N, p.sym) <= sms) bn = 64;
  {
    const int v = options().gemm_bn;
    if (v == 64 || v == 128 || v == 256) bn = v;
  }
  if (bn == 64) {  // B in boxes of 64 rows
    rc = encode_tmap_2d(&tmB, a.dtype, a.B, (uint64_t)a.K, rows_b, (uint64_t)a.ldb, BK, 64);
    if (rc != FM_OK) return rc;
  }
  if (a.dtype == FM_BF16)
    return bn == 256   ? launch<__nv_bfloat16, 256>(tmA, tmB, p, stream)
           : bn == 128 ? launch<__nv_bfloat16, 128>(tmA, tmB, p, stream)
                       : launch<__nv_bfloat16, 64>(tmA, tmB, p, stream);
  return bn == 256   ? launch<__half, 256>(tmA, tmB, p, stream)
         : bn == 128 ? launch<__half, 128>(tmA, tmB, p, stream)
                     : launch<__half, 64>(tmA, tmB, p, stream);
}

size_t gemm_sk_bytes(int dtype, int64_t M, int64_t N, int64_t K, int sym) {
  if (dtype != FM_BF16 && dtype != FM_F16) return 0;
  if (options().gemm_impl == 1) return 0;
  return gemm_tc2_sk_bytes(dtype, M, N, K, sym);
}

}  // namespace fm
