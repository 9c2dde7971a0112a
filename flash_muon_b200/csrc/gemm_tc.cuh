// Internal interface of the tcgen05 GEMM family (see gemm_tc.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fm {

struct GemmArgs {
  int dtype = 0;             // FM_BF16 or FM_F16
  const void* A = nullptr;   // [M,K] row-major, row pitch lda
  int64_t lda = 0;
  const void* B = nullptr;   // [N,K] row-major, row pitch ldb
  int64_t ldb = 0;
  int64_t M = 0, N = 0, K = 0;
  int sym = 0;               // 1: A == B, triangular schedule, mirrored store through CT
  const void* D = nullptr;   // optional addend [M,N], row pitch ldd
  int64_t ldd = 0;
  float alpha = 0.f, beta = 1.f;
  int precise = 0;
  void* C = nullptr;         // element (r,c) at C[r*ldc_r + c*ldc_c]
  int64_t ldc_r = 0, ldc_c = 1;
  void* CT = nullptr;        // element (r,c) at CT[c*ldt_r + r*ldt_c]
  int64_t ldt_r = 0, ldt_c = 1;
  // Batched launch: `batch` problems of identical extents.  Problem g reads rows
  // [g*a_batch_rows, +M) of A and [g*b_batch_rows, +N) of B (the operands of all problems are
  // stacked along the rows of one allocation each) and addresses D, C, CT at g*{d,c,t}_batch
  // elements from their bases; with c_tab (host array of `batch` pointers) the direct output of
  // problem g goes to c_tab[g] instead.
  int batch = 1;
  int64_t a_batch_rows = 0, b_batch_rows = 0;
  int64_t d_batch = 0, c_batch = 0, t_batch = 0;
  void* const* c_tab = nullptr;
  // Scratch for the balanced tail of long tile lists (may be null: tiles are then dealt whole).
  // gemm_sk_bytes() bytes, 256-byte aligned, owned by the caller; launches that may overlap on
  // the GPU need distinct scratch.
  void* sk_ws = nullptr;
  size_t sk_bytes = 0;
};

// Bytes of scratch with which a product of these extents runs the balanced tail (0: it never
// would, whatever scratch is offered).
size_t gemm_sk_bytes(int dtype, int64_t M, int64_t N, int64_t K, int sym);

// Validates, encodes the tensor maps and enqueues the kernel on `stream`.
int gemm_tc(const GemmArgs& args, cudaStream_t stream);

// CTA-pair (cluster of two) variant on 256 x 256 tiles, gemm_tc2.cu.
struct GemmParams;
int gemm_tc2_tiles(int64_t M, int64_t N, int sym);
int gemm_tc2_max_pairs(int dtype);
int gemm_tc2_launch(int dtype, const CUtensorMap& tmA, const CUtensorMap& tmB,
                    const CUtensorMap& tmC, const CUtensorMap& tmT, const CUtensorMap& tmD,
                    GemmParams& p, void* sk_ws, size_t sk_bytes, cudaStream_t stream);
size_t gemm_tc2_sk_bytes(int dtype, int64_t M, int64_t N, int64_t K, int sym);

// Exact-fp32 FFMA symmetric rank-k update for f32 inputs and layouts TMA cannot address.
int syrk_simt(const void* x, void* y, int64_t M, int64_t K, int64_t ldx, int64_t ldy_row,
              int64_t ldy_col, int dtype, cudaStream_t stream);

}  // namespace fm
