// Exact-fp32 symmetric rank-k update  y = x x^T  on the FFMA pipes.
// Correctness path, not a throughput path: it serves f32 inputs (TF32 tensor cores cannot meet a
// 1e-5 tolerance) and 16-bit inputs whose layout TMA cannot address (K % 8 != 0, misaligned base).
// Same schedule idea as the tensor-core kernel: only tile pairs on or above the diagonal are
// computed and every tile is stored twice, so y is bitwise symmetric
// (reference behaviour: flash_muon/matmul_transpose_triton.py:43-44, :63-75).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemm_tc.cuh"

namespace fm {
namespace {

constexpr int TS = 64;   // tile edge
constexpr int TK = 16;   // k slab

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
syrk_simt_kernel(const T* __restrict__ x, T* __restrict__ y, int M, int K, long long ldx,
                 long long ldy_r, long long ldy_c) {
  __shared__ float As[TK][TS + 1];
  __shared__ float Bs[TK][TS + 1];
  // linear block index -> (bi <= bj)
  const int t = blockIdx.x;
  int bj = (int)((sqrtf(8.f * (float)t + 1.f) - 1.f) * 0.5f);
  while ((long long)(bj + 1) * (bj + 2) / 2 <= t) ++bj;
  while ((long long)bj * (bj + 1) / 2 > t) --bj;
  const int bi = t - bj * (bj + 1) / 2;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int r0 = bi * TS, c0 = bj * TS;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += TK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      const int rr = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      const int ra = r0 + rr, rb = c0 + rr;
      As[kk][rr] = (ra < M && k < K) ? to_f<T>(x[(long long)ra * ldx + k]) : 0.f;
      Bs[kk][rr] = (rb < M && k < K) ? to_f<T>(x[(long long)rb * ldx + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  const bool diag = (bi == bj);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + tx * 4 + j;
      if (c >= M) continue;
      if (diag && c < r) continue;
      const T v = from_f<T>(acc[i][j]);
      y[(long long)r * ldy_r + (long long)c * ldy_c] = v;
      if (c != r) y[(long long)c * ldy_r + (long long)r * ldy_c] = v;
    }
  }
}

}  // namespace

int syrk_simt(const void* x, void* y, int64_t M, int64_t K, int64_t ldx, int64_t ldy_row,
              int64_t ldy_col, int dtype, cudaStream_t stream) {
  if (M <= 0 || K <= 0 || M > (1 << 24) || K > (1 << 30))
    return fail(FM_ERR_INVALID, "bad extents M=%lld K=%lld", (long long)M, (long long)K);
  const long long T = (M + TS - 1) / TS;
  const long long blocks = T * (T + 1) / 2;
  if (blocks > 0x7fffffffLL) return fail(FM_ERR_UNSUPPORTED, "matrix too large for the FFMA path");
  const dim3 grid((unsigned)blocks);
  switch (dtype) {
    case FM_F32:
      syrk_simt_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)y, (int)M, (int)K,
                                                        ldx, ldy_row, ldy_col);
      break;
    case FM_BF16:
      syrk_simt_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
          (const __nv_bfloat16*)x, (__nv_bfloat16*)y, (int)M, (int)K, ldx, ldy_row, ldy_col);
      break;
    case FM_F16:
      syrk_simt_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)x, (__half*)y, (int)M,
                                                         (int)K, ldx, ldy_row, ldy_col);
      break;
    default:
      return fail(FM_ERR_UNSUPPORTED, "unknown dtype %d", dtype);
  }
  FM_CUDA_CHECK(cudaGetLastError());
  return FM_OK;
}

}  // namespace fm
