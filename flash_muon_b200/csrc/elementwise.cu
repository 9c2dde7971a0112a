// HBM-bound kernels of the Muon hot path: Frobenius normalisation (with the transposed copy the
// GEMMs need), fused momentum + Nesterov, fused weight decay + scaled update.  All use 16-byte
// global accesses and grid sizes tied to the SM count; arithmetic keeps the reference's rounding
// points (torch's element kernels compute in fp32 and round once per op).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "muon_kernels.cuh"

namespace fm {
namespace {

constexpr int kNormBlocks = 1024;  // upper bound of partial sums (floats of scratch)

__device__ __forceinline__ void ptx_grid_dep_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename T> __device__ __forceinline__ float ld_f(T v);
template <> __device__ __forceinline__ float ld_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float ld_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T st_f(float v);
template <> __device__ __forceinline__ float st_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 st_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half st_f<__half>(float v) { return __float2half_rn(v); }

// value of the input after the reference's `G.bfloat16()` (flash_muon/muon.py:15)
template <typename T>
__device__ __forceinline__ float as_bf16_value(T v) {
  return __bfloat162float(__float2bfloat16_rn(ld_f<T>(v)));
}
template <>
__device__ __forceinline__ float as_bf16_value<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

__device__ __forceinline__ float block_sum_256(float v, float* red /* 8 floats */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) s += red[w];  // same order in every thread and every block
  return s;
}

// Matrices of one normalisation launch (blockIdx.y selects one).  `g` is [rows, cols] with row
// pitch ldg; xd receives the scaled copy in the same orientation, xt its transpose (either may be
// null); `partials` holds norm_blocks(rows * cols) partial sums of squares.
constexpr int kMaxNormBatch = 16;
struct NormEntry {
  const void* g;
  long long rows, cols, ldg;
  __nv_bfloat16* xd;
  long long ldxd;
  __nv_bfloat16* xt;
  long long ldxt;
  float* partials;
};
struct NormTable {
  NormEntry e[kMaxNormBatch];
};

// Blocks (= partial sums) of the sum-of-squares pass over n elements.  The fused momentum kernel
// uses the same grid and the same element-to-thread assignment, so both produce the same
// partial sums bit for bit.
__host__ __device__ inline int norm_blocks(long long n) {
  long long nb = (n + 8191) / 8192;
  if (nb > kNormBlocks) nb = kNormBlocks;
  if (nb < 1) nb = 1;
  return (int)nb;
}

// ---------------------------------------------------------------- sum of squares, partials
template <typename T>
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const __grid_constant__ NormTable tab, int vec_ok) {
  __shared__ float red[8];
  constexpr int V = 16 / sizeof(T);
  const NormEntry& en = tab.e[blockIdx.y];
  const T* __restrict__ g = reinterpret_cast<const T*>(en.g);
  const long long rows = en.rows, cols = en.cols, ldg = en.ldg;
  float* __restrict__ partials = en.partials;
  float s = 0.f;
  const long long n = rows * cols;
  if (vec_ok) {  // contiguous, 16-byte aligned, n % V == 0
    const long long nv = n / V;
    const uint4* g4 = reinterpret_cast<const uint4*>(g);
#pragma unroll 4
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < nv;
         i += (long long)gridDim.x * 256) {
      const uint4 raw = __ldg(g4 + i);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float f = as_bf16_value<T>(e[j]);
        s = fmaf(f, f, s);
      }
    }
  } else {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n;
         i += (long long)gridDim.x * 256) {
      const long long r = i / cols, c = i - r * cols;
      const float f = as_bf16_value<T>(g[r * ldg + c]);
      s = fmaf(f, f, s);
    }
  }
  const float tot = block_sum_256(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = tot;
}

// ---------------------------------------------------------------- scale + transposed copy
// One 64x64 tile of G per block.  Every block first folds the partial sums in one fixed order, so
// all blocks derive the same denominator without a third launch.
template <typename T>
__global__ void __launch_bounds__(256)
scale_transpose_kernel(const __grid_constant__ NormTable tab, int nparts) {
  __shared__ float red[8];
  __shared__ __nv_bfloat16 tile[64][66];
  ptx_grid_dep_launch();  // the GEMM that follows may set itself up while this kernel runs
  const NormEntry& en = tab.e[blockIdx.y];
  const T* __restrict__ g = reinterpret_cast<const T*>(en.g);
  const long long rows = en.rows, cols = en.cols, ldg = en.ldg;
  const float* __restrict__ partials = en.partials;
  __nv_bfloat16* __restrict__ xd = en.xd;
  __nv_bfloat16* __restrict__ xt = en.xt;
  const long long ldxd = en.ldxd, ldxt = en.ldxt;
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 256) s += partials[i];
  const float total = block_sum_256(s, red);
  // torch: norm -> bf16, (+1e-7) -> bf16, x / that -> bf16  (flash_muon/muon.py:23)
  const float d = __bfloat162float(__float2bfloat16_rn(sqrtf(total)));
  const float dp = __bfloat162float(__float2bfloat16_rn(d + 1e-7f));

  const long long tiles_c = (cols + 63) / 64;
  const long long tr = blockIdx.x / tiles_c, tc = blockIdx.x - tr * tiles_c;
  const long long r0 = tr * 64, c0 = tc * 64;
  {
    const int rr = threadIdx.x >> 2, cs = (threadIdx.x & 3) * 16;
    const long long r = r0 + rr;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const long long c = c0 + cs + e;
      __nv_bfloat16 q = __float2bfloat16_rn(0.f);
      if (r < rows && c < cols) {
        q = __float2bfloat16_rn(as_bf16_value<T>(g[r * ldg + c]) / dp);
        if (xd) xd[r * ldxd + c] = q;
      }
      tile[rr][cs + e] = q;
    }
  }
  if (xt == nullptr) return;
  __syncthreads();
  {
    const int cc = threadIdx.x >> 2, rs = (threadIdx.x & 3) * 16;
    const long long c = c0 + cc;
    if (c < cols) {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const long long r = r0 + rs + e;
        if (r < rows) xt[c * ldxt + r] = tile[rs + e][cc];
      }
    }
  }
}


// Fast path of the kernel above for matrices whose rows and columns are multiples of 64 and whose
// pointers and pitches allow 16-byte accesses.  A block walks tiles of 128 rows x 64 columns
// (blockIdx.x, + gridDim.x, ...): it folds the partial sums once, keeps the loads of its next tile
// in flight while it writes the current one, writes X in 128-byte and the transposed copy in
// 256-byte row segments, every access a full 16-byte vector.
constexpr int kScaleTileRows = 128;

template <typename T>
__global__ void __launch_bounds__(256, sizeof(T) == 2 ? 4 : 2)
scale_transpose_vec_kernel(const __grid_constant__ NormTable tab, int nparts) {
  ptx_grid_dep_launch();
  const NormEntry& en = tab.e[blockIdx.y];
  const T* __restrict__ g = reinterpret_cast<const T*>(en.g);
  const long long rows = en.rows, cols = en.cols, ldg = en.ldg;
  const float* __restrict__ partials = en.partials;
  __nv_bfloat16* __restrict__ xd = en.xd;
  __nv_bfloat16* __restrict__ xt = en.xt;
  const long long ldxd = en.ldxd, ldxt = en.ldxt;
  constexpr int R = kScaleTileRows, C = 64;
  constexpr int V = 16 / sizeof(T);        // input elements per 16-byte load
  constexpr int CHUNKS = C / V;            // loads per tile row
  constexpr int LOADS = (R * CHUNKS) / 256;
  __shared__ float red[8];
  // Staging tile, [R][C] bf16 = [R][32] words.  The 8-element column groups of a row are
  // XOR-swizzled with the row group, and the halves of a group are swapped in rows >= 64 (rows r
  // and r + 64 share a group), so that both the row-wise 16-byte stores and the column-wise
  // 4-byte gathers below are free of bank conflicts.
  __shared__ __align__(16) uint32_t tile[R][C / 2];
  auto swz = [](int r, int c) {  // element column c of row r -> element position in the row
    return (((c >> 3) ^ ((r >> 3) & 7)) << 3) | ((c & 7) ^ (((r >> 6) & 1) << 2));
  };
  // (32-bit tile arithmetic: a 64-bit division per tile costs as much as the tile's conversions)
  const unsigned tiles_c = (unsigned)(cols / C);
  const unsigned tiles = (unsigned)((rows + R - 1) / R) * tiles_c;   // < 2^31, checked by the host

  // Per-thread constants of the tile walk: the thread's column chunk is the same in all of its
  // LOADS vectors, its rows are RSTEP apart; in the transposed phase its 8 rows are the same for
  // all of its column pairs, which are 2 * PSTEP columns apart.
  constexpr int RSTEP = 256 / CHUNKS;
  constexpr int PSTEP = 256 / (R / 8);
  const int rr0 = threadIdx.x / CHUNKS, cc = (threadIdx.x % CHUNKS) * V;
  const int cp0 = threadIdx.x / (R / 8), rs = (threadIdx.x % (R / 8)) * 8;
  const long long g_off = (long long)rr0 * ldg + cc, g_step = (long long)RSTEP * ldg;
  const long long d_off = (long long)rr0 * ldxd + cc, d_step = (long long)RSTEP * ldxd;
  const long long t_off = (long long)(2 * cp0) * ldxt + rs, t_step = (long long)(2 * PSTEP) * ldxt;

  uint4 raw[LOADS], nxt[LOADS];
  auto fetch = [&](unsigned t, uint4* dst) {
    const unsigned tr = t / tiles_c, tc = t - tr * tiles_c;
    const long long r0 = (long long)tr * R;
    const T* src = g + r0 * ldg + (long long)tc * C + g_off;
#pragma unroll
    for (int i = 0; i < LOADS; ++i)
      dst[i] = (r0 + rr0 + i * RSTEP < rows) ? __ldg(reinterpret_cast<const uint4*>(src + i * g_step))
                                             : make_uint4(0u, 0u, 0u, 0u);
  };
  unsigned t = blockIdx.x;
  // the first tile's loads go out first; folding the partial sums hides under their latency
  if (t < tiles) fetch(t, raw);
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 256) s += partials[i];
  const float total = block_sum_256(s, red);
  // torch: norm -> bf16, (+1e-7) -> bf16, x / that -> bf16  (flash_muon/muon.py:23)
  const float d = __bfloat162float(__float2bfloat16_rn(sqrtf(total)));
  const float dp = __bfloat162float(__float2bfloat16_rn(d + 1e-7f));
  const float rdp = 1.f / dp;

  for (; t < tiles; t += gridDim.x) {
    const unsigned tn = t + gridDim.x;
    if (tn < tiles) fetch(tn, nxt);
    const unsigned tr = t / tiles_c, tc = t - tr * tiles_c;
    const long long r0 = (long long)tr * R, c0 = (long long)tc * C;
    __nv_bfloat16* const xd_t = xd + r0 * ldxd + c0 + d_off;
#pragma unroll
    for (int i = 0; i < LOADS; ++i) {
      const int rr = rr0 + i * RSTEP;
      const T* e = reinterpret_cast<const T*>(&raw[i]);
      // x * (1 / dp) lies within 2.5 fp32 ulps of x / dp, hence within 2 ulps of the correctly
      // rounded quotient: both round to the same bf16 value unless the product is within 2 ulps
      // of the midpoint between two bf16 values (low 16 bits 0x7ffe .. 0x8002).  A vector with an
      // element whose low bits fall in 0x7ffc .. 0x8003 (one vector in 1000) takes the division.
      float y[V];
      bool near_mid = false;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        y[j] = as_bf16_value<T>(e[j]) * rdp;
        near_mid |= ((__float_as_uint(y[j]) + 4u) & 0xfff8u) == 0x8000u;
      }
      if (near_mid) {  // one vector in 1000
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = as_bf16_value<T>(e[j]) / dp;
      }
      alignas(16) __nv_bfloat162 q[V / 2];
#pragma unroll
      for (int j = 0; j < V / 2; ++j) q[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
      if (xd != nullptr && r0 + rr < rows) {
        if (V == 8) *reinterpret_cast<uint4*>(xd_t + i * d_step) = *reinterpret_cast<uint4*>(q);
        else *reinterpret_cast<uint2*>(xd_t + i * d_step) = *reinterpret_cast<uint2*>(q);
      }
      if (V == 8) {
        const uint4 v = *reinterpret_cast<uint4*>(q);
        *reinterpret_cast<uint4*>(&tile[rr][(swz(rr, cc) & ~7) >> 1]) =
            (rr & 64) ? make_uint4(v.z, v.w, v.x, v.y) : v;
      } else {
        *reinterpret_cast<uint2*>(&tile[rr][swz(rr, cc) >> 1]) = *reinterpret_cast<uint2*>(q);
      }
    }
    if (xt != nullptr) {
      __syncthreads();
      // A thread takes two neighbouring columns (one 4-byte word per row) of 8 rows and writes
      // two 16-byte vectors of the transposed copy.
      __nv_bfloat16* const xt_t = xt + c0 * ldxt + r0 + t_off;
#pragma unroll
      for (int i = 0; i < (R * C) / (256 * 16); ++i) {
        const int cp = cp0 + i * PSTEP;          // column pair; C/2 pairs x R/8 row groups
        const int word = swz(rs, 2 * cp) >> 1;   // the same for the 8 rows of a group
        uint32_t w[8];
#pragma unroll
        for (int e2 = 0; e2 < 8; ++e2) w[e2] = tile[rs + e2][word];
        if (r0 + rs < rows) {
          uint4 lo, hi;
          lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
          lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
          lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
          lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
          __nv_bfloat16* dst = xt_t + i * t_step;
          *reinterpret_cast<uint4*>(dst) = lo;
          *reinterpret_cast<uint4*>(dst + ldxt) = hi;
        }
      }
      __syncthreads();  // the next tile overwrites the staging tile
    }
#pragma unroll
    for (int i = 0; i < LOADS; ++i) raw[i] = nxt[i];
  }
}

// ---------------------------------------------------------------- momentum + Nesterov
// torch's lerp (element kernel in fp32): w < 0.5 ? a + w*(b-a) : b - (b-a)*(1-w)
__device__ __forceinline__ float lerp_f(float a, float b, float w) {
  return (fabsf(w) < 0.5f) ? a + w * (b - a) : b - (b - a) * (1.f - w);
}

// Tensors of one momentum launch (blockIdx.y selects one).  With `partials` the kernel also
// leaves the partial sums of squares of the values Newton-Schulz will read (the gradient after
// the Nesterov step, or the momentum buffer), saving the normalisation its own pass over them.
constexpr int kMaxMomentumBatch = 16;
struct MomentumTable {
  void* grad[kMaxMomentumBatch];
  void* buf[kMaxMomentumBatch];
  float* partials[kMaxMomentumBatch];
  long long n[kMaxMomentumBatch];
};

// kSumsq: the grid is norm_blocks(n) blocks and every thread walks the 16-byte vectors exactly
// as sumsq_partial_kernel does (same stride, same order of the fused multiply-adds, same block
// reduction), so partials[blockIdx.x] is bit for bit what that kernel would compute afterwards.
// Requires 16-byte aligned tensors with n a multiple of the vector width.
template <typename T, bool kSumsq>
__global__ void __launch_bounds__(256)
momentum_kernel(const __grid_constant__ MomentumTable tab, float w_buf, float w_grad, int nesterov,
                int vec_ok) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[8];
  T* __restrict__ grad = reinterpret_cast<T*>(tab.grad[blockIdx.y]);
  T* __restrict__ buf = reinterpret_cast<T*>(tab.buf[blockIdx.y]);
  const long long n = tab.n[blockIdx.y];
  const long long stride = (long long)gridDim.x * 256;
  float s = 0.f;
  if (vec_ok) {
    const long long nv = n / V;
    uint4* g4 = reinterpret_cast<uint4*>(grad);
    uint4* b4 = reinterpret_cast<uint4*>(buf);
#pragma unroll 4
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < nv; i += stride) {
      uint4 graw = g4[i], braw = b4[i];
      T* ge = reinterpret_cast<T*>(&graw);
      T* be = reinterpret_cast<T*>(&braw);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float gv = ld_f<T>(ge[j]);
        const T nb = st_f<T>(lerp_f(ld_f<T>(be[j]), gv, w_buf));
        be[j] = nb;
        if (nesterov) ge[j] = st_f<T>(lerp_f(gv, ld_f<T>(nb), w_grad));
        if (kSumsq) {
          const float f = as_bf16_value<T>(nesterov ? ge[j] : nb);
          s = fmaf(f, f, s);
        }
      }
      b4[i] = braw;
      if (nesterov) g4[i] = graw;
    }
    // tail
    for (long long i = nv * V + (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
      const float gv = ld_f<T>(grad[i]);
      const T nb = st_f<T>(lerp_f(ld_f<T>(buf[i]), gv, w_buf));
      buf[i] = nb;
      if (nesterov) grad[i] = st_f<T>(lerp_f(gv, ld_f<T>(nb), w_grad));
    }
  } else {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
      const float gv = ld_f<T>(grad[i]);
      const T nb = st_f<T>(lerp_f(ld_f<T>(buf[i]), gv, w_buf));
      buf[i] = nb;
      if (nesterov) grad[i] = st_f<T>(lerp_f(gv, ld_f<T>(nb), w_grad));
    }
  }
  if (kSumsq) {
    const float tot = block_sum_256(s, red);
    if (threadIdx.x == 0) tab.partials[blockIdx.y][blockIdx.x] = tot;
  }
}

// ---------------------------------------------------------------- decay + update, multi-tensor
// torch: mul_(scalar) is one fp32 multiply, add_(u, alpha) is a + alpha*b contracted to one fma;
// the intrinsics pin that shape so fp32 parameters (no rounding in between) match bit for bit.
constexpr int kMaxTensors = 32;
struct UpdateTable {
  void* p[kMaxTensors];
  const void* u[kMaxTensors];
  long long n[kMaxTensors];
  float alpha[kMaxTensors];
};

template <typename T>
__global__ void __launch_bounds__(256)
update_kernel(const UpdateTable tab, float decay) {
  constexpr int V = 8;  // elements per iteration: one 16-byte load of the bf16 update
  const int ti = blockIdx.y;
  T* __restrict__ p = reinterpret_cast<T*>(tab.p[ti]);
  const __nv_bfloat16* __restrict__ u = reinterpret_cast<const __nv_bfloat16*>(tab.u[ti]);
  const long long n = tab.n[ti];
  const float alpha = tab.alpha[ti];
  const long long stride = (long long)gridDim.x * 256;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) &&
                      ((reinterpret_cast<uintptr_t>(u) & 15u) == 0);
  long long done = 0;
  if (vec_ok) {
    const long long nv = n / V;
    const uint4* u4 = reinterpret_cast<const uint4*>(u);
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < nv; i += stride) {
      const uint4 uraw = __ldg(u4 + i);
      const __nv_bfloat16* ue = reinterpret_cast<const __nv_bfloat16*>(&uraw);
      alignas(16) T pv[V];
      if (sizeof(T) == 2) {
        *reinterpret_cast<uint4*>(pv) = reinterpret_cast<uint4*>(p)[i];
      } else {
        reinterpret_cast<uint4*>(pv)[0] = reinterpret_cast<uint4*>(p)[2 * i];
        reinterpret_cast<uint4*>(pv)[1] = reinterpret_cast<uint4*>(p)[2 * i + 1];
      }
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const T dec = st_f<T>(__fmul_rn(ld_f<T>(pv[j]), decay));
        pv[j] = st_f<T>(__fmaf_rn(alpha, __bfloat162float(ue[j]), ld_f<T>(dec)));
      }
      if (sizeof(T) == 2) {
        reinterpret_cast<uint4*>(p)[i] = *reinterpret_cast<uint4*>(pv);
      } else {
        reinterpret_cast<uint4*>(p)[2 * i] = reinterpret_cast<uint4*>(pv)[0];
        reinterpret_cast<uint4*>(p)[2 * i + 1] = reinterpret_cast<uint4*>(pv)[1];
      }
    }
    done = nv * V;
  }
  for (long long i = done + (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const T dec = st_f<T>(__fmul_rn(ld_f<T>(p[i]), decay));
    p[i] = st_f<T>(__fmaf_rn(alpha, __bfloat162float(u[i]), ld_f<T>(dec)));
  }
}

int elementwise_grid(long long n, int per_thread) {
  const long long want = (n + 256LL * per_thread - 1) / (256LL * per_thread);
  const long long cap = (long long)sm_count() * 8;
  long long g = want < cap ? want : cap;
  return (int)(g < 1 ? 1 : g);
}

template <typename T>
bool sumsq_vec_ok(const void* g, long long rows, long long cols, long long ldg) {
  constexpr int V = 16 / sizeof(T);
  return (ldg == cols || rows == 1) && ((reinterpret_cast<uintptr_t>(g) & 15u) == 0) &&
         ((rows * cols) % V == 0);
}

// Partial sums of squares of `count` matrices of identical extents, one launch.
template <typename T>
int sumsq_batch_t(const NormTable& tab, int count, cudaStream_t stream) {
  const NormEntry& e0 = tab.e[0];
  int vec_ok = 1;
  for (int i = 0; i < count; ++i)
    vec_ok = vec_ok && sumsq_vec_ok<T>(tab.e[i].g, tab.e[i].rows, tab.e[i].cols, tab.e[i].ldg);
  const dim3 grid((unsigned)norm_blocks(e0.rows * e0.cols), (unsigned)count);
  sumsq_partial_kernel<T><<<grid, 256, 0, stream>>>(tab, vec_ok);
  FM_CUDA_CHECK(cudaGetLastError());
  return FM_OK;
}

template <typename T>
int normalize_batch_t(const NormTable& tab, int count, bool sumsq_ready, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const NormEntry& e0 = tab.e[0];
  const long long rows = e0.rows, cols = e0.cols;
  if (!sumsq_ready) {
    const int rc = sumsq_batch_t<T>(tab, count, stream);
    if (rc != FM_OK) return rc;
  }
  const long long tiles = ((rows + 63) / 64) * ((cols + 63) / 64);
  if (tiles > 0x7fffffffLL) return fail(FM_ERR_UNSUPPORTED, "matrix too large");
  bool fast = (rows % 64 == 0) && (cols % 64 == 0);
  for (int i = 0; i < count && fast; ++i) {
    const NormEntry& e = tab.e[i];
    fast = (e.ldg % V == 0) && ((reinterpret_cast<uintptr_t>(e.g) & 15u) == 0) &&
           (e.xd == nullptr || (e.ldxd % 8 == 0 && (reinterpret_cast<uintptr_t>(e.xd) & 15u) == 0)) &&
           (e.xt == nullptr || (e.ldxt % 8 == 0 && (reinterpret_cast<uintptr_t>(e.xt) & 15u) == 0));
  }
  const int nparts = norm_blocks(rows * cols);
  if (fast) {
    // one tile per block while that is at most two rounds of resident blocks; beyond that as
    // many blocks as are resident at once, every one walking the same number of tiles
    static long long resident = 0;
    if (resident == 0) {
      int per_sm = 0;
      FM_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, scale_transpose_vec_kernel<T>, 256, 0));
      resident = (long long)(per_sm > 0 ? per_sm : 1) * sm_count();
    }
    const long long per = ((rows + kScaleTileRows - 1) / kScaleTileRows) * (cols / 64);
    long long blocks = per;
    if (per * count > 2 * resident) {
      const long long share = resident / count > 0 ? resident / count : 1;
      const long long tiles_per_block = (per + share - 1) / share;
      blocks = (per + tiles_per_block - 1) / tiles_per_block;
    }
    scale_transpose_vec_kernel<T><<<dim3((unsigned)blocks, (unsigned)count), 256, 0, stream>>>(tab, nparts);
  } else {
    scale_transpose_kernel<T><<<dim3((unsigned)tiles, (unsigned)count), 256, 0, stream>>>(tab, nparts);
  }
  FM_CUDA_CHECK(cudaGetLastError());
  return FM_OK;
}

int fill_norm_table(NormTable* tab, const NormItem* items, int count) {
  if (count < 1 || count > kMaxNormBatch)
    return fail(FM_ERR_INVALID, "normalisation batch must be 1..%d", kMaxNormBatch);
  for (int i = 0; i < count; ++i) {
    const NormItem& it = items[i];
    if (!it.g || !it.partials || (!it.xd && !it.xt)) return fail(FM_ERR_INVALID, "null pointer");
    if (it.rows != items[0].rows || it.cols != items[0].cols)
      return fail(FM_ERR_INVALID, "matrices of a batch must have identical extents");
    if (it.rows <= 0 || it.cols <= 0 || it.ldg < it.cols || (it.xd && it.ldxd < it.cols) ||
        (it.xt && it.ldxt < it.rows))
      return fail(FM_ERR_INVALID, "bad extents");
    NormEntry& e = tab->e[i];
    e.g = it.g; e.rows = it.rows; e.cols = it.cols; e.ldg = it.ldg;
    e.xd = static_cast<__nv_bfloat16*>(it.xd); e.ldxd = it.ldxd;
    e.xt = static_cast<__nv_bfloat16*>(it.xt); e.ldxt = it.ldxt;
    e.partials = it.partials;
  }
  return FM_OK;
}

template <typename T>
bool momentum_fusable_t(const MomentumItem* items, int count) {
  constexpr int V = 16 / sizeof(T);
  for (int i = 0; i < count; ++i) {
    if ((reinterpret_cast<uintptr_t>(items[i].grad) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(items[i].buf) & 15u) != 0 || items[i].n % V != 0 ||
        items[i].n != items[0].n)
      return false;
  }
  return true;
}

template <typename T>
int momentum_batch_t(const MomentumItem* items, int count, double momentum, int nesterov,
                     cudaStream_t stream) {
  MomentumTable tab;
  long long nmax = 0;
  bool want_sumsq = true;
  int vec_ok = 1;
  for (int i = 0; i < count; ++i) {
    tab.grad[i] = items[i].grad;
    tab.buf[i] = items[i].buf;
    tab.partials[i] = items[i].partials;
    tab.n[i] = items[i].n;
    if (items[i].n > nmax) nmax = items[i].n;
    if (!items[i].partials) want_sumsq = false;
    vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(items[i].grad) & 15u) == 0) &&
             ((reinterpret_cast<uintptr_t>(items[i].buf) & 15u) == 0);
  }
  if (nmax == 0) return FM_OK;
  // the reference passes python floats: lerp_(g, 1 - momentum) and lerp_(buf, momentum)
  const float w_buf = (float)(1.0 - momentum);
  const float w_grad = (float)momentum;
  if (want_sumsq && momentum_fusable_t<T>(items, count)) {
    const dim3 grid((unsigned)norm_blocks(nmax), (unsigned)count);
    momentum_kernel<T, true><<<grid, 256, 0, stream>>>(tab, w_buf, w_grad, nesterov, 1);
    FM_CUDA_CHECK(cudaGetLastError());
    return FM_OK;
  }
  int gx = elementwise_grid(nmax, sizeof(T) == 4 ? 4 : 8);
  gx = (gx + count - 1) / count;  // share the SMs between the tensors of the launch
  const dim3 grid((unsigned)(gx < 1 ? 1 : gx), (unsigned)count);
  momentum_kernel<T, false><<<grid, 256, 0, stream>>>(tab, w_buf, w_grad, nesterov, vec_ok);
  FM_CUDA_CHECK(cudaGetLastError());
  if (!want_sumsq) return FM_OK;
  // tensors the fused kernel cannot take (odd sizes or alignment): a separate pass over the
  // values Newton-Schulz will read leaves the same partial sums
  for (int i = 0; i < count; ++i) {
    if (items[i].n == 0) continue;
    NormTable nt;
    NormEntry& e = nt.e[0];
    e.g = nesterov ? items[i].grad : items[i].buf;
    e.rows = 1; e.cols = items[i].n; e.ldg = items[i].n;
    e.xd = nullptr; e.ldxd = 0; e.xt = nullptr; e.ldxt = 0;
    e.partials = items[i].partials;
    const int rc = sumsq_batch_t<T>(nt, 1, stream);
    if (rc != FM_OK) return rc;
  }
  return FM_OK;
}

}  // namespace

int normalize_batch(const NormItem* items, int count, int g_dtype, bool sumsq_ready,
                    cudaStream_t stream) {
  NormTable tab;
  const int rc = fill_norm_table(&tab, items, count);
  if (rc != FM_OK) return rc;
  switch (g_dtype) {
    case FM_BF16: return normalize_batch_t<__nv_bfloat16>(tab, count, sumsq_ready, stream);
    case FM_F16: return normalize_batch_t<__half>(tab, count, sumsq_ready, stream);
    case FM_F32: return normalize_batch_t<float>(tab, count, sumsq_ready, stream);
    default: return fail(FM_ERR_UNSUPPORTED, "unknown dtype %d", g_dtype);
  }
}

int momentum_batch(const MomentumItem* items, int count, int dtype, double momentum, int nesterov,
                   cudaStream_t stream) {
  if (count < 0) return fail(FM_ERR_INVALID, "negative tensor count");
  for (int base = 0; base < count; base += kMaxMomentumBatch) {
    const int m = (count - base) < kMaxMomentumBatch ? (count - base) : kMaxMomentumBatch;
    for (int i = 0; i < m; ++i) {
      if (!items[base + i].grad || !items[base + i].buf) return fail(FM_ERR_INVALID, "null pointer");
      if (items[base + i].n < 0) return fail(FM_ERR_INVALID, "negative element count");
    }
    int rc;
    switch (dtype) {
      case FM_BF16: rc = momentum_batch_t<__nv_bfloat16>(items + base, m, momentum, nesterov, stream); break;
      case FM_F16: rc = momentum_batch_t<__half>(items + base, m, momentum, nesterov, stream); break;
      case FM_F32: rc = momentum_batch_t<float>(items + base, m, momentum, nesterov, stream); break;
      default: return fail(FM_ERR_UNSUPPORTED, "unknown dtype %d", dtype);
    }
    if (rc != FM_OK) return rc;
  }
  return FM_OK;
}

}  // namespace fm

extern "C" size_t fm_norm_scratch_floats(void) { return fm::kNormBlocks; }

extern "C" int fm_normalize(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype,
                            void* xd, int64_t ldxd, void* xt, int64_t ldxt, float* partials,
                            void* stream) {
  using namespace fm;
  clear_error();
  NormItem it;
  it.g = G; it.rows = rows; it.cols = cols; it.ldg = ldg;
  it.xd = xd; it.ldxd = ldxd; it.xt = xt; it.ldxt = ldxt;
  it.partials = partials;
  return normalize_batch(&it, 1, g_dtype, false, static_cast<cudaStream_t>(stream));
}

extern "C" int fm_momentum(void* grad, void* buf, int64_t n, int dtype, double momentum,
                           int nesterov, float* sumsq_partials, void* stream) {
  using namespace fm;
  clear_error();
  MomentumItem it;
  it.grad = grad; it.buf = buf; it.n = n; it.partials = sumsq_partials;
  return momentum_batch(&it, 1, dtype, momentum, nesterov, static_cast<cudaStream_t>(stream));
}

extern "C" int fm_update_multi(void* const* params, const void* const* updates,
                               const int64_t* numels, const double* alphas, int count, int p_dtype,
                               double decay, void* stream) {
  using namespace fm;
  clear_error();
  if (count < 0) return fail(FM_ERR_INVALID, "negative tensor count");
  if (count == 0) return FM_OK;
  if (!params || !updates || !numels || !alphas) return fail(FM_ERR_INVALID, "null table");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int base = 0; base < count; base += kMaxTensors) {
    const int m = (count - base) < kMaxTensors ? (count - base) : kMaxTensors;
    UpdateTable tab;
    long long nmax = 0;
    for (int i = 0; i < m; ++i) {
      if (!params[base + i] || !updates[base + i] || numels[base + i] < 0)
        return fail(FM_ERR_INVALID, "bad entry %d of the update table", base + i);
      tab.p[i] = params[base + i];
      tab.u[i] = updates[base + i];
      tab.n[i] = numels[base + i];
      tab.alpha[i] = (float)alphas[base + i];
      if (tab.n[i] > nmax) nmax = tab.n[i];
    }
    if (nmax == 0) continue;
    int gx = elementwise_grid(nmax, 8);
    // share the SMs between the tensors of the launch
    gx = (gx + m - 1) / m;
    if (gx < 1) gx = 1;
    const dim3 grid((unsigned)gx, (unsigned)m);
    switch (p_dtype) {
      case FM_BF16: update_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(tab, (float)decay); break;
      case FM_F16: update_kernel<__half><<<grid, 256, 0, st>>>(tab, (float)decay); break;
      case FM_F32: update_kernel<float><<<grid, 256, 0, st>>>(tab, (float)decay); break;
      default: return fail(FM_ERR_UNSUPPORTED, "unknown dtype %d", p_dtype);
    }
    FM_CUDA_CHECK(cudaGetLastError());
  }
  return FM_OK;
}
