// Pieces shared by the single-CTA and the CTA-pair tensor-core GEMM kernels: kernel parameters,
// numeric traits and the register epilogue (addend load, rounding-faithful arithmetic, direct and
// transposed global stores with the mirror rule of the symmetric product).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace fm {

constexpr int kMaxGemmBatch = 16;

struct GemmParams {
  int M, N, K;
  int sym;        // 1: triangular schedule + mirrored store (requires A == B, M == N)
  int tiles_m;    // row tiles of the schedule
  int tiles_n;    // CTA-pair kernel, general products: > 0 = column tiles, tiles walk along columns first
  int num_tiles;  // length of the static tile list
  int num_kb;     // ceil(K / 64)
  int strip_w;    // CTA-pair kernel, symmetric lists: width of the column strips (0: column order)
  const void* D;  // optional addend, row-major, unit column stride
  long long ldd;
  void* C;        // direct output (may be null): C[r*ldc_r + c*ldc_c]
  long long ldc_r, ldc_c;
  void* CT;       // transposed output (may be null): element (r,c) goes to CT[c*ldt_r + r*ldt_c]
  long long ldt_r, ldt_c;
  float alpha, beta;
  int precise;    // 1: single rounding of alpha*D + beta*acc
  int d_vec;      // D rows can be read with 16-byte loads
  int c_vec;      // C rows can be written with 16-byte stores
  int t_pack;     // CT can be written as pairs of adjacent rows (4-byte stores)
  int stages;     // slots (64-wide K blocks) of the shared-memory ring (CTA-pair kernel)
  int kb_per_stage;  // K blocks per pipeline stage (1 or 2)
  int early_trigger; // 1: CTAs release the next kernel of the stream when they start their last item
  // balanced tail of the CTA-pair kernel (all zero: every tile is dealt whole)
  int sk_dp_tiles;         // tiles dealt whole, round-robin; the rest is cut by K blocks
  int sk_per;              // K blocks per pair in the balanced region
  long long sk_total;      // K blocks of the balanced region
  float* sk_ws;            // scratch for partial accumulators
  unsigned int* sk_cnt;    // per (tile, CTA rank) count of deposited parts, zero between launches
  unsigned int* err;
  // Batched launch (CTA-pair kernel): `batch` problems of identical extents whose operands are
  // stacked along the rows of one tensor map each; the tile list is the single-problem list
  // repeated `batch` times.  batch == 1: plain launch, every field below is zero.
  int batch;
  int tiles_per_batch;
  int a_batch_rows, b_batch_rows;       // rows between consecutive problems in the operand stacks
  long long d_batch, c_batch, t_batch;  // elements between consecutive problems in D, C, CT
  int use_c_tab;                        // 1: problem g writes its direct output to c_tab[g]
  void* c_tab[kMaxGemmBatch];
  // CTA-pair kernel: outputs leave through shared-memory staging and TMA tile stores (full
  // 64- and 128-byte row segments) instead of per-lane global stores.  Set by the host when every
  // output is a 16-byte aligned, unit-column-stride matrix; tiles on the diagonal of a symmetric
  // product keep the register path (their element-wise mirror rule).
  int tma_store;
  int c_batch_rows, t_batch_rows;       // rows between consecutive problems in the C / CT maps
  int tma_d;                            // pair kernel: the addend arrives by TMA tile loads
  int d_batch_rows;                     // rows between consecutive problems in the D map
};

// Base pointers of one problem of a (possibly batched) launch.
struct EpiPtrs {
  const void* D;
  void* C;
  void* CT;
};

__device__ __forceinline__ EpiPtrs epilogue_ptrs(const GemmParams& p, int g, int elem_bytes) {
  EpiPtrs e;
  e.D = p.D;
  e.C = p.C;
  e.CT = p.CT;
  if (p.batch > 1) {
    if (e.D) e.D = static_cast<const char*>(p.D) + (long long)g * p.d_batch * elem_bytes;
    if (p.use_c_tab) e.C = p.c_tab[g];
    else if (e.C) e.C = static_cast<char*>(p.C) + (long long)g * p.c_batch * elem_bytes;
    if (e.CT) e.CT = static_cast<char*>(p.CT) + (long long)g * p.t_batch * elem_bytes;
  }
  return e;
}

template <typename T>
struct Num;
template <>
struct Num<__nv_bfloat16> {
  static constexpr uint32_t kFormat = 1;
  static __device__ __forceinline__ __nv_bfloat16 rn(float f) { return __float2bfloat16_rn(f); }
  static __device__ __forceinline__ float f(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <>
struct Num<__half> {
  static constexpr uint32_t kFormat = 0;
  static __device__ __forceinline__ __half rn(float f) { return __float2half_rn(f); }
  static __device__ __forceinline__ float f(__half v) { return __half2float(v); }
};

// Addend values D[row][c0 .. c0+31] of one epilogue chunk (zeros outside the matrix).
template <typename T>
__device__ __forceinline__ void epilogue_load_d(const GemmParams& p, const EpiPtrs& e, int row, int c0,
                                                T (&dv)[32]) {
  const T* Dp = reinterpret_cast<const T*>(e.D);
  if (Dp == nullptr) return;
  if (row < p.M && c0 < p.N) {
    const T* dptr = Dp + (long long)row * p.ldd + c0;
    if (p.d_vec && c0 + 32 <= p.N) {
      const uint4* d4 = reinterpret_cast<const uint4*>(dptr);
#pragma unroll
      for (int v = 0; v < 4; ++v) reinterpret_cast<uint4*>(dv)[v] = __ldg(d4 + v);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) dv[j] = (c0 + j < p.N) ? dptr[j] : Num<T>::rn(0.f);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) dv[j] = Num<T>::rn(0.f);
  }
}

// Arithmetic of one 32-column chunk of one accumulator row:
//   raw : fp32 accumulator bits of columns c0..c0+31 of the row,  dv : the addend values
//   out = round(round(alpha*D) + round(beta*round(acc)))  (one rounding with `precise`), or
//   round(acc) without an addend.
template <typename T>
__device__ __forceinline__ void epilogue_values(const GemmParams& p, const EpiPtrs& e,
                                                const uint32_t (&raw)[32], const T (&dv)[32],
                                                T (&outv)[32]) {
  if (e.D != nullptr) {
    if (p.precise) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        outv[j] = Num<T>::rn(fmaf(p.alpha, Num<T>::f(dv[j]), p.beta * __uint_as_float(raw[j])));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const T tacc = Num<T>::rn(__uint_as_float(raw[j]));
        const T u = Num<T>::rn(p.alpha * Num<T>::f(dv[j]));
        const T w = Num<T>::rn(p.beta * Num<T>::f(tacc));
        outv[j] = Num<T>::rn(Num<T>::f(u) + Num<T>::f(w));
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) outv[j] = Num<T>::rn(__uint_as_float(raw[j]));
  }
}

// Global stores of one chunk from registers (direct rows + transposed columns).
//   bi  : index of the 128-row block `row` belongs to (diagonal test of the symmetric product)
// Symmetric mode: a 128-column block left of the diagonal block is skipped (its mirror image is
// produced by the block above the diagonal); on the diagonal only c >= row is stored and
// c > row mirrored, so both triangles come from the same rounded registers.
template <typename T>
__device__ __forceinline__ void epilogue_store_regs(const GemmParams& p, const EpiPtrs& e,
                                                    const T (&outv)[32], int row, int c0, int bi) {
  if (c0 >= p.N) return;  // warp-uniform
  const int cb = c0 >> 7;
  if (p.sym && cb < bi) return;  // warp-uniform
  // Inside the diagonal 128 x 128 block the warp's 32 rows meet this chunk's 32 columns in one
  // of three ways: wholly below the diagonal (nothing to store), wholly above (same as any
  // other block) or on it (element-wise rule).  All three tests are warp-uniform.
  bool diag = false;
  if (p.sym && cb == bi) {
    const int r_first = row & ~31;
    if (c0 + 31 < r_first) return;
    diag = (c0 < r_first + 32);
  }
  const bool full_cols = (c0 + 32 <= p.N);
  const bool row_ok = row < p.M;
  T* const Cp = reinterpret_cast<T*>(e.C);
  T* const CTp = reinterpret_cast<T*>(e.CT);

  if (Cp != nullptr && row_ok) {
    if (p.c_vec && full_cols && !diag) {
      uint4* c4 = reinterpret_cast<uint4*>(Cp + (long long)row * p.ldc_r + c0);
#pragma unroll
      for (int v = 0; v < 4; ++v) c4[v] = reinterpret_cast<const uint4*>(outv)[v];
    } else {
      T* cptr = Cp + (long long)row * p.ldc_r + (long long)c0 * p.ldc_c;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int c = c0 + j;
        if (c < p.N && (!diag || c >= row)) cptr[(long long)j * p.ldc_c] = outv[j];
      }
    }
  }
  if (CTp != nullptr) {
    // the 32 rows of this warp start at a multiple of 32: all of them in range <=> last one is
    const bool warp_rows_ok = ((row | 31) < p.M);
    if (p.t_pack && full_cols && !diag && warp_rows_ok) {
      // Lanes 2u and 2u+1 hold adjacent rows.  Exchange packed column pairs so that the even
      // lane writes rows (2u, 2u+1) of the even columns and the odd lane those of the odd
      // columns: 16 four-byte stores per lane instead of 32 two-byte stores.
      const uint32_t* own = reinterpret_cast<const uint32_t*>(outv);
      const bool odd = (row & 1) != 0;
      T* tbase = CTp + (long long)c0 * p.ldt_r + (row & ~1);
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const uint32_t mine = own[jj];
        const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
        // even lane: {own[2jj], partner[2jj]}; odd lane: {partner[2jj+1], own[2jj+1]}
        const uint32_t v = odd ? __byte_perm(theirs, mine, 0x7632) : __byte_perm(mine, theirs, 0x5410);
        const int j = 2 * jj + (odd ? 1 : 0);
        *reinterpret_cast<uint32_t*>(tbase + (long long)j * p.ldt_r) = v;
      }
    } else if (row_ok) {
      T* tptr = CTp + (long long)c0 * p.ldt_r + (long long)row * p.ldt_c;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int c = c0 + j;
        if (c < p.N && (!diag || c > row)) tptr[(long long)j * p.ldt_r] = outv[j];
      }
    }
  }
}

// Arithmetic + register stores of one chunk.
template <typename T>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, const EpiPtrs& e,
                                               const uint32_t (&raw)[32], const T (&dv)[32], int row,
                                               int c0, int bi) {
  if (c0 >= p.N) return;  // warp-uniform
  alignas(16) T outv[32];
  epilogue_values<T>(p, e, raw, dv, outv);
  epilogue_store_regs<T>(p, e, outv, row, c0, bi);
}

// Staging of one chunk for the TMA tile stores.  `lane` holds one row of the warp's 32 x 64
// block (two chunks); half selects the chunk.
//   sC : [32 rows][64 columns], rows of 128 bytes under the 128-byte swizzle (16-byte piece q of
//        row r sits at piece q ^ (r & 7)), the layout a SWIZZLE_128B tensor map reads;
//   sT : [64 columns][32 rows], rows of 64 bytes, no swizzle.
// Both writes are free of bank conflicts: 8 consecutive lanes cover the 8 pieces of a 128-byte
// span of sC, and the packed transposed words of one instruction fill 128 consecutive bytes of sT.
template <typename T>
__device__ __forceinline__ void epilogue_stage(const T (&outv)[32], uint8_t* sC, uint8_t* sT,
                                               int lane, int half, bool want_c, bool want_t) {
  if (want_c) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int piece = (half * 4 + v) ^ (lane & 7);
      *reinterpret_cast<uint4*>(sC + lane * 128 + piece * 16) = reinterpret_cast<const uint4*>(outv)[v];
    }
  }
  if (want_t) {
    const uint32_t* own = reinterpret_cast<const uint32_t*>(outv);
    const bool odd = (lane & 1) != 0;
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) {
      const uint32_t mine = own[jj];
      const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
      const uint32_t v = odd ? __byte_perm(theirs, mine, 0x7632) : __byte_perm(mine, theirs, 0x5410);
      const int col = half * 32 + 2 * jj + (odd ? 1 : 0);
      *reinterpret_cast<uint32_t*>(sT + col * 64 + (lane & ~1) * 2) = v;
    }
  }
}

}  // namespace fm
