// Internal interface of the HBM-bound kernels (elementwise.cu) in their batched form, used by the
// Newton-Schulz plans and the whole-step call.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace fm {

// One matrix of a normalisation launch: g is [rows, cols] with row pitch ldg; xd receives
// bf16(g) / (||bf16(g)||_F + 1e-7) in the same orientation (row pitch ldxd), xt its transpose
// (row pitch ldxt); either may be null.  `partials` is this matrix's scratch of
// fm_norm_scratch_floats() floats.
struct NormItem {
  const void* g = nullptr;
  int64_t rows = 0, cols = 0, ldg = 0;
  void* xd = nullptr;
  int64_t ldxd = 0;
  void* xt = nullptr;
  int64_t ldxt = 0;
  float* partials = nullptr;
};

// Normalises `count` matrices of identical extents (1..16) with two launches, or one when
// `sumsq_ready` says that every item's partial sums of squares were already left in `partials`
// by momentum_batch.
int normalize_batch(const NormItem* items, int count, int g_dtype, bool sumsq_ready,
                    cudaStream_t stream);

// One tensor of a momentum launch.  With `partials` (all items or none) the partial sums of
// squares of the tensor Newton-Schulz reads next (grad if nesterov, else buf) are produced too.
struct MomentumItem {
  void* grad = nullptr;
  void* buf = nullptr;
  int64_t n = 0;
  float* partials = nullptr;
};

int momentum_batch(const MomentumItem* items, int count, int dtype, double momentum, int nesterov,
                   cudaStream_t stream);

}  // namespace fm
