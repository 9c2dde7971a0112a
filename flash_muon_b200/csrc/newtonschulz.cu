// Host side of the C ABI for the GEMM-shaped entry points and the Newton-Schulz launch plan.
// fm_newtonschulz enqueues the whole orthogonalisation (2 normalisation kernels + 3 GEMM kernels
// per step) on one stream with no allocation, no synchronisation and no host round trip, following
// flash_muon/muon.py:13-33 operation by operation:
//   X = bf16(G) (transposed if tall) / (||X|| + 1e-7)
//   repeat: A = X X^T;  B = b*A + c*(A A^T);  X = a*X + B X
// The iterate is kept in both orientations (X [m,k] and XT [k,m]) so that every GEMM reads
// K-major operands through plain TMA tiles: X feeds X X^T, XT is the right operand of B X, and
// the epilogue of B X writes the next X and XT together.  No transposed copy is ever made by a
// separate kernel (the reference pays a contiguous() copy per step for tall inputs,
// flash_muon/matmul_transpose_triton.py:88).
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "gemm_common.cuh"
#include "muon_kernels.cuh"

extern "C" size_t fm_norm_scratch_floats(void);

namespace fm {
namespace {

inline int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Workspace of a Newton-Schulz pass over `count` matrices whose smaller / larger dimensions are
// m / k: the iterate in both orientations, twice (ping-pong), A and B, the partial sums of the
// norms, and (single matrices with long tile lists only) the scratch of the balanced GEMM tail.
// The matrices of a batch are stacked along the rows of each region.
struct NsLayout {
  int64_t m, k, ldk, ldm;
  int count;
  int64_t x_batch, xt_batch, a_batch;  // elements between consecutive matrices of a region
  size_t off_x[2], off_xt[2], off_a, off_b, off_partials, off_sk, sk_bytes, total;
};

bool ns_layout(int count, int64_t rows, int64_t cols, NsLayout* L) {
  if (rows <= 0 || cols <= 0 || rows > (1 << 24) || cols > (1 << 24)) return false;
  if (count < 1 || count > kMaxGemmBatch) return false;
  L->count = count;
  L->m = rows <= cols ? rows : cols;
  L->k = rows <= cols ? cols : rows;
  L->ldk = round_up(L->k, 8);  // row pitches are multiples of 16 bytes for TMA
  L->ldm = round_up(L->m, 8);
  L->x_batch = L->m * L->ldk;
  L->xt_batch = L->k * L->ldm;
  L->a_batch = L->m * L->ldm;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += (bytes + 255) / 256 * 256;
    return o;
  };
  const size_t xb = (size_t)count * L->x_batch * 2, xtb = (size_t)count * L->xt_batch * 2;
  const size_t ab = (size_t)count * L->a_batch * 2;
  L->off_x[0] = take(xb);
  L->off_x[1] = take(xb);
  L->off_xt[0] = take(xtb);
  L->off_xt[1] = take(xtb);
  L->off_a = take(ab);
  L->off_b = take(ab);
  L->off_partials = take((size_t)count * fm_norm_scratch_floats() * sizeof(float));
  L->sk_bytes = 0;
  if (count == 1) {
    const int64_t m = L->m, k = L->k;
    size_t sk = gemm_sk_bytes(FM_BF16, m, m, k, 1);
    auto upto = [&](size_t v) { if (v > sk) sk = v; };
    upto(gemm_sk_bytes(FM_BF16, m, m, m, 1));
    upto(gemm_sk_bytes(FM_BF16, m, k, m, 0));
    upto(gemm_sk_bytes(FM_BF16, k, m, m, 0));
    L->sk_bytes = sk;
  }
  L->off_sk = take(L->sk_bytes);
  L->total = off;
  return true;
}

// One Newton-Schulz pass, following flash_muon/muon.py:13-33 operation by operation for every
// matrix of the batch.  G[i] is rows[i] x cols[i] with row pitch ldg[i]; all share (m, k).
int ns_run(const void* const* G, const int64_t* rows, const int64_t* cols, const int64_t* ldg,
           int count, int g_dtype, int steps, void* const* out, void* workspace,
           size_t workspace_bytes, int flags, cudaStream_t st) {
  if (!G || !rows || !cols || !ldg || !out || !workspace) return fail(FM_ERR_INVALID, "null pointer");
  if (steps < 0) return fail(FM_ERR_INVALID, "negative step count");
  if (count < 1 || count > kMaxGemmBatch)
    return fail(FM_ERR_INVALID, "a batch holds 1..%d matrices, got %d", kMaxGemmBatch, count);
  if ((flags & ~(FM_NS_PRECISE | FM_NS_SUMSQ_READY)) != 0)
    return fail(FM_ERR_INVALID, "unknown flags %d", flags);
  NsLayout L;
  if (!ns_layout(count, rows[0], cols[0], &L))
    return fail(FM_ERR_INVALID, "bad extents rows=%lld cols=%lld", (long long)rows[0], (long long)cols[0]);
  for (int i = 0; i < count; ++i) {
    if (!G[i] || !out[i]) return fail(FM_ERR_INVALID, "null matrix pointer at %d", i);
    const int64_t mi = rows[i] <= cols[i] ? rows[i] : cols[i], ki = rows[i] <= cols[i] ? cols[i] : rows[i];
    if (rows[i] <= 0 || cols[i] <= 0 || mi != L.m || ki != L.k)
      return fail(FM_ERR_INVALID, "matrix %d is %lld x %lld: a batch shares its smaller and larger dimension (%lld, %lld)",
                  i, (long long)rows[i], (long long)cols[i], (long long)L.m, (long long)L.k);
    if (ldg[i] < cols[i]) return fail(FM_ERR_INVALID, "row pitch of matrix %d smaller than its width", i);
  }
  if (workspace_bytes < L.total)
    return fail(FM_ERR_WORKSPACE, "workspace of %zu bytes, %zu needed", workspace_bytes, L.total);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(FM_ERR_INVALID, "workspace must be 256-byte aligned");

  char* ws = static_cast<char*>(workspace);
  __nv_bfloat16* X[2] = {reinterpret_cast<__nv_bfloat16*>(ws + L.off_x[0]),
                         reinterpret_cast<__nv_bfloat16*>(ws + L.off_x[1])};
  __nv_bfloat16* XT[2] = {reinterpret_cast<__nv_bfloat16*>(ws + L.off_xt[0]),
                          reinterpret_cast<__nv_bfloat16*>(ws + L.off_xt[1])};
  __nv_bfloat16* Am = reinterpret_cast<__nv_bfloat16*>(ws + L.off_a);
  __nv_bfloat16* Bm = reinterpret_cast<__nv_bfloat16*>(ws + L.off_b);
  float* partials = reinterpret_cast<float*>(ws + L.off_partials);
  const size_t pfloats = fm_norm_scratch_floats();
  void* sk = L.sk_bytes ? ws + L.off_sk : nullptr;
  const int64_t m = L.m, k = L.k;
  const bool sumsq_ready = (flags & FM_NS_SUMSQ_READY) != 0;
  const int precise = (flags & FM_NS_PRECISE) ? 1 : 0;

  // Stack order: wide matrices (rows <= cols) first, tall ones after, so that the one GEMM that
  // differs between the two orientations (the last) runs on two contiguous ranges of the stack.
  int perm[kMaxGemmBatch];
  int nw = 0;
  for (int i = 0; i < count; ++i) if (rows[i] <= cols[i]) perm[nw++] = i;
  int nt = nw;
  for (int i = 0; i < count; ++i) if (rows[i] > cols[i]) perm[nt++] = i;

  NormItem items[kMaxGemmBatch];
  if (steps == 0) {  // the normalised input in its own orientation (flash_muon/muon.py:23, :31-32)
    for (int lo = 0, hi = nw; lo < count; lo = hi, hi = count) {
      if (hi == lo) continue;
      for (int s = lo; s < hi; ++s) {
        const int i = perm[s];
        NormItem& it = items[s - lo];
        it = NormItem();
        it.g = G[i]; it.rows = rows[i]; it.cols = cols[i]; it.ldg = ldg[i];
        it.xd = out[i]; it.ldxd = cols[i];
        it.partials = partials + (size_t)i * pfloats;
      }
      const int rc = normalize_batch(items, hi - lo, g_dtype, sumsq_ready, st);
      if (rc != FM_OK) return rc;
    }
    return FM_OK;
  }

  // G is [rows, cols]: for a wide input the direct copy is X and the transposed one XT, for a
  // tall input the direct copy is XT ([k, m]) and the transposed one X ([m, k]).
  for (int lo = 0, hi = nw; lo < count; lo = hi, hi = count) {
    if (hi == lo) continue;
    for (int s = lo; s < hi; ++s) {
      const int i = perm[s];
      NormItem& it = items[s - lo];
      it.g = G[i]; it.rows = rows[i]; it.cols = cols[i]; it.ldg = ldg[i];
      it.partials = partials + (size_t)i * pfloats;
      if (s < nw) {
        it.xd = X[0] + (size_t)s * L.x_batch; it.ldxd = L.ldk;
        it.xt = XT[0] + (size_t)s * L.xt_batch; it.ldxt = L.ldm;
      } else {
        it.xd = XT[0] + (size_t)s * L.xt_batch; it.ldxd = L.ldm;
        it.xt = X[0] + (size_t)s * L.x_batch; it.ldxt = L.ldk;
      }
    }
    const int rc = normalize_batch(items, hi - lo, g_dtype, sumsq_ready, st);
    if (rc != FM_OK) return rc;
  }

  const float ca = 3.4445f, cb = -4.7750f, cc = 2.0315f;  // flash_muon/muon.py:14
  void* outs[kMaxGemmBatch];
  for (int s = 0; s < count; ++s) outs[s] = out[perm[s]];
  int rc = FM_OK;
  int cur = 0;
  for (int s = 0; s < steps; ++s) {
    const bool last = (s == steps - 1);
    {  // A = X X^T                                   (muon.py:26)
      GemmArgs a;
      a.dtype = FM_BF16;
      a.A = X[cur]; a.lda = L.ldk;
      a.B = X[cur]; a.ldb = L.ldk;
      a.M = m; a.N = m; a.K = k;
      a.sym = 1;
      a.C = Am; a.ldc_r = L.ldm; a.ldc_c = 1;
      a.CT = Am; a.ldt_r = L.ldm; a.ldt_c = 1;
      a.batch = count; a.a_batch_rows = m; a.b_batch_rows = m;
      a.c_batch = L.a_batch; a.t_batch = L.a_batch;
      a.sk_ws = sk; a.sk_bytes = L.sk_bytes;
      if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
    }
    {  // B = b*A + c*(A A^T)                         (muon.py:27-28)
      GemmArgs a;
      a.dtype = FM_BF16;
      a.A = Am; a.lda = L.ldm;
      a.B = Am; a.ldb = L.ldm;
      a.M = m; a.N = m; a.K = m;
      a.sym = 1;
      a.D = Am; a.ldd = L.ldm;
      a.alpha = cb; a.beta = cc; a.precise = precise;
      a.C = Bm; a.ldc_r = L.ldm; a.ldc_c = 1;
      a.CT = Bm; a.ldt_r = L.ldm; a.ldt_c = 1;
      a.batch = count; a.a_batch_rows = m; a.b_batch_rows = m;
      a.d_batch = L.a_batch; a.c_batch = L.a_batch; a.t_batch = L.a_batch;
      a.sk_ws = sk; a.sk_bytes = L.sk_bytes;
      if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
    }
    if (!last) {  // X' = a*X + B X  (and its transpose)  (muon.py:29)
      GemmArgs a;
      a.dtype = FM_BF16;
      a.A = Bm; a.lda = L.ldm;
      a.B = XT[cur]; a.ldb = L.ldm;
      a.M = m; a.N = k; a.K = m;
      a.sym = 0;
      a.D = X[cur]; a.ldd = L.ldk;
      a.alpha = ca; a.beta = 1.f; a.precise = precise;
      a.C = X[cur ^ 1]; a.ldc_r = L.ldk; a.ldc_c = 1;
      a.CT = XT[cur ^ 1]; a.ldt_r = L.ldm; a.ldt_c = 1;
      a.batch = count; a.a_batch_rows = m; a.b_batch_rows = k;
      a.d_batch = L.x_batch; a.c_batch = L.x_batch; a.t_batch = L.xt_batch;
      a.sk_ws = sk; a.sk_bytes = L.sk_bytes;
      if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
    } else {
      if (nw > 0) {  // wide: out [m, k] = a*X + B X
        GemmArgs a;
        a.dtype = FM_BF16;
        a.A = Bm; a.lda = L.ldm;
        a.B = XT[cur]; a.ldb = L.ldm;
        a.M = m; a.N = k; a.K = m;
        a.sym = 0;
        a.D = X[cur]; a.ldd = L.ldk;
        a.alpha = ca; a.beta = 1.f; a.precise = precise;
        a.C = outs[0]; a.ldc_r = k; a.ldc_c = 1;
        a.batch = nw; a.a_batch_rows = m; a.b_batch_rows = k;
        a.d_batch = L.x_batch;
        a.c_tab = nw > 1 ? outs : nullptr;
        a.sk_ws = sk; a.sk_bytes = L.sk_bytes;
        if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
      }
      if (count > nw) {
        // tall: only X'^T = a*X^T + X^T B is wanted (B is symmetric), and in that orientation it
        // is the direct, 16-byte-store output.  Same products summed in the same order as B X, so
        // the values are those of the other orientation.
        const int ntall = count - nw;
        GemmArgs a;
        a.dtype = FM_BF16;
        a.A = XT[cur] + (size_t)nw * L.xt_batch; a.lda = L.ldm;
        a.B = Bm + (size_t)nw * L.a_batch; a.ldb = L.ldm;
        a.M = k; a.N = m; a.K = m;
        a.sym = 0;
        a.D = XT[cur] + (size_t)nw * L.xt_batch; a.ldd = L.ldm;
        a.alpha = ca; a.beta = 1.f; a.precise = precise;
        a.C = outs[nw]; a.ldc_r = m; a.ldc_c = 1;          // out [rows = k, cols = m]
        a.batch = ntall; a.a_batch_rows = k; a.b_batch_rows = m;
        a.d_batch = L.xt_batch;
        a.c_tab = ntall > 1 ? outs + nw : nullptr;
        a.sk_ws = sk; a.sk_bytes = L.sk_bytes;
        if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
      }
    }
    cur ^= 1;
  }
  return FM_OK;
}

}  // namespace

// Internal form of fm_newtonschulz_batched for callers inside the library.
int newtonschulz_batched(const void* const* G, const int64_t* rows, const int64_t* cols, int count,
                         int g_dtype, int steps, void* const* out, void* workspace,
                         size_t workspace_bytes, int flags, cudaStream_t stream) {
  return ns_run(G, rows, cols, cols, count, g_dtype, steps, out, workspace, workspace_bytes, flags,
                stream);
}

}  // namespace fm

extern "C" size_t fm_syrk_workspace_bytes(int64_t M, int64_t K, int dtype) {
  if (M <= 0 || K <= 0) return 0;
  return fm::gemm_sk_bytes(dtype, M, M, K, 1);
}

extern "C" int fm_syrk(const void* x, void* y, int64_t M, int64_t K, int64_t ldx, int64_t ldy_row,
                       int64_t ldy_col, int dtype, void* workspace, size_t workspace_bytes,
                       void* stream) {
  using namespace fm;
  clear_error();
  if (!x || !y) return fail(FM_ERR_INVALID, "null pointer");
  if (M <= 0 || K <= 0 || ldx < K) return fail(FM_ERR_INVALID, "bad extents M=%lld K=%lld ldx=%lld",
                                                (long long)M, (long long)K, (long long)ldx);
  if (dtype != FM_BF16 && dtype != FM_F16 && dtype != FM_F32)
    return fail(FM_ERR_UNSUPPORTED, "unknown dtype %d", dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool tma_ok = (dtype != FM_F32) && (ldx % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  if (!tma_ok) return syrk_simt(x, y, M, K, ldx, ldy_row, ldy_col, dtype, st);
  GemmArgs a;
  a.dtype = dtype;
  a.A = x; a.lda = ldx;
  a.B = x; a.ldb = ldx;
  a.M = M; a.N = M; a.K = K;
  a.sym = 1;
  a.C = y; a.ldc_r = ldy_row; a.ldc_c = ldy_col;
  a.CT = y; a.ldt_r = ldy_row; a.ldt_c = ldy_col;
  if (workspace != nullptr) {
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
      return fail(FM_ERR_INVALID, "workspace must be 256-byte aligned");
    a.sk_ws = workspace;
    a.sk_bytes = workspace_bytes;
  }
  return gemm_tc(a, st);
}

extern "C" int fm_syrk_poly(const void* x, int64_t ldx, int64_t M, int64_t K, const void* D,
                            int64_t ldd, float alpha, float beta, void* out, int64_t ldo, int dtype,
                            int precise, void* stream) {
  using namespace fm;
  clear_error();
  if (!x || !D || !out) return fail(FM_ERR_INVALID, "null pointer");
  if (M <= 0 || K <= 0 || ldx < K || ldd < M || ldo < M) return fail(FM_ERR_INVALID, "bad extents");
  GemmArgs a;
  a.dtype = dtype;
  a.A = x; a.lda = ldx;
  a.B = x; a.ldb = ldx;
  a.M = M; a.N = M; a.K = K;
  a.sym = 1;
  a.D = D; a.ldd = ldd;
  a.alpha = alpha; a.beta = beta; a.precise = precise;
  a.C = out; a.ldc_r = ldo; a.ldc_c = 1;
  a.CT = out; a.ldt_r = ldo; a.ldt_c = 1;
  return gemm_tc(a, static_cast<cudaStream_t>(stream));
}

extern "C" int fm_gemm_nt(const void* A, int64_t lda, const void* B, int64_t ldb, int64_t M,
                          int64_t N, int64_t K, const void* D, int64_t ldd, float alpha, float beta,
                          void* C, int64_t ldc, void* CT, int64_t ldct, int dtype, int precise,
                          void* stream) {
  using namespace fm;
  clear_error();
  if (!A || !B || (!C && !CT)) return fail(FM_ERR_INVALID, "null pointer");
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < K || (D && ldd < N) || (C && ldc < N) ||
      (CT && ldct < M))
    return fail(FM_ERR_INVALID, "bad extents");
  GemmArgs a;
  a.dtype = dtype;
  a.A = A; a.lda = lda;
  a.B = B; a.ldb = ldb;
  a.M = M; a.N = N; a.K = K;
  a.sym = 0;
  a.D = D; a.ldd = ldd;
  a.alpha = alpha; a.beta = beta; a.precise = precise;
  a.C = C; a.ldc_r = ldc; a.ldc_c = 1;
  a.CT = CT; a.ldt_r = ldct; a.ldt_c = 1;
  return gemm_tc(a, static_cast<cudaStream_t>(stream));
}

extern "C" size_t fm_ns_workspace_bytes(int64_t rows, int64_t cols) {
  fm::NsLayout L;
  if (!fm::ns_layout(1, rows, cols, &L)) return 0;
  return L.total;
}

extern "C" size_t fm_ns_partials_offset(int64_t rows, int64_t cols) {
  fm::NsLayout L;
  if (!fm::ns_layout(1, rows, cols, &L)) return 0;
  return L.off_partials;
}

extern "C" size_t fm_ns_batched_workspace_bytes(int count, int64_t rows, int64_t cols) {
  fm::NsLayout L;
  if (!fm::ns_layout(count, rows, cols, &L)) return 0;
  return L.total;
}

extern "C" size_t fm_ns_batched_partials_offset(int count, int64_t rows, int64_t cols) {
  fm::NsLayout L;
  if (!fm::ns_layout(count, rows, cols, &L)) return 0;
  return L.off_partials;
}

extern "C" int fm_newtonschulz(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype,
                               int steps, void* out, void* workspace, size_t workspace_bytes,
                               int flags, void* stream) {
  using namespace fm;
  clear_error();
  if (!G || !out || !workspace) return fail(FM_ERR_INVALID, "null pointer");
  return ns_run(&G, &rows, &cols, &ldg, 1, g_dtype, steps, &out, workspace, workspace_bytes, flags,
                static_cast<cudaStream_t>(stream));
}

extern "C" int fm_newtonschulz_batched(const void* const* G, const int64_t* rows,
                                       const int64_t* cols, int count, int g_dtype, int steps,
                                       void* const* out, void* workspace, size_t workspace_bytes,
                                       int flags, void* stream) {
  using namespace fm;
  clear_error();
  return ns_run(G, rows, cols, cols, count, g_dtype, steps, out, workspace, workspace_bytes, flags,
                static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------
// Newton-Schulz without a caller workspace, for hosts that may not allocate device memory.
// The scratch of fm_newtonschulz (both orientations of the iterate twice, A, B, the partial
// sums) lives in one file-scope device array; every device that loads the library carries it
// until the process ends.  The name of the array is only a host-side handle: the device address
// is looked up once per device with cudaGetSymbolAddress and that pointer is what the kernels get.
namespace fm {
namespace {

constexpr int64_t kStaticMaxSmall = 1024;  // largest min(rows, cols)
constexpr int64_t kStaticMaxLarge = 4096;  // largest max(rows, cols)
constexpr size_t kStaticScratchBytes =
    (size_t)(4 * kStaticMaxSmall * kStaticMaxLarge + 2 * kStaticMaxSmall * kStaticMaxSmall) * 2 +
    8192;  // + partial sums and the 256-byte rounding of the seven regions

static __device__ __align__(256) unsigned char g_ns_static_scratch[kStaticScratchBytes];

// Device address of the scratch array on the current device, resolved on first use.
int static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  FM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FM_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_ns_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(FM_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s",
                  cudaGetErrorString(e));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return FM_OK;
}

}  // namespace
}  // namespace fm

extern "C" int fm_newtonschulz_static(const void* G, int64_t rows, int64_t cols, int64_t ldg,
                                      int g_dtype, int steps, void* out, int flags, void* stream) {
  using namespace fm;
  clear_error();
  if (rows <= 0 || cols <= 0) return fail(FM_ERR_INVALID, "bad extents");
  const int64_t small = rows <= cols ? rows : cols, large = rows <= cols ? cols : rows;
  NsLayout L;
  if (small > kStaticMaxSmall || large > kStaticMaxLarge || !ns_layout(1, rows, cols, &L) ||
      L.total > kStaticScratchBytes)
    return fail(FM_ERR_WORKSPACE,
                "fm_newtonschulz_static handles matrices up to %lld x %lld (either orientation); "
                "got %lld x %lld -- use fm_newtonschulz with a caller workspace",
                (long long)kStaticMaxSmall, (long long)kStaticMaxLarge, (long long)rows,
                (long long)cols);
  void* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);
  if (rc != FM_OK) return rc;
  return fm_newtonschulz(G, rows, cols, ldg, g_dtype, steps, out, scratch, kStaticScratchBytes,
                         flags, stream);
}
