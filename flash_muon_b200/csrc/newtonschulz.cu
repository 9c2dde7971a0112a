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

extern "C" int fm_normalize(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype,
                            void* xd, int64_t ldxd, void* xt, int64_t ldxt, float* partials,
                            void* stream);
extern "C" size_t fm_norm_scratch_floats(void);

namespace fm {
namespace {

inline int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct NsLayout {
  int64_t m, k, ldk, ldm;
  size_t off_x[2], off_xt[2], off_a, off_b, off_partials, total;
};

bool ns_layout(int64_t rows, int64_t cols, NsLayout* L) {
  if (rows <= 0 || cols <= 0 || rows > (1 << 24) || cols > (1 << 24)) return false;
  L->m = rows <= cols ? rows : cols;
  L->k = rows <= cols ? cols : rows;
  L->ldk = round_up(L->k, 8);  // row pitches are multiples of 16 bytes for TMA
  L->ldm = round_up(L->m, 8);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += (bytes + 255) / 256 * 256;
    return o;
  };
  const size_t xb = (size_t)L->m * L->ldk * 2, xtb = (size_t)L->k * L->ldm * 2;
  const size_t ab = (size_t)L->m * L->ldm * 2;
  L->off_x[0] = take(xb);
  L->off_x[1] = take(xb);
  L->off_xt[0] = take(xtb);
  L->off_xt[1] = take(xtb);
  L->off_a = take(ab);
  L->off_b = take(ab);
  L->off_partials = take(fm_norm_scratch_floats() * sizeof(float));
  L->total = off;
  return true;
}

}  // namespace
}  // namespace fm

extern "C" int fm_syrk(const void* x, void* y, int64_t M, int64_t K, int64_t ldx, int64_t ldy_row,
                       int64_t ldy_col, int dtype, void* stream) {
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
  if (!fm::ns_layout(rows, cols, &L)) return 0;
  return L.total;
}

extern "C" int fm_newtonschulz(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype,
                               int steps, void* out, void* workspace, size_t workspace_bytes,
                               int flags, void* stream) {
  using namespace fm;
  clear_error();
  if (!G || !out || !workspace) return fail(FM_ERR_INVALID, "null pointer");
  if (steps < 0) return fail(FM_ERR_INVALID, "negative step count");
  NsLayout L;
  if (!ns_layout(rows, cols, &L) || ldg < cols)
    return fail(FM_ERR_INVALID, "bad extents rows=%lld cols=%lld ldg=%lld", (long long)rows,
                (long long)cols, (long long)ldg);
  if (workspace_bytes < L.total)
    return fail(FM_ERR_WORKSPACE, "workspace of %zu bytes, %zu needed", workspace_bytes, L.total);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(FM_ERR_INVALID, "workspace must be 256-byte aligned");
  if (flags != FM_NS_FAITHFUL && flags != FM_NS_PRECISE)
    return fail(FM_ERR_INVALID, "unknown flags %d", flags);

  char* ws = static_cast<char*>(workspace);
  void* X[2] = {ws + L.off_x[0], ws + L.off_x[1]};
  void* XT[2] = {ws + L.off_xt[0], ws + L.off_xt[1]};
  void* Am = ws + L.off_a;
  void* Bm = ws + L.off_b;
  float* partials = reinterpret_cast<float*>(ws + L.off_partials);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool tall = rows > cols;
  const int64_t m = L.m, k = L.k;

  if (steps == 0)  // the normalised input in its own orientation (flash_muon/muon.py:23, :31-32)
    return fm_normalize(G, rows, cols, ldg, g_dtype, out, cols, nullptr, 0, partials, stream);

  // G is [rows, cols]: for a wide input the direct copy is X and the transposed one XT,
  // for a tall input the direct copy is XT ([k, m]) and the transposed one X ([m, k]).
  int rc = tall ? fm_normalize(G, rows, cols, ldg, g_dtype, XT[0], L.ldm, X[0], L.ldk, partials, stream)
                : fm_normalize(G, rows, cols, ldg, g_dtype, X[0], L.ldk, XT[0], L.ldm, partials, stream);
  if (rc != FM_OK) return rc;

  const float ca = 3.4445f, cb = -4.7750f, cc = 2.0315f;  // flash_muon/muon.py:14
  const int precise = (flags == FM_NS_PRECISE);
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
      if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
    }
    if (last && tall) {
      // Last step of a tall input: only X'^T = a*X^T + X^T B is wanted (B is symmetric), and in
      // that orientation it is the direct, 16-byte-store output.  Same products summed in the
      // same order as B X, so the values are those of the other orientation.
      GemmArgs a;
      a.dtype = FM_BF16;
      a.A = XT[cur]; a.lda = L.ldm;
      a.B = Bm; a.ldb = L.ldm;
      a.M = k; a.N = m; a.K = m;
      a.sym = 0;
      a.D = XT[cur]; a.ldd = L.ldm;
      a.alpha = ca; a.beta = 1.f; a.precise = precise;
      a.C = out; a.ldc_r = cols; a.ldc_c = 1;         // out [rows=k, cols=m]
      if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
    } else {  // X' = a*X + B X  (and its transpose)  (muon.py:29)
      GemmArgs a;
      a.dtype = FM_BF16;
      a.A = Bm; a.lda = L.ldm;
      a.B = XT[cur]; a.ldb = L.ldm;
      a.M = m; a.N = k; a.K = m;
      a.sym = 0;
      a.D = X[cur]; a.ldd = L.ldk;
      a.alpha = ca; a.beta = 1.f; a.precise = precise;
      if (!last) {
        a.C = X[cur ^ 1]; a.ldc_r = L.ldk; a.ldc_c = 1;
        a.CT = XT[cur ^ 1]; a.ldt_r = L.ldm; a.ldt_c = 1;
      } else {
        a.C = out; a.ldc_r = cols; a.ldc_c = 1;       // out [rows=m, cols=k]
      }
      if ((rc = gemm_tc(a, st)) != FM_OK) return rc;
    }
    cur ^= 1;
  }
  return FM_OK;
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
  if (small > kStaticMaxSmall || large > kStaticMaxLarge || !ns_layout(rows, cols, &L) ||
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
