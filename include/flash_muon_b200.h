/*
 * flash_muon_b200 -- C ABI of the B200 (sm_100a) Muon hot path.
 *
 * The reference project (nil0x9/flash-muon) is pure Python; its operator interface is
 *   flash_muon/__init__.py:1-4   matmul_transpose, matmul_transpose_assign, fast_newtonschulz, Muon
 * Each entry point below names the reference function whose device work it replaces.
 *
 * Conventions
 *  - Every function returns an fm_status (0 = ok, negative = error).  Nothing throws.
 *  - All data pointers are DEVICE pointers owned by the caller; no entry point allocates or frees
 *    memory and nothing synchronises unless stated.  Scratch memory is passed in by the caller
 *    (the *_workspace_bytes functions give its size); calls that may overlap on the GPU need
 *    distinct scratch.  The one exception is fm_newtonschulz_static, whose ~38 MB scratch array
 *    is part of the library's device image and exists on every GPU that loads it.
 *  - What a call launches depends on its arguments and the process-wide options only, never on
 *    what else is running: the same call gives the same bits every time.
 *  - `stream` is a cudaStream_t passed as void* (0 = the legacy default stream).  All work of a
 *    call is enqueued on that stream of the CURRENT device.
 *  - Leading dimensions and strides are in ELEMENTS.
 *  - Arguments are validated on the host before any launch.  fm_last_error() returns a
 *    thread-local message for the last failing call of the calling thread.
 */
#ifndef FLASH_MUON_B200_H_
#define FLASH_MUON_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FM_OK = 0,
  FM_ERR_INVALID = -1,     /* bad argument (null pointer, negative size, misaligned) */
  FM_ERR_UNSUPPORTED = -2, /* dtype / shape outside what the kernels cover */
  FM_ERR_CUDA = -3,        /* a CUDA runtime or driver call failed */
  FM_ERR_DEVICE_WAIT = -4, /* a bounded wait inside a kernel ran out (see fm_device_status) */
  FM_ERR_WORKSPACE = -5    /* workspace too small */
} fm_status;

typedef enum { FM_BF16 = 0, FM_F16 = 1, FM_F32 = 2 } fm_dtype;

/* flags of fm_newtonschulz (bit mask) */
enum {
  FM_NS_FAITHFUL = 0,   /* reproduce every intermediate rounding of the reference formulation */
  FM_NS_PRECISE = 1,    /* one rounding per fused epilogue (closer to exact, further from reference) */
  FM_NS_SUMSQ_READY = 2 /* fm_momentum already left the partial sums of squares in the workspace */
};

/* Library version: major * 10000 + minor * 100 + patch. */
int fm_version(void);

/*
 * Process-wide tuning switches, for experiments and A/B comparisons (the defaults are the
 * product).  Names: "gemm_impl" (0 by size, 1 single-CTA kernel, 2 CTA-pair kernel), "gemm_bn"
 * (tile width of the single-CTA kernel: 0 by size, 64, 128, 256), "gemm_stages" (ring depth of the
 * pair kernel, 0 = default), "gemm_balance" (0: never cut the tail of a tile list by K blocks),
 * "gemm_strip" (tile order of symmetric lists: -1 by size, 0 column order, w = strips of w tile
 * columns), "pdl" (0: no programmatic dependent launch), "gemm_tma_store" (0: the pair kernel
 * writes its outputs with per-lane global stores instead of TMA tile stores), "gemm_tma_d" (0: it
 * fetches the addend with per-lane global loads instead of TMA tile loads).  Initial values come
 * from the environment variables FM_GEMM_IMPL, FM_GEMM_BN, FM_GEMM_STAGES, FM_GEMM_BALANCE,
 * FM_GEMM_STRIP, FM_PDL, FM_GEMM_TMA_STORE and FM_GEMM_TMA_D, read once.  Stands in for the autotune table of the reference
 * (flash_muon/matmul_transpose_triton.py:6-18); not thread-safe against concurrent launches.
 */
int fm_set_option(const char* name, int value);
int fm_get_option(const char* name, int* value);

/* Message of the last error raised on the calling thread ("" if none). */
const char* fm_last_error(void);

/*
 * Synchronises the current device and reports whether any kernel of this library gave up a
 * bounded wait since the last call (0 = none).  Clears the flag.  *code receives a word that
 * identifies kernel, role and barrier.  No reference counterpart (the reference never checks
 * device state); used by tests and by callers that want a post-step health check.
 */
int fm_device_status(unsigned int* code);

/*
 * y[M,M] = x[M,K] * x^T, fp32 accumulation, one rounding to `dtype`; only upper-triangular tile
 * pairs are computed and every tile is also stored transposed, so y is bitwise symmetric.
 * x is row-major with row pitch ldx and unit column stride; y is addressed as
 * y[i*ldy_row + j*ldy_col] (arbitrary strides, as the reference passes them to its kernel).
 * Replaces: mmt_kernel + matmul_transpose_assign, flash_muon/matmul_transpose_triton.py:19-101.
 * bf16/f16 with ldx % 8 == 0 and a 16-byte aligned x run on tcgen05 tensor cores; f32 and other
 * layouts run on an exact-fp32 FFMA kernel.
 * workspace (may be null): fm_syrk_workspace_bytes(M, K, dtype) bytes of 256-byte aligned device
 * scratch.  Long tile lists (e.g. 8192 x 8192) use it to split the last tiles by K so that no SM
 * idles through a partial last wave; without it every tile is computed whole.  Both schedules
 * are deterministic; they differ in the order of the fp32 sums of the split tiles.
 */
size_t fm_syrk_workspace_bytes(int64_t M, int64_t K, int dtype);
int fm_syrk(const void* x, void* y, int64_t M, int64_t K, int64_t ldx, int64_t ldy_row,
            int64_t ldy_col, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * General C[M,N] = A[M,K] * B[N,K]^T (+ fused epilogue), bf16/f16, both operands row-major with
 * unit column stride (K-major).  out = round(round(alpha*D) + round(beta*round(acc))) when D is
 * non-null (single rounding of alpha*D + beta*acc when `precise` != 0), round(acc) otherwise.
 * C (direct, row pitch ldc) and CT (transposed copy, CT[j*ldct + i]) may each be null but not both.
 * Building block of fm_newtonschulz (the reference's `B @ X` and `a*X + ...`,
 * flash_muon/muon.py:29); exported for tests and benchmarks.
 */
int fm_gemm_nt(const void* A, int64_t lda, const void* B, int64_t ldb, int64_t M, int64_t N,
               int64_t K, const void* D, int64_t ldd, float alpha, float beta, void* C,
               int64_t ldc, void* CT, int64_t ldct, int dtype, int precise, void* stream);

/*
 * Symmetric rank-k update with the polynomial epilogue of the Newton-Schulz step:
 * out = round(round(alpha*D) + round(beta*round(x x^T))) with D symmetric, out bitwise symmetric.
 * Replaces matmul_transpose_assign(buf1, buf2) followed by `b*buf1 + c*buf2`,
 * flash_muon/muon.py:27-28.
 */
int fm_syrk_poly(const void* x, int64_t ldx, int64_t M, int64_t K, const void* D, int64_t ldd,
                 float alpha, float beta, void* out, int64_t ldo, int dtype, int precise,
                 void* stream);

/* Bytes of device workspace fm_newtonschulz needs for a rows x cols input (0 on bad sizes), and
 * the byte offset inside it of the fm_norm_scratch_floats() partial sums that fm_momentum may
 * fill ahead of the call (FM_NS_SUMSQ_READY). */
size_t fm_ns_workspace_bytes(int64_t rows, int64_t cols);
size_t fm_ns_partials_offset(int64_t rows, int64_t cols);

/*
 * out = Newton-Schulz orthogonalisation of G (rows x cols, row pitch ldg, dtype g_dtype), `steps`
 * quintic iterations with (a,b,c) = (3.4445, -4.7750, 2.0315) after a Frobenius normalisation,
 * all storage in bf16 and fp32 accumulation.  `out` is bf16 [rows, cols], contiguous, and must
 * not alias G or the workspace.  Tall inputs (rows > cols) are iterated on transposed, as the
 * reference does, without materialising a transposed copy per step.
 * Replaces: fast_newtonschulz, flash_muon/muon.py:6-33.
 */
int fm_newtonschulz(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype, int steps,
                    void* out, void* workspace, size_t workspace_bytes, int flags, void* stream);

/*
 * Newton-Schulz of `count` (1..16) matrices in one pass: G[i] is rows[i] x cols[i] (contiguous,
 * dtype g_dtype), out[i] the bf16 result of the same shape.  All matrices must have the same
 * smaller and the same larger dimension (a 4096 x 1024 and a 1024 x 4096 matrix may share a
 * batch, as they share a numel group in flash_muon/muon.py:68).  Every GEMM of the iteration is
 * ONE launch whose tile list covers all matrices, so matrices that are too small to fill the GPU
 * on their own (a 1024 x 1024 product is 10 tiles for 74 CTA pairs) share it, and the number of
 * launches per matrix drops by `count`.  The arithmetic per matrix is that of fm_newtonschulz:
 * results are bit-identical.  Replaces: `count` calls of fast_newtonschulz,
 * flash_muon/muon.py:6-33, for the matrices a rank owns in consecutive rounds (muon.py:90-103).
 * Workspace: fm_ns_batched_workspace_bytes(count, rows[0], cols[0]); with FM_NS_SUMSQ_READY the
 * partial sums of matrix i are expected at fm_ns_batched_partials_offset(...) +
 * i * fm_norm_scratch_floats() * sizeof(float).
 */
size_t fm_ns_batched_workspace_bytes(int count, int64_t rows, int64_t cols);
size_t fm_ns_batched_partials_offset(int count, int64_t rows, int64_t cols);
int fm_newtonschulz_batched(const void* const* G, const int64_t* rows, const int64_t* cols,
                            int count, int g_dtype, int steps, void* const* out, void* workspace,
                            size_t workspace_bytes, int flags, void* stream);

/*
 * fm_newtonschulz for callers that cannot allocate device memory -- a plugin running inside a
 * host that owns the allocator, code already inside a stream capture, a real-time loop that must
 * not touch cudaMalloc.  Same arguments and result as fm_newtonschulz, minus the workspace: the
 * scratch is a fixed array inside the library (about 38 MB per GPU, resident from the moment the
 * library's device code is loaded until the process exits).  This entry point has no counterpart
 * in the reference, which allocates two buffers and several temporaries per call
 * (flash_muon/muon.py:19-20, :23-29).
 *  - Limit: min(rows, cols) <= 1024 and max(rows, cols) <= 4096; larger inputs are rejected with
 *    FM_ERR_WORKSPACE and a message, nothing is launched.
 *  - The first call on each device resolves the array's device address (one
 *    cudaGetSymbolAddress with that device current); make that call before any stream capture.
 *    No call allocates or frees memory.
 *  - All calls on a device share the one array.  Nothing in it has to start at zero (every region
 *    is written before it is read), but two calls whose kernels overlap on the GPU -- different
 *    streams, or different host threads -- race on it: serialise them on one stream.
 */
int fm_newtonschulz_static(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype,
                           int steps, void* out, int flags, void* stream);

/*
 * Frobenius normalisation used by fm_newtonschulz, exported for tests:
 * xd[rows,cols] (row pitch ldxd) = bf16(G) / (||bf16(G)||_F + 1e-7) and xt[cols,rows] (row pitch
 * ldxt) = its transpose, with the reference's roundings (norm, sum and quotient each rounded to
 * bf16).  `partials` is a device scratch of at least fm_norm_scratch_floats() floats that the
 * call overwrites.  Either of xd / xt may be null.
 * Replaces: `X / (X.norm(...) + 1e-7)`, flash_muon/muon.py:15-23.
 */
int fm_normalize(const void* G, int64_t rows, int64_t cols, int64_t ldg, int g_dtype, void* xd,
                 int64_t ldxd, void* xt, int64_t ldxt, float* partials, void* stream);
size_t fm_norm_scratch_floats(void);

/*
 * Momentum + Nesterov, in place, n elements of `dtype`:
 *   buf <- lerp(buf, grad, 1 - momentum);  grad <- nesterov ? lerp(grad, buf, momentum) : grad
 * each lerp rounded to `dtype` like torch's lerp_.  With nesterov == 0 grad is left untouched and
 * the caller uses buf.  Replaces: flash_muon/muon.py:99-100.
 * sumsq_partials (may be null): fm_norm_scratch_floats() floats that receive the partial sums of
 * squares of the tensor Newton-Schulz reads next (grad if nesterov, else buf) -- bit for bit the
 * partial sums fm_normalize would compute itself, so that fm_newtonschulz with FM_NS_SUMSQ_READY
 * can skip its own pass over the matrix (flash_muon/muon.py:23 reads it once more for the norm).
 */
int fm_momentum(void* grad, void* buf, int64_t n, int dtype, double momentum, int nesterov,
                float* sumsq_partials, void* stream);

/*
 * Fused decoupled weight decay + scaled update over `count` tensors in one launch:
 *   p_i <- round(p_i * decay);  p_i <- round(p_i + alpha_i * u_i)      (u_i is bf16)
 * params / updates are HOST arrays of device pointers.  Replaces: flash_muon/muon.py:87-89.
 */
int fm_update_multi(void* const* params, const void* const* updates, const int64_t* numels,
                    const double* alphas, int count, int p_dtype, double decay, void* stream);

/*
 * One numel group of a Muon step on one GPU (all arrays are HOST arrays of `count` entries).
 * Matrix i is params[i] (dtype p_dtype) with gradient grads[i] and momentum buffer momentum[i]
 * (both g_dtype), all contiguous, seen as rows[i] x cols[i] (conv filters: size(0) x the rest,
 * flash_muon/muon.py:101-102).  alphas[i] = -lr * sqrt(max(1, size(-2) / size(-1))) of the
 * ORIGINAL shape (muon.py:89), decay = 1 - lr * weight_decay (muon.py:87).  Consecutive matrices
 * with the same smaller and larger dimension go through Newton-Schulz `batch` at a time
 * (fm_newtonschulz_batched: one launch per GEMM for all of them; batch = 1 for matrices that fill
 * the GPU on their own).  slots holds 2 * lanes * batch device buffers of rows*cols bf16 each: the
 * update of matrix j of pass c is written to slot (c mod (2 * lanes)) * batch + j, the role the
 * reference's update_buffer plays (muon.py:69, :103).
 */
typedef struct {
  void* const* params;
  void* const* grads;
  void* const* momentum;
  const int64_t* rows;
  const int64_t* cols;
  const double* alphas;
  int32_t count;
  int32_t p_dtype;
  int32_t g_dtype;
  int32_t nesterov;
  int32_t ns_steps;
  int32_t lanes;        /* 1..4 streams the rounds of this group rotate over */
  int32_t batch;        /* 1..16 consecutive same-shape matrices per Newton-Schulz pass */
  int32_t reserved;     /* 0 */
  double momentum_coef; /* mu of muon.py:99-100 */
  double decay;
  void* const* slots;
} fm_muon_group;

/*
 * A whole Muon step with world_size == 1 in one call: for every matrix of every group, in order,
 * momentum + Nesterov, Newton-Schulz into an update slot, decay + update.  Replaces the Python
 * round loop of Muon.step, flash_muon/muon.py:77-110, for the case without an exchange between
 * ranks; the device work per matrix is that of fm_momentum, fm_newtonschulz and fm_update_multi
 * in the same order, so the parameters come out bit-identical to driving those from a host loop.
 * Rounds rotate over lanes: lane 0 is `stream`, the others and the stream of the decay + update
 * kernels belong to the library (created on the first call per device, as are the events that
 * order them); all of them wait for `stream` at entry and `stream` waits for all of them before
 * the call returns, so to the caller the step is ordinary work on `stream`.
 * workspaces: HOST array of one device buffer of workspace_bytes per lane (as many as the
 * largest `lanes` of the groups), each at least fm_ns_batched_workspace_bytes(batch, rows, cols)
 * of the most demanding group.
 * One step at a time per device.  gradients are overwritten when nesterov != 0, as by the
 * reference (muon.py:100).
 */
int fm_muon_step(const fm_muon_group* groups, int ngroups, void* const* workspaces,
                 size_t workspace_bytes, void* stream);

/*
 * Peer-memory plumbing of the copy-engine all-gather that stands in for
 * dist.all_gather_into_tensor (flash_muon/muon.py:108) inside one NVLink-connected box.  Each rank
 * copies its finished slot into every peer's gather buffer with DMA engines and orders the
 * exchange with 32-bit flags written and awaited by the streams themselves, so no SM is taken from
 * the Newton-Schulz GEMMs the transfer overlaps.
 *  fm_ipc_export : CUDA IPC handle (64 bytes) of the allocation that contains `ptr`, and the byte
 *                  offset of `ptr` inside it.
 *  fm_ipc_import : address, in this process, of offset `offset` of a peer's exported allocation
 *                  (opened once per handle and device, peer access enabled on first use).
 *  fm_ipc_close_all : closes every imported allocation.
 *  fm_copy_async : device-to-device cudaMemcpyAsync on `stream`; dst / src may be peer addresses.
 *  fm_stream_write32 : `stream` stores `value` to the 4-byte aligned device word `addr` (local or
 *                  peer) after all prior work of the stream.
 *  fm_stream_wait32_geq : `stream` stalls until (int32)(*addr - value) >= 0; later work of the
 *                  stream sees remote writes that preceded the flag.  No host thread blocks.
 */
int fm_ipc_export(const void* ptr, unsigned char* handle64, uint64_t* offset);
int fm_ipc_import(const unsigned char* handle64, uint64_t offset, void** ptr);
int fm_ipc_close_all(void);
int fm_copy_async(void* dst, const void* src, size_t bytes, void* stream);
int fm_stream_write32(void* addr, uint32_t value, void* stream);
int fm_stream_wait32_geq(const void* addr, uint32_t value, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_MUON_B200_H_ */
