// One whole Muon step on one GPU as a single host call.
// The reference walks its parameters in a Python loop (flash_muon/muon.py:77-110): per matrix two
// lerp_ kernels, fast_newtonschulz, an all-gather and mul_/add_.  With world_size == 1 there is
// no exchange, and what is left of the loop is pure launch bookkeeping: which stream a round runs
// on, which update slot it writes, which events order the decay + update of round i behind its
// Newton-Schulz and ahead of the reuse of its slot.  fm_muon_step does that bookkeeping in the
// library: rounds rotate over up to four streams ("lanes"; lane 0 is the caller's stream) and two
// update slots per lane, the decay + update kernels run on one more stream, everything is forked
// from and joined back into the caller's stream with events.  The kernels and their order per
// matrix are exactly those of the per-matrix entry points, so the result is bit-identical to
// driving fm_momentum / fm_newtonschulz / fm_update_multi from the host loop.
#include <mutex>

#include "common.cuh"
#include "gemm_common.cuh"
#include "muon_kernels.cuh"

namespace fm {
namespace {

constexpr int kMaxLanes = 4;
constexpr int kMaxSlots = 2 * kMaxLanes;

struct StepState {
  bool ready = false;
  cudaStream_t lane[kMaxLanes - 1] = {};
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join_side = nullptr;
  cudaEvent_t join_lane[kMaxLanes - 1] = {};
  cudaEvent_t ns_done[kMaxSlots] = {};
  cudaEvent_t upd_done[kMaxSlots] = {};
};

// Streams and events of the current device, created on first use and kept for the life of the
// process.  One step at a time per device: concurrent callers would share the events.
StepState* step_state() {
  static std::mutex mu;
  static StepState per_dev[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  StepState& s = per_dev[dev];
  if (!s.ready) {
    bool ok = true;
    for (int i = 0; i < kMaxLanes - 1; ++i) {
      ok = ok && cudaStreamCreateWithFlags(&s.lane[i], cudaStreamNonBlocking) == cudaSuccess;
      ok = ok && cudaEventCreateWithFlags(&s.join_lane[i], cudaEventDisableTiming) == cudaSuccess;
    }
    ok = ok && cudaStreamCreateWithFlags(&s.side, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&s.join_side, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < kMaxSlots; ++i) {
      ok = ok && cudaEventCreateWithFlags(&s.ns_done[i], cudaEventDisableTiming) == cudaSuccess;
      ok = ok && cudaEventCreateWithFlags(&s.upd_done[i], cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) {
      cudaGetLastError();
      return nullptr;
    }
    s.ready = true;
  }
  return &s;
}

int validate_group(const fm_muon_group& g, int gi) {
  if (g.count < 0) return fail(FM_ERR_INVALID, "group %d: negative count", gi);
  if (g.count == 0) return FM_OK;
  if (!g.params || !g.grads || !g.momentum || !g.rows || !g.cols || !g.alphas || !g.slots)
    return fail(FM_ERR_INVALID, "group %d: null array", gi);
  if (g.lanes < 1 || g.lanes > kMaxLanes)
    return fail(FM_ERR_INVALID, "group %d: lanes must be 1..%d", gi, kMaxLanes);
  if (g.batch < 1 || g.batch > kMaxGemmBatch)
    return fail(FM_ERR_INVALID, "group %d: batch must be 1..%d", gi, kMaxGemmBatch);
  if (g.ns_steps < 0) return fail(FM_ERR_INVALID, "group %d: negative ns_steps", gi);
  for (int i = 0; i < g.count; ++i) {
    if (!g.params[i] || !g.grads[i] || !g.momentum[i])
      return fail(FM_ERR_INVALID, "group %d: null tensor pointer at %d", gi, i);
    if (g.rows[i] < 0 || g.cols[i] < 0) return fail(FM_ERR_INVALID, "group %d: negative size at %d", gi, i);
  }
  for (int b = 0; b < 2 * g.lanes * g.batch; ++b)
    if (!g.slots[b]) return fail(FM_ERR_INVALID, "group %d: null update slot %d", gi, b);
  return FM_OK;
}

inline int64_t small_dim(const fm_muon_group& g, int i) { return g.rows[i] < g.cols[i] ? g.rows[i] : g.cols[i]; }
inline int64_t large_dim(const fm_muon_group& g, int i) { return g.rows[i] < g.cols[i] ? g.cols[i] : g.rows[i]; }

// Matrices [i, end) of the group that go through Newton-Schulz together: up to `batch`
// consecutive non-empty matrices with the same smaller and larger dimension.
int chunk_end(const fm_muon_group& g, int i) {
  int e = i + 1;
  if (g.rows[i] * g.cols[i] == 0) return e;
  while (e < g.count && e - i < g.batch && g.rows[e] * g.cols[e] != 0 &&
         small_dim(g, e) == small_dim(g, i) && large_dim(g, e) == large_dim(g, i))
    ++e;
  return e;
}

}  // namespace

int newtonschulz_batched(const void* const* G, const int64_t* rows, const int64_t* cols, int count,
                         int g_dtype, int steps, void* const* out, void* workspace,
                         size_t workspace_bytes, int flags, cudaStream_t stream);

}  // namespace fm

extern "C" int fm_muon_step(const fm_muon_group* groups, int ngroups, void* const* workspaces,
                            size_t workspace_bytes, void* stream) {
  using namespace fm;
  clear_error();
  if (ngroups < 0 || (ngroups > 0 && !groups)) return fail(FM_ERR_INVALID, "bad group list");
  if (ngroups == 0) return FM_OK;
  if (!workspaces) return fail(FM_ERR_INVALID, "null workspace list");
  int max_lanes = 1;
  for (int gi = 0; gi < ngroups; ++gi) {
    const fm_muon_group& g = groups[gi];
    const int rc = validate_group(g, gi);
    if (rc != FM_OK) return rc;
    if (g.count > 0 && g.lanes > max_lanes) max_lanes = g.lanes;
    for (int i = 0; i < g.count;) {
      const int e = chunk_end(g, i);
      if (g.rows[i] * g.cols[i] != 0 &&
          fm_ns_batched_workspace_bytes(e - i, g.rows[i], g.cols[i]) > workspace_bytes)
        return fail(FM_ERR_WORKSPACE, "group %d: matrices %d..%d need a larger Newton-Schulz workspace",
                    gi, i, e - 1);
      i = e;
    }
  }
  for (int l = 0; l < max_lanes; ++l)
    if (!workspaces[l]) return fail(FM_ERR_INVALID, "null workspace for lane %d", l);
  StepState* st = step_state();
  if (!st) return fail(FM_ERR_CUDA, "could not create the streams and events of the step");

  cudaStream_t main_stream = static_cast<cudaStream_t>(stream);
  cudaStream_t lanes[kMaxLanes] = {main_stream, st->lane[0], st->lane[1], st->lane[2]};
  // fork: the gradients were produced on the caller's stream
  FM_CUDA_CHECK(cudaEventRecord(st->fork, main_stream));
  for (int l = 1; l < kMaxLanes; ++l) FM_CUDA_CHECK(cudaStreamWaitEvent(lanes[l], st->fork, 0));

  int rc = FM_OK;
  char first_error[512] = {0};
  auto keep = [&](int code) {
    if (code != FM_OK && rc == FM_OK) {
      rc = code;
      snprintf(first_error, sizeof(first_error), "%s", fm_last_error());
    }
    return code == FM_OK;
  };
  auto cuda_ok = [&](cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
      cudaGetLastError();
      return keep(fail(FM_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e)));
    }
    return true;
  };
  const size_t pfloats = fm_norm_scratch_floats();

  for (int gi = 0; gi < ngroups && rc == FM_OK; ++gi) {
    const fm_muon_group& g = groups[gi];
    const int nl = g.lanes, nset = 2 * g.lanes;
    bool have_upd[kMaxSlots] = {false};
    // decay + update of matrices [i0, i1), whose updates lie in slot set `set`, on the side stream
    auto update = [&](int i0, int i1, int set) {
      if (!cuda_ok(cudaStreamWaitEvent(st->side, st->ns_done[set], 0), "cudaStreamWaitEvent")) return;
      void* p[kMaxGemmBatch];
      const void* u[kMaxGemmBatch];
      int64_t n[kMaxGemmBatch];
      double alpha[kMaxGemmBatch];
      for (int i = i0; i < i1; ++i) {
        p[i - i0] = g.params[i];
        u[i - i0] = g.slots[set * g.batch + (i - i0)];
        n[i - i0] = g.rows[i] * g.cols[i];
        alpha[i - i0] = g.alphas[i];
      }
      if (!keep(fm_update_multi(p, u, n, alpha, i1 - i0, g.p_dtype, g.decay, st->side))) return;
      if (cuda_ok(cudaEventRecord(st->upd_done[set], st->side), "cudaEventRecord")) have_upd[set] = true;
    };
    int prev_i0 = -1, prev_i1 = -1, prev_set = -1;
    int chunk = 0;
    for (int i0 = 0; i0 < g.count && rc == FM_OK; ++chunk) {
      const int i1 = chunk_end(g, i0);
      const int cnt = i1 - i0;
      const int set = chunk % nset;
      cudaStream_t lane = lanes[set % nl];
      if (have_upd[set]) {  // the slots of `set` are free once the update that read them has run
        if (!cuda_ok(cudaStreamWaitEvent(lane, st->upd_done[set], 0), "cudaStreamWaitEvent")) break;
        have_upd[set] = false;
      }
      if (g.rows[i0] * g.cols[i0] != 0) {
        char* ws = static_cast<char*>(workspaces[set % nl]);
        float* partials = reinterpret_cast<float*>(
            ws + fm_ns_batched_partials_offset(cnt, g.rows[i0], g.cols[i0]));
        MomentumItem mi[kMaxGemmBatch];
        const void* src[kMaxGemmBatch];
        void* dst[kMaxGemmBatch];
        for (int j = 0; j < cnt; ++j) {
          mi[j].grad = g.grads[i0 + j];
          mi[j].buf = g.momentum[i0 + j];
          mi[j].n = g.rows[i0 + j] * g.cols[i0 + j];
          mi[j].partials = partials + (size_t)j * pfloats;
          src[j] = g.nesterov ? g.grads[i0 + j] : g.momentum[i0 + j];
          dst[j] = g.slots[set * g.batch + j];
        }
        // momentum + Nesterov, leaving the partial sums of the norm behind (muon.py:99-100, :23)
        if (!keep(momentum_batch(mi, cnt, g.g_dtype, g.momentum_coef, g.nesterov, lane))) break;
        if (!keep(newtonschulz_batched(src, g.rows + i0, g.cols + i0, cnt, g.g_dtype, g.ns_steps, dst,
                                       ws, workspace_bytes, FM_NS_FAITHFUL | FM_NS_SUMSQ_READY, lane)))
          break;
      }
      if (!cuda_ok(cudaEventRecord(st->ns_done[set], lane), "cudaEventRecord")) break;
      if (prev_set >= 0) update(prev_i0, prev_i1, prev_set);
      prev_i0 = i0; prev_i1 = i1; prev_set = set;
      i0 = i1;
    }
    if (rc == FM_OK && prev_set >= 0) update(prev_i0, prev_i1, prev_set);
  }

  // join, also after an error: the caller's stream is again the only one with work pending
  cudaError_t e = cudaEventRecord(st->join_side, st->side);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(main_stream, st->join_side, 0);
  for (int l = 1; l < kMaxLanes && e == cudaSuccess; ++l) {
    e = cudaEventRecord(st->join_lane[l - 1], lanes[l]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(main_stream, st->join_lane[l - 1], 0);
  }
  cuda_ok(e, "joining the streams of the step");
  if (rc != FM_OK) return fail(rc, "%s", first_error);
  return FM_OK;
}
