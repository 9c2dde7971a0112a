// Error reporting, device queries and tensor-map encoding shared by the library.
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace fm {

namespace {
thread_local char tl_error[512] = {0};
constexpr int kMaxDevices = 64;

// Set by a kernel whose bounded wait ran out; one instance per device that loads the library.
__device__ unsigned int g_wait_error = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return code;
}
void clear_error() { tl_error[0] = 0; }

Options& options() {
  static Options opt;
  static std::once_flag once;
  std::call_once(once, [] {
    auto env = [](const char* name, int* dst) {
      if (const char* e = getenv(name)) *dst = atoi(e);
    };
    env("FM_GEMM_IMPL", &opt.gemm_impl);
    env("FM_GEMM_BN", &opt.gemm_bn);
    env("FM_GEMM_STAGES", &opt.gemm_stages);
    env("FM_GEMM_BALANCE", &opt.gemm_balance);
    env("FM_GEMM_STRIP", &opt.gemm_strip);
    env("FM_PDL", &opt.pdl);
    env("FM_GEMM_TMA_STORE", &opt.gemm_tma_store);
    env("FM_GEMM_TMA_D", &opt.gemm_tma_d);
    env("FM_GEMM_KB_PER_STAGE", &opt.gemm_kb_per_stage);
    env("FM_PDL_TRIGGER", &opt.pdl_trigger);
    env("FM_GEMM_L2_PROMOTION", &opt.gemm_l2_promotion);
  });
  return opt;
}

namespace {
int* option_slot(const char* name) {
  Options& o = options();
  if (!name) return nullptr;
  if (!strcmp(name, "gemm_impl")) return &o.gemm_impl;
  if (!strcmp(name, "gemm_bn")) return &o.gemm_bn;
  if (!strcmp(name, "gemm_stages")) return &o.gemm_stages;
  if (!strcmp(name, "gemm_balance")) return &o.gemm_balance;
  if (!strcmp(name, "gemm_strip")) return &o.gemm_strip;
  if (!strcmp(name, "pdl")) return &o.pdl;
  if (!strcmp(name, "gemm_tma_store")) return &o.gemm_tma_store;
  if (!strcmp(name, "gemm_tma_d")) return &o.gemm_tma_d;
  if (!strcmp(name, "gemm_kb_per_stage")) return &o.gemm_kb_per_stage;
  if (!strcmp(name, "pdl_trigger")) return &o.pdl_trigger;
  if (!strcmp(name, "gemm_l2_promotion")) return &o.gemm_l2_promotion;
  return nullptr;
}
}  // namespace

int sm_count() {
  static int cached[kMaxDevices] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

unsigned int* device_error_word() {
  static unsigned int* cached[kMaxDevices] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_wait_error) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned int*>(p);
  }
  return cached[dev];
}

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tmap_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(FM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMapDataType dt;
  if (dtype == FM_BF16)
    dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else if (dtype == FM_F16)
    dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  else
    return fail(FM_ERR_UNSUPPORTED, "tensor maps are built for 16-bit types only");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_elems * 2) % 16 != 0)
    return fail(FM_ERR_INVALID, "operand base and row pitch must be multiples of 16 bytes");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  options().gemm_l2_promotion == 0   ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                  : options().gemm_l2_promotion == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                  : options().gemm_l2_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                     : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FM_OK;
}

}  // namespace fm

extern "C" int fm_version(void) { return 200; }

extern "C" int fm_set_option(const char* name, int value) {
  fm::clear_error();
  int* slot = fm::option_slot(name);
  if (!slot) return fm::fail(FM_ERR_INVALID, "unknown option '%s'", name ? name : "(null)");
  *slot = value;
  return FM_OK;
}

extern "C" int fm_get_option(const char* name, int* value) {
  fm::clear_error();
  int* slot = fm::option_slot(name);
  if (!slot || !value) return fm::fail(FM_ERR_INVALID, "unknown option '%s'", name ? name : "(null)");
  *value = *slot;
  return FM_OK;
}

extern "C" const char* fm_last_error(void) { return fm::tl_error; }

extern "C" int fm_device_status(unsigned int* code) {
  unsigned int* w = fm::device_error_word();
  if (!w) return fm::fail(FM_ERR_CUDA, "no current CUDA device");
  FM_CUDA_CHECK(cudaDeviceSynchronize());
  unsigned int v = 0;
  FM_CUDA_CHECK(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
  if (code) *code = v;
  if (v != 0) {
    unsigned int zero = 0;
    FM_CUDA_CHECK(cudaMemcpy(w, &zero, sizeof(zero), cudaMemcpyHostToDevice));
    return fm::fail(FM_ERR_DEVICE_WAIT, "a kernel gave up a bounded wait (code 0x%08x)", v);
  }
  return FM_OK;
}
