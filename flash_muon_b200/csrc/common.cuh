// Host-side helpers shared by the translation units of the library: error reporting,
// device queries, the device-side "wait gave up" word, tensor-map encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/flash_muon_b200.h"

namespace fm {

// Thread-local message of the last failure; returns `code` so callers can `return fail(...)`.
int fail(int code, const char* fmt, ...);
void clear_error();

#define FM_CUDA_CHECK(expr)                                                                  \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return ::fm::fail(FM_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                                 \
  } while (0)

// Number of SMs of the current device (cached per device).
int sm_count();

// Address of the device word kernels set when a bounded wait runs out.
unsigned int* device_error_word();

// Encodes a 2-D row-major tensor map (inner = contiguous dimension) for 16-bit elements, with the
// 128-byte swizzle (box rows of 128 bytes) or without any.  Returns FM_OK or an error status.
int encode_tmap_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer, bool swizzle128 = true);

// Process-wide tuning switches (fm_set_option / fm_get_option).  Initial values come from the
// FM_GEMM_* / FM_PDL environment variables, read once when the library is first used; nothing on
// a launch path calls getenv.
struct Options {
  int gemm_impl = 0;     // 0: by tile count; 1: single-CTA kernel; 2: CTA-pair kernel
  int gemm_bn = 0;       // single-CTA kernel: 0 by tile count, 64, 128 or 256
  int gemm_stages = 0;   // CTA-pair kernel: 0 = default ring depth, else 2..7
  int gemm_balance = 1;  // 0: never cut the tail of a tile list by K blocks
  int gemm_strip = -1;   // symmetric lists of the pair kernel: -1 by size, 0 column order, w strips
  int pdl = 1;           // 0: launch the GEMM kernels without programmatic stream serialization
  int gemm_l2_promotion = 3;  // L2 promotion of the tensor maps: 0 none, 1 64 B, 2 128 B, 3 256 B
  int pdl_trigger = 0;   // when CTAs release the next kernel: 0 by schedule, 1 always early, 2 never
  int gemm_kb_per_stage = 2;  // pair kernel: 64-wide K blocks per pipeline stage (1..3)
  int gemm_tma_store = 1;  // 0: the pair kernel writes its outputs with per-lane global stores
  int gemm_tma_d = 1;      // 0: the pair kernel fetches the addend with per-lane global loads
};
Options& options();

inline size_t dtype_bytes(int dtype) { return dtype == FM_F32 ? 4 : 2; }

}  // namespace fm
