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

// Encodes a 2-D row-major tensor map (inner = contiguous dimension) with the 128-byte swizzle.
// elem_bytes 2 only.  Returns FM_OK or an error status.
int encode_tmap_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer);

inline size_t dtype_bytes(int dtype) { return dtype == FM_F32 ? 4 : 2; }

}  // namespace fm
