// Peer-memory plumbing for the copy-engine all-gather of Muon.step.
// The reference publishes each round's updates with one NCCL all-gather
// (flash_muon/muon.py:108).  NCCL's kernels need SMs, and the persistent GEMM kernels of the next
// round's Newton-Schulz hold every SM, so the two serialise instead of overlapping.  These entry
// points let the host side move the slots with DMA copy engines over NVLink and order everything
// with stream memory operations (a 32-bit flag written / waited on by the stream itself): no
// kernel, no SM, no host synchronisation.
//   fm_ipc_export / fm_ipc_import : CUDA IPC handle of the allocation behind a device pointer,
//                                   and the peer-mapped address of such an allocation
//   fm_copy_async                 : cudaMemcpyAsync device->device (peer addresses allowed)
//   fm_stream_write32 / fm_stream_wait32_geq : cuStreamWriteValue32 / cuStreamWaitValue32
// All loads from peer memory are plain DMA reads issued by copy engines.
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace fm {
namespace {

typedef CUresult (*WriteValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
typedef CUresult (*WaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
typedef CUresult (*DeviceGetAttributeFn)(int*, CUdevice_attribute, CUdevice);

struct DriverFns {
  WriteValue32Fn write32 = nullptr;
  WaitValue32Fn wait32 = nullptr;
  GetAddressRangeFn range = nullptr;
  DeviceGetAttributeFn attr = nullptr;
};

const DriverFns& driver() {
  static DriverFns fns;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* name) -> void* {
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
          q != cudaDriverEntryPointSuccess)
        return nullptr;
      return p;
    };
    fns.write32 = reinterpret_cast<WriteValue32Fn>(get("cuStreamWriteValue32"));
    fns.wait32 = reinterpret_cast<WaitValue32Fn>(get("cuStreamWaitValue32"));
    fns.range = reinterpret_cast<GetAddressRangeFn>(get("cuMemGetAddressRange"));
    fns.attr = reinterpret_cast<DeviceGetAttributeFn>(get("cuDeviceGetAttribute"));
  });
  return fns;
}

struct Imported {
  cudaIpcMemHandle_t handle;
  int device;
  void* base;
};
std::mutex g_import_mu;
std::vector<Imported> g_imports;

// 1 if a wait may be followed by a flush of remote writes on the current device, 0 if not.
int can_flush_remote_writes() {
  static int cached[64];
  static bool known[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!known[dev]) {
    int v = 0;
    const DriverFns& d = driver();
    if (d.attr && d.attr(&v, CU_DEVICE_ATTRIBUTE_CAN_FLUSH_REMOTE_WRITES, (CUdevice)dev) != CUDA_SUCCESS)
      v = 0;
    cached[dev] = v;
    known[dev] = true;
  }
  return cached[dev];
}

}  // namespace
}  // namespace fm

extern "C" int fm_ipc_export(const void* ptr, unsigned char* handle64, uint64_t* offset) {
  using namespace fm;
  clear_error();
  if (!ptr || !handle64 || !offset) return fail(FM_ERR_INVALID, "null pointer");
  const DriverFns& d = driver();
  if (!d.range) return fail(FM_ERR_CUDA, "cuMemGetAddressRange is not available");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = d.range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) return fail(FM_ERR_CUDA, "cuMemGetAddressRange failed (%d)", (int)r);
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(FM_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  memcpy(handle64, &h, 64);
  *offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
  return FM_OK;
}

extern "C" int fm_ipc_import(const unsigned char* handle64, uint64_t offset, void** ptr) {
  using namespace fm;
  clear_error();
  if (!handle64 || !ptr) return fail(FM_ERR_INVALID, "null pointer");
  int dev = 0;
  FM_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_import_mu);
  for (const Imported& im : g_imports) {
    if (im.device == dev && memcmp(&im.handle, handle64, 64) == 0) {
      *ptr = static_cast<char*>(im.base) + offset;
      return FM_OK;
    }
  }
  Imported im;
  memcpy(&im.handle, handle64, 64);
  im.device = dev;
  im.base = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&im.base, im.handle, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(FM_ERR_CUDA, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  }
  g_imports.push_back(im);
  *ptr = static_cast<char*>(im.base) + offset;
  return FM_OK;
}

extern "C" int fm_ipc_close_all(void) {
  using namespace fm;
  clear_error();
  std::lock_guard<std::mutex> lock(g_import_mu);
  for (const Imported& im : g_imports) cudaIpcCloseMemHandle(im.base);
  cudaGetLastError();
  g_imports.clear();
  return FM_OK;
}

extern "C" int fm_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
  using namespace fm;
  clear_error();
  if (bytes == 0) return FM_OK;
  if (!dst || !src) return fail(FM_ERR_INVALID, "null pointer");
  FM_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice,
                                static_cast<cudaStream_t>(stream)));
  return FM_OK;
}

extern "C" int fm_stream_write32(void* addr, uint32_t value, void* stream) {
  using namespace fm;
  clear_error();
  if (!addr || (reinterpret_cast<uintptr_t>(addr) & 3u)) return fail(FM_ERR_INVALID, "bad flag address");
  const DriverFns& d = driver();
  if (!d.write32) return fail(FM_ERR_CUDA, "cuStreamWriteValue32 is not available");
  const CUresult r = d.write32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(addr),
                               value, CU_STREAM_WRITE_VALUE_DEFAULT);
  if (r != CUDA_SUCCESS) return fail(FM_ERR_CUDA, "cuStreamWriteValue32 failed (%d)", (int)r);
  return FM_OK;
}

extern "C" int fm_stream_wait32_geq(const void* addr, uint32_t value, void* stream) {
  using namespace fm;
  clear_error();
  if (!addr || (reinterpret_cast<uintptr_t>(addr) & 3u)) return fail(FM_ERR_INVALID, "bad flag address");
  const DriverFns& d = driver();
  if (!d.wait32) return fail(FM_ERR_CUDA, "cuStreamWaitValue32 is not available");
  unsigned int flags = CU_STREAM_WAIT_VALUE_GEQ;
  if (can_flush_remote_writes()) flags |= CU_STREAM_WAIT_VALUE_FLUSH;
  const CUresult r = d.wait32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(addr),
                              value, flags);
  if (r != CUDA_SUCCESS) return fail(FM_ERR_CUDA, "cuStreamWaitValue32 failed (%d)", (int)r);
  return FM_OK;
}
