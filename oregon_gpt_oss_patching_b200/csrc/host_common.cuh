// Host-side helpers shared by the translation units of the library: the driver's tensor-map
// encoder, a device guard, the device check and the per-(kernel, device) shared-memory attribute.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/b200attn.h"

namespace b200attn {
namespace host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up once; the pointer is immutable afterwards.
inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Makes `device` current for the duration of a call and restores the caller's device after.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != device && cudaSetDevice(device) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

inline int check_device(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return B200ATTN_ECUDA;
  return major == 10 ? B200ATTN_OK : B200ATTN_EDEVICE;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Raises a kernel's dynamic shared-memory limit.  The attribute belongs to the (kernel, device) pair and
// never changes afterwards, so it is set once per pair instead of on every launch.
constexpr int kMaxDevices = 64;
template <auto kKernel>
int set_smem(size_t bytes) {
  static std::atomic<bool> done[kMaxDevices];   // one array per kernel; zero-initialised
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return B200ATTN_ECUDA;
  const bool cacheable = device >= 0 && device < kMaxDevices;
  if (cacheable && done[device].load(std::memory_order_acquire)) return B200ATTN_OK;
  if (cudaFuncSetAttribute(kKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
    return B200ATTN_ECUDA;
  if (cacheable) done[device].store(true, std::memory_order_release);
  return B200ATTN_OK;
}


inline int launch_status() { return cudaGetLastError() == cudaSuccess ? B200ATTN_OK : B200ATTN_ECUDA; }

}  // namespace host
}  // namespace b200attn
