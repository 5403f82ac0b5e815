// Host-side launch helpers shared by every kernel launcher of the library.
#pragma once

#include <cuda_runtime.h>

#include <atomic>

namespace lf {

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the CURRENT device only, so
// "done once" has to be remembered per device: a process that drives several GPUs would
// otherwise launch with the default 48 KB limit on every device but the first.  One instance
// per kernel (a function-local static in its launcher); safe to use from several host threads.
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  std::atomic<bool> done[kMaxDevices];
  PerDeviceOnce() {
    for (auto& d : done) d.store(false, std::memory_order_relaxed);
  }
};

// Raise the dynamic shared-memory limit of `kern` on the current device unless this was
// already done there.  Returns cudaSuccess or the error of the failing call.
template <typename Kernel>
inline cudaError_t ensure_max_dynamic_smem(PerDeviceOnce& once, Kernel kern, int smem_bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < PerDeviceOnce::kMaxDevices;
  if (tracked && once.done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e == cudaSuccess && tracked) once.done[dev].store(true, std::memory_order_release);
  return e;
}

}  // namespace lf
