// Per-device bookkeeping of the host side of the library.
//
// One process may drive several GPUs and call the entry points from several
// threads.  Two things the launch code wants to remember are properties of a
// DEVICE, not of the process: the number of SMs (grid size of the persistent
// kernels) and the dynamic shared-memory limit a kernel has been configured
// with (cudaFuncSetAttribute applies to the current device only).  Both caches
// here are keyed by the device index and guarded by a mutex.
#pragma once

#include <cuda_runtime.h>

#include <mutex>

#include "fgb_common.cuh"

namespace fgb {

constexpr int kMaxDevices = 64;

// Table of one non-negative value per device; `get` fills an entry on first use through `query(device)`.
// The table itself knows nothing about CUDA, so its logic can be exercised on a machine without a GPU.
class PerDeviceTable {
 public:
  template <typename Query>
  int64_t get(int device, Query query) {
    if (device < 0 || device >= kMaxDevices) return query(device);
    std::lock_guard<std::mutex> lock(mu_);
    if (!known_[device]) {
      const int64_t v = query(device);
      if (v < 0) return v;  // not cached: the query failed
      value_[device] = v;
      known_[device] = true;
    }
    return value_[device];
  }
  // raises the entry to at least `need`; `apply(device, need)` runs (under the lock) only when it has to grow and
  // returns 0 on success
  template <typename Apply>
  int raise_to(int device, int64_t need, Apply apply) {
    if (device < 0 || device >= kMaxDevices) return apply(device, need);
    std::lock_guard<std::mutex> lock(mu_);
    if (known_[device] && value_[device] >= need) return 0;
    const int rc = apply(device, need);
    if (rc != 0) return rc;
    value_[device] = need;
    known_[device] = true;
    return 0;
  }

 private:
  std::mutex mu_;
  int64_t value_[kMaxDevices] = {};
  bool known_[kMaxDevices] = {};
};

inline int current_device() {
  int dev = 0;
  return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

// SMs of the current device (148 when the query fails: the part this library is written for)
inline int device_sm_count() {
  static PerDeviceTable table;
  const int64_t n = table.get(current_device(), [](int dev) -> int64_t {
    int sms = 0;
    if (dev < 0 || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -1;
    return sms;
  });
  return n > 0 ? static_cast<int>(n) : 148;
}

// Makes sure `kernel` may be launched with `bytes` of dynamic shared memory on the current device.  `table` is the
// kernel's own (one per kernel instance: a function-static at the call site).
template <typename Kernel>
inline int ensure_dynamic_smem(PerDeviceTable& table, Kernel kernel, size_t bytes) {
  return table.raise_to(current_device(), static_cast<int64_t>(bytes), [&](int, int64_t need) -> int {
    return cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(need)));
  });
}

// Chained launches (programmatic dependent launch).  A kernel started with launch_chained may be set up on the SMs
// while the kernel before it in the stream is still running.  It must call chain_wait() before it touches global
// memory: the call returns once the earlier kernel has completed and its writes are visible (at once when the kernel
// was launched the ordinary way).  chain_release() lets the next chained kernel of the stream begin its own set-up; the
// next kernel is not started before every CTA of this one has called it or exited, so a chain cannot starve itself.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// first error of a sequence of launches
struct LaunchErrors {
  cudaError_t first = cudaSuccess;
  void add(cudaError_t e) {
    if (e != cudaSuccess && first == cudaSuccess) first = e;
  }
};

}  // namespace fgb
