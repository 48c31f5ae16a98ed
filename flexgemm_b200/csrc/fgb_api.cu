// Version and error strings of the C ABI.
#include "fgb_common.cuh"
#include "fgb_device.cuh"

extern "C" const char* fgb_version(void) { return "flexgemm_b200 0.1.0 (sm_100a)"; }

extern "C" const char* fgb_error_string(int code) {
  switch (code) {
    case FGB_OK:
      return "ok";
    case FGB_E_NULL:
      return "a required pointer is null";
    case FGB_E_SIZE:
      return "a size or count is out of range";
    case FGB_E_DTYPE:
      return "unsupported element type or key width";
    case FGB_E_ALIGN:
      return "pointer or channel count is not 16-byte aligned";
    case FGB_E_WORKSPACE:
      return "workspace too small";
    case FGB_E_DRIVER:
      return "CUDA driver entry point unavailable or tensor map rejected";
    case FGB_E_STATIC_LIMIT:
      return "size exceeds the built-in scratch of the no-allocation entry point";
    default:
      break;
  }
  if (code >= FGB_E_CUDA_BASE) return cudaGetErrorString(static_cast<cudaError_t>(code - FGB_E_CUDA_BASE));
  return "unknown error";
}

// Host-only check of the per-device caches behind the launch code (no CUDA call): an entry is queried once per
// device, devices do not share entries, a failed query is not cached, and a limit is applied again only when it
// has to grow.  Returns 0, or the number of the first expectation that failed.
extern "C" int fgb_selftest_device_tables(void) {
  using fgb::PerDeviceTable;
  PerDeviceTable sms;
  int queries = 0;
  auto q = [&](int dev) -> int64_t {
    ++queries;
    return dev == 3 ? -1 : 100 + dev;
  };
  if (sms.get(0, q) != 100 || sms.get(1, q) != 101 || sms.get(0, q) != 100 || queries != 2) return 1;
  if (sms.get(3, q) != -1 || sms.get(3, q) != -1 || queries != 4) return 2;  // failures are asked again
  if (sms.get(-1, q) != 99 || sms.get(fgb::kMaxDevices, q) != 100 + fgb::kMaxDevices) return 3;  // out of range: not cached
  PerDeviceTable limit;
  int applied = 0, fail = 0;
  auto a = [&](int, int64_t) -> int {
    if (fail) return fail;
    ++applied;
    return 0;
  };
  if (limit.raise_to(0, 1000, a) != 0 || limit.raise_to(0, 500, a) != 0 || applied != 1) return 4;
  if (limit.raise_to(1, 500, a) != 0 || applied != 2) return 5;  // another device starts from nothing
  if (limit.raise_to(0, 2000, a) != 0 || applied != 3) return 6;
  fail = 7;
  if (limit.raise_to(0, 4000, a) != 7) return 7;
  fail = 0;
  if (limit.raise_to(0, 3000, a) != 0 || applied != 4) return 8;  // the failed raise left the old limit in place
  return 0;
}

// Device-to-host copy of a few words on `stream` (the neighbour-cache build fetches its pair count and status this way);
// host_dst should be pinned memory, else the copy is not asynchronous.  (A one-warp kernel storing the words into the
// pinned buffer was measured against this call: no difference for the build.)
extern "C" int fgb_fetch_words_async(void* host_dst, const void* device_src, int64_t bytes, void* stream) {
  if (bytes < 0) return FGB_E_SIZE;
  if (bytes == 0) return FGB_OK;
  if (!host_dst || !device_src) return FGB_E_NULL;
  return fgb::cuda_status(cudaMemcpyAsync(host_dst, device_src, static_cast<size_t>(bytes), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
}
