// Version and error strings of the C ABI.
#include "fgb_common.cuh"

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
