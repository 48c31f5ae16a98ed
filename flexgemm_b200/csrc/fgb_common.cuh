// Shared host/device helpers of the flexgemm_b200 library.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flexgemm_b200.h"

namespace fgb {

constexpr uint32_t kInvalid = 0xFFFFFFFFu;
constexpr int kMapBlock = 256;  // voxels per CTA in the map / compaction kernels

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? FGB_OK : FGB_E_CUDA_BASE + static_cast<int>(e); }

// Launch-error check that does not synchronise.
inline int launch_status() { return cuda_status(cudaPeekAtLastError()); }

__device__ __forceinline__ void report(int32_t* status, int32_t code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

inline int elem_bytes(int dtype) {
  switch (dtype) {
    case FGB_F16:
    case FGB_BF16:
      return 2;
    case FGB_F32_TF32:
    case FGB_F32_IEEE:
      return 4;
    default:
      return 0;
  }
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// fprop / dgrad of a small input (fewer work items than SMs) split every item's offsets into shares that run as
// separate items into fp32 slabs (fgb_igemm.cu): the number of shares for n output rows x nout channels on the current
// device, and the bytes of the slabs (0 when the launch is not split).  The workspace sizes are built from these.
int igemm_splits(int64_t n, int nout, int V);
int64_t igemm_partial_bytes(int64_t n, int nout, int V);

#ifdef __CUDACC__
// Murmur3 finalisers: the hash of every table in the library
__device__ __forceinline__ uint32_t fmix32(uint32_t k) {
  k ^= k >> 16;
  k *= 0x85ebca6bu;
  k ^= k >> 13;
  k *= 0xc2b2ae35u;
  k ^= k >> 16;
  return k;
}
__device__ __forceinline__ uint32_t fmix64_hi(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return static_cast<uint32_t>(k >> 32) ^ static_cast<uint32_t>(k);
}
#endif

// Tensor map over a row-major matrix of 16-bit elements whose box is 128 bytes of one row (fgb_igemm.cu).
int make_rows_tmap(CUtensorMap* map, const void* rows, int64_t n_rows, int row_elems);

}  // namespace fgb
