// Operand splitting for the fp32-accurate (TF32-disabled) mode; see fgb_precision.cuh.
#include "fgb_precision.cuh"

namespace fgb {

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__global__ void __launch_bounds__(256) split3_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t rows, int C, int mode) {
  const int64_t i = blockIdx.x * int64_t(256) + threadIdx.x;
  if (i >= rows * C) return;
  const int64_t r = i / C;
  const int c = static_cast<int>(i - r * C);
  const float x = __ldg(&src[i]);
  const float hi = tf32_round(x), lo = x - hi;
  float* d = dst + r * 3 * C + c;
  d[0] = hi;
  d[C] = mode == kSplitActivations ? hi : lo;
  d[2 * C] = mode == kSplitActivations ? lo : hi;
}

__global__ void __launch_bounds__(256) split2_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo, int64_t count) {
  const int64_t i = blockIdx.x * int64_t(256) + threadIdx.x;
  if (i >= count) return;
  const float x = __ldg(&src[i]);
  const float h = tf32_round(x);
  hi[i] = h;
  lo[i] = x - h;
}

int launch_split3(const float* src, float* dst, int64_t rows, int C, SplitMode mode, cudaStream_t s) {
  const int64_t count = rows * C;
  if (count == 0) return FGB_OK;
  split3_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, s>>>(src, dst, rows, C, static_cast<int>(mode));
  return launch_status();
}

int launch_split2(const float* src, float* hi, float* lo, int64_t count, cudaStream_t s) {
  if (count == 0) return FGB_OK;
  split2_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, s>>>(src, hi, lo, count);
  return launch_status();
}

}  // namespace fgb
