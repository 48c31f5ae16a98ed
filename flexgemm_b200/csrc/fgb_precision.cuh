// fp32-accurate products on TF32 tensor cores.
//
// With TF32 disabled for fp32 inputs, every operand x is split into
//   hi = x rounded to TF32 (10 mantissa bits),   lo = x - hi  (exact in fp32),
// and a product a*b is evaluated as  a_hi*b_hi + a_hi*b_lo + a_lo*b_hi  with
// fp32 accumulation; the dropped lo*lo term and the truncation of lo are below
// 2^-21 relative.  For fprop and dgrad the three products are folded into ONE
// run of the TF32 kernel by tripling the reduction (channel) dimension:
//   activations  [hi | hi | lo],   weights  [hi | lo | hi].
// wgrad reduces over pairs, not channels, so it runs three passes that add into
// the same fp32 output.
#pragma once

#include "fgb_common.cuh"

namespace fgb {

enum SplitMode { kSplitActivations = 0, kSplitWeights = 1 };

// dst[r, 0:C | C:2C | 2C:3C] = [hi|hi|lo] (activations) or [hi|lo|hi] (weights) of src[r, 0:C]
int launch_split3(const float* src, float* dst, int64_t rows, int C, SplitMode mode, cudaStream_t s);
// hi[i] = tf32(src[i]), lo[i] = src[i] - hi[i]
int launch_split2(const float* src, float* hi, float* lo, int64_t count, cudaStream_t s);

inline int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

}  // namespace fgb
