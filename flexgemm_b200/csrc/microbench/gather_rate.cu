// Micro-benchmark: the rate at which one CTA per SM can gather random 128-byte row slices of an L2-resident
// matrix into a 128B-swizzled shared-memory tile -- the access pattern of the implicit-GEMM kernels' gather warps --
// for several thread counts, numbers of cp.async groups in flight, and with plain loads + stores for comparison.
// Stand-alone (not part of the library):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o gather_rate gather_rate.cu && ./gather_rate
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <vector>
#include <random>
template <int MODE>  // 0: cp.async.cg 16B  1: cp.async.ca 16B  2: ld.global.v4 + st.shared
__global__ void gather_kernel(const char* __restrict__ x, const uint32_t* __restrict__ idx, int rows_per_cta_iter, int iters,
                              int row_bytes, int groups_in_flight, unsigned long long* out_ns) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int piece = tid & 7;
  const int lanes_rows = nthr / 8;           // rows covered per pass
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  (void)idx;  // the row indices are computed in registers below, so that nothing but the copies is timed
  const int stage_bytes = rows_per_cta_iter * 128;
  float4 sink = make_float4(0, 0, 0, 0);
  int slot = 0;
  for (int it = 0; it < iters; ++it) {
    uint8_t* st = smem + slot * stage_bytes;
    if (++slot == groups_in_flight) slot = 0;
    for (int r = tid >> 3; r < rows_per_cta_iter; r += lanes_rows) {
      const uint32_t row = (blockIdx.x * 7919u + it * 104729u + r * 977u + (r >> 3) * 15485863u) % 163736u;
      const char* src = x + (size_t)row * 512 + piece * 16 + (it & 3) * 128;  // constants: a runtime modulo here made an earlier version ALU-bound
      uint32_t dst = (uint32_t)__cvta_generic_to_shared(st + r * 128 + ((piece ^ (r & 7)) << 4));
      if (MODE == 0) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      else if (MODE == 1) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      else { float4 v = __ldg((const float4*)src); *(float4*)(st + r * 128 + ((piece ^ (r & 7)) << 4)) = v; }
    }
    if (MODE < 2) {
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (groups_in_flight == 1) asm volatile("cp.async.wait_group 0;" ::: "memory");
      else if (groups_in_flight == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else if (groups_in_flight == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
      else if (groups_in_flight == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
      else asm volatile("cp.async.wait_group 5;" ::: "memory");
    }
  }
  if (MODE < 2) asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  sink.x += smem[tid];
  unsigned long long t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
  if (tid == 0) out_ns[blockIdx.x] = t1 - t0 + (sink.x == 12345.f);
}
int main() {
  const int n_rows = 163736, row_bytes = 512;
  char* x; cudaMalloc(&x, (size_t)n_rows * row_bytes); cudaMemset(x, 1, (size_t)n_rows * row_bytes);
  const int ctas = 148, iters = 400;
  std::mt19937 rng(1);
  for (int rows : {256}) {
    std::vector<uint32_t> h((size_t)ctas * iters * rows);
    for (auto& v : h) v = rng() % n_rows;
    uint32_t* idx; cudaMalloc(&idx, h.size() * 4); cudaMemcpy(idx, h.data(), h.size() * 4, cudaMemcpyHostToDevice);
    unsigned long long* ns; cudaMalloc(&ns, ctas * 8);
    for (int threads : {128, 256, 512, 1024}) for (int gif : {1, 2, 3, 4, 6}) for (int mode : {0, 2}) {
      if (gif == 6 && mode == 2) continue;
      size_t smem = (size_t)gif * rows * 128;
      if (smem > 200 * 1024) continue;
      auto launch = [&](auto kern) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kern<<<ctas, threads, smem>>>(x, idx, rows, iters, row_bytes, gif, ns);  // warm L2
        cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
        cudaEventRecord(a);
        kern<<<ctas, threads, smem>>>(x, idx, rows, iters, row_bytes, gif, ns);
        cudaEventRecord(b); cudaEventSynchronize(b);
        float ms; cudaEventElapsedTime(&ms, a, b);
        double bytes = (double)ctas * iters * rows * 128;
        printf("rows/iter %4d threads %4d in-flight %d mode %d : %7.1f us  %6.1f GB/s per SM  %6.2f TB/s total  err=%d\n", rows, threads, gif, mode,
               ms * 1e3, bytes / ctas / (ms * 1e-3) / 1e9, bytes / (ms * 1e-3) / 1e12, (int)cudaGetLastError());
      };
      if (mode == 0) launch(gather_kernel<0>); else if (mode == 1) launch(gather_kernel<1>); else launch(gather_kernel<2>);
    }
    // The same gather with fewer CTAs (one per SM, fewer SMs busy): if the rate per SM rises, the ceiling above is the L2's
    // output as a whole; if it stays, it is each SM's own port.
    for (int fewer : {148, 111, 74, 37, 16}) {
      const int threads = 512, gif = 3;
      const size_t smem = (size_t)gif * rows * 128;
      cudaFuncSetAttribute(gather_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      gather_kernel<0><<<fewer, threads, smem>>>(x, idx, rows, iters, row_bytes, gif, ns);
      cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
      cudaEventRecord(a);
      gather_kernel<0><<<fewer, threads, smem>>>(x, idx, rows, iters, row_bytes, gif, ns);
      cudaEventRecord(b); cudaEventSynchronize(b);
      float ms; cudaEventElapsedTime(&ms, a, b);
      const double bytes = (double)fewer * iters * rows * 128;
      printf("CTAs %4d threads %4d in-flight %d mode 0 : %7.1f us  %6.1f GB/s per SM  %6.2f TB/s total  err=%d\n", fewer, threads, gif,
             ms * 1e3, bytes / fewer / (ms * 1e-3) / 1e9, bytes / (ms * 1e-3) / 1e12, (int)cudaGetLastError());
    }
    cudaFree(idx); cudaFree(ns);
  }
  return 0;
}
