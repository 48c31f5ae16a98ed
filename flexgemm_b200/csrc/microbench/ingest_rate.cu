// Micro-benchmark: do the two ways an SM pulls L2-resident data into shared memory -- 16-byte cp.async row gathers (the
// LSU path of the implicit-GEMM kernels' activation rows) and bulk async copies (the TMA path of their weight tiles) --
// share one per-SM limit, or do they add up?  One CTA per SM; every iteration brings in `rows` random 128-byte row
// slices with cp.async (256 threads, 3 or 6 groups in flight) and/or one contiguous `bulk_bytes` block with cp.async.bulk
// (one thread, as many copies in flight, completion on an mbarrier; every wait is bounded).
// Stand-alone (not part of the library):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o ingest_rate ingest_rate.cu && ./ingest_rate
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

constexpr int kMaxInFlight = 6;
constexpr uint32_t kRows = 163736, kRowBytes = 512;  // 84 MB: L2-resident

__device__ __forceinline__ bool wait_parity(uint64_t* bar, uint32_t parity) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(bar);
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

__global__ void ingest_kernel(const char* __restrict__ x, int rows, int bulk_bytes, int iters, int kInFlight, int* err) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t bar[kMaxInFlight];
  const int tid = threadIdx.x;
  const int gather_stage = rows * 128;
  uint8_t* bulk_base = smem + kInFlight * gather_stage;
  if (tid == 0) {
    for (int i = 0; i < kInFlight; ++i) {
      const uint32_t a = (uint32_t)__cvta_generic_to_shared(&bar[i]);
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(a));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int piece = tid & 7;
  const uint32_t blocks = kRows * kRowBytes / 32768u - 2u;  // the longest copy (64 KB) stays inside the matrix
  int slot = -1, round = 0;  // ring position and how often the ring has been walked, advanced by hand
  for (int it = 0; it < iters; ++it) {
    if (++slot == kInFlight) slot = 0, ++round;
    if (bulk_bytes > 0 && tid == blockDim.x - 1) {
      if (round > 0 && !wait_parity(&bar[slot], (round - 1) & 1)) {
        *err = 1;
        break;
      }
      const uint32_t b = (uint32_t)__cvta_generic_to_shared(&bar[slot]);
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(bulk_base + slot * bulk_bytes);
      const char* src = x + size_t((blockIdx.x * 7919u + it * 104729u) % blocks) * 32768u;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bulk_bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bulk_bytes), "r"(b) : "memory");
    }
    if (rows > 0 && tid < 256) {
      uint8_t* st = smem + slot * gather_stage;
      for (int r = tid >> 3; r < rows; r += 32) {
        const uint32_t row = (blockIdx.x * 7919u + it * 104729u + r * 977u + (r >> 3) * 15485863u) % kRows;
        const char* src = x + size_t(row) * kRowBytes + piece * 16 + (it & 3) * 128;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(st + r * 128 + ((piece ^ (r & 7)) << 4));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (kInFlight == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
      else asm volatile("cp.async.wait_group 5;" ::: "memory");
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (bulk_bytes > 0 && tid == blockDim.x - 1) {  // drain the copies still in flight before the CTA exits
    for (int it = iters > kInFlight ? iters - kInFlight : 0; it < iters; ++it)
      if (!wait_parity(&bar[it % kInFlight], (it / kInFlight) & 1)) *err = 1;
  }
  __syncthreads();
}

int main() {
  char* x;
  cudaMalloc(&x, size_t(kRows) * kRowBytes);
  cudaMemset(x, 1, size_t(kRows) * kRowBytes);
  int* err;
  cudaMalloc(&err, 4);
  cudaMemset(err, 0, 4);
  const int ctas = 148, iters = 402, threads = 288;  // iterations: a multiple of both ring depths
  struct Case { int rows, bulk, in_flight; };
  const Case cases[] = {{256, 0, 3}, {0, 32768, 3}, {256, 32768, 3}, {256, 16384, 3}, {128, 32768, 3}, {0, 16384, 3}, {0, 65536, 3},
                        {256, 0, 6},  {0, 32768, 6},  {128, 16384, 6}, {256, 0, 6}, {128, 0, 6}, {128, 0, 3}};
  for (const Case& c : cases) {
    const size_t smem = size_t(c.in_flight) * (c.rows * 128 + c.bulk);
    cudaFuncSetAttribute(ingest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    ingest_kernel<<<ctas, threads, smem>>>(x, c.rows, c.bulk, iters, c.in_flight, err);  // warms L2
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a);
    ingest_kernel<<<ctas, threads, smem>>>(x, c.rows, c.bulk, iters, c.in_flight, err);
    cudaEventRecord(b);
    cudaEventSynchronize(b);
    float ms;
    cudaEventElapsedTime(&ms, a, b);
    int h_err = 0;
    cudaMemcpy(&h_err, err, 4, cudaMemcpyDeviceToHost);
    const double gather = double(iters) * c.rows * 128, bulk = double(iters) * c.bulk;
    printf("in flight %d: gather %3d rows + bulk %5d B per iteration: %7.1f us   gather %5.1f + bulk %5.1f = %5.1f GB/s per SM   wait-timeout=%d cuda=%d\n", c.in_flight, c.rows,
           c.bulk, ms * 1e3, gather / (ms * 1e-3) / 1e9, bulk / (ms * 1e-3) / 1e9, (gather + bulk) / (ms * 1e-3) / 1e9, h_err,
           int(cudaGetLastError()));
  }
  return 0;
}
