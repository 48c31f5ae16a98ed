// Post-processing of the neighbour map for the masked implicit GEMM:
// wgrad pair lists, per-tile offset masks and their list form (the sorted row
// order is in fgb_sort.cu).
#include "fgb_common.cuh"
#include "fgb_device.cuh"

namespace fgb {

// ------------------------------------------------------------------ pair lists
// One CTA per 256 voxels (the blocking of the lookup kernel, whose per-block
// counts were scanned into block_offsets).  The CTA's slice of the map is
// staged in shared memory with coalesced loads; rank inside the CTA comes from
// warp ballots, so every offset's list keeps ascending row order.
//
// Rows in key order (submanifold map, *unsorted == 0) need no map at all: a translation keeps the key order, so the
// neighbours of offset v's output rows, in list order, are exactly the output rows of the opposite offset V-1-v in
// their list order -- valid_signal_i of offset v is valid_signal_o of offset V-1-v, and both follow from the masks.
__global__ void __launch_bounds__(kMapBlock)
    valid_signal_kernel(const uint32_t* __restrict__ nbr, const int32_t* __restrict__ gray, uint32_t n, int V,
                        const uint32_t* __restrict__ block_offsets, uint32_t nblk, const uint32_t* __restrict__ seg,
                        uint32_t* __restrict__ vs_i, uint32_t* __restrict__ vs_o, const uint32_t* __restrict__ unsorted) {
  extern __shared__ uint32_t s_map[];     // [256 * V]
  __shared__ uint32_t s_wcount[32][8];    // valid rows per (offset, warp), then exclusive prefix
  __shared__ uint32_t s_base[32];         // list position of the CTA's first pair, per offset
  __shared__ uint32_t s_base_opp[32];     // the same position in the opposite offset's list
  const uint32_t n0 = blockIdx.x * kMapBlock;
  const uint32_t nv = min(static_cast<uint32_t>(kMapBlock), n - n0);
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  chain_release();
  chain_wait();
  const bool mirror = unsorted != nullptr && __ldg(unsorted) == 0u;  // the same for every thread of the grid
  if (!mirror) {
    const uint32_t words = nv * V;
    const uint32_t* src = nbr + static_cast<size_t>(n0) * V;
    for (uint32_t i = t; i < words; i += kMapBlock) s_map[i] = __ldg(&src[i]);
  }
  const uint32_t g = t < nv ? static_cast<uint32_t>(__ldg(&gray[n0 + t])) : 0u;
  if (t < V) {
    const uint32_t in_list = block_offsets[static_cast<size_t>(t) * nblk + blockIdx.x];
    s_base[t] = seg[t] + in_list;
    s_base_opp[t] = seg[V - 1 - t] + in_list;
  }
  for (int v = 0; v < V; ++v) {
    const uint32_t b = __ballot_sync(0xffffffffu, (g >> v) & 1u);
    if (lane == 0) s_wcount[v][w] = __popc(b);
  }
  __syncthreads();
  if (t < V) {
    uint32_t acc = 0;
    for (int i = 0; i < 8; ++i) {
      uint32_t c = s_wcount[t][i];
      s_wcount[t][i] = acc;
      acc += c;
    }
  }
  __syncthreads();
  for (int v = 0; v < V; ++v) {
    const bool ok = (g >> v) & 1u;
    const uint32_t b = __ballot_sync(0xffffffffu, ok);
    if (ok) {
      const uint32_t rank = s_wcount[v][w] + __popc(b & ((1u << lane) - 1u));
      vs_o[s_base[v] + rank] = n0 + t;
      if (mirror) vs_i[s_base_opp[v] + rank] = n0 + t;
      else vs_i[s_base[v] + rank] = s_map[t * V + v];
    }
  }
}

// ------------------------------------------------------------------ tile masks
// one warp per tile of `block` sorted rows
__global__ void tile_mask_kernel(const int32_t* __restrict__ gray, const int64_t* __restrict__ sorted_idx, int64_t n, int block,
                                 int64_t ntiles, uint32_t* __restrict__ masks) {
  const int64_t tile = (blockIdx.x * int64_t(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tile >= ntiles) return;
  uint32_t m = 0;
  const int64_t r0 = tile * block;
  for (int i = lane; i < block; i += 32) {
    const int64_t r = r0 + i;
    if (r < n) m |= static_cast<uint32_t>(__ldg(&gray[__ldg(&sorted_idx[r])]));
  }
  m = __reduce_or_sync(0xffffffffu, m);
  if (lane == 0) masks[tile] = m;
}

// single CTA: seg = exclusive scan of popcounts, then expand the set bits
__global__ void __launch_bounds__(1024)
    valid_kernel_kernel(const uint32_t* __restrict__ masks, uint32_t nblk, int32_t* __restrict__ vk, int32_t* __restrict__ seg) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  if (t == 0) {
    s_carry = 0;
    seg[0] = 0;
  }
  __syncthreads();
  for (uint32_t base = 0; base < nblk; base += 1024) {
    const uint32_t i = base + t;
    uint32_t m = i < nblk ? __ldg(&masks[i]) : 0u;
    const uint32_t x = __popc(m);
    uint32_t inc = x;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += y;
    }
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    if (w == 0) {
      uint32_t ws = s_warp[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        uint32_t y = __shfl_up_sync(0xffffffffu, ws, d);
        if (lane >= d) ws += y;
      }
      s_warp[lane] = ws;
    }
    __syncthreads();
    const uint32_t carry = s_carry;
    const uint32_t end = carry + (w == 0 ? 0u : s_warp[w - 1]) + inc;
    if (i < nblk) {
      seg[i + 1] = static_cast<int32_t>(end);
      uint32_t pos = end - x;
      while (m) {
        const int bit = __ffs(m) - 1;
        vk[pos++] = bit;
        m &= m - 1;
      }
    }
    __syncthreads();
    if (t == 1023) s_carry = carry + s_warp[31];
    __syncthreads();
  }
}

}  // namespace fgb

extern "C" int fgb_pp_valid_signal(const uint32_t* neighbor_map, const int32_t* gray_code, int64_t n, int V,
                                   const uint32_t* block_offsets, const uint32_t* valid_signal_seg, uint32_t* valid_signal_i,
                                   uint32_t* valid_signal_o, const uint32_t* unsorted_flag, void* stream) {
  using namespace fgb;
  if (n < 0 || n >= (int64_t(1) << 32) - 1 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!neighbor_map || !gray_code || !block_offsets || !valid_signal_seg || !valid_signal_i || !valid_signal_o) return FGB_E_NULL;
  const uint32_t nblk = static_cast<uint32_t>(ceil_div(n, kMapBlock));
  const size_t smem = size_t(kMapBlock) * V * sizeof(uint32_t);
  const cudaError_t e = launch_chained(valid_signal_kernel, dim3(nblk), dim3(kMapBlock), smem, static_cast<cudaStream_t>(stream), neighbor_map,
                                       gray_code, static_cast<uint32_t>(n), V, block_offsets, nblk, valid_signal_seg, valid_signal_i,
                                       valid_signal_o, unsorted_flag);
  if (e != cudaSuccess) return cuda_status(e);
  return launch_status();
}

extern "C" int fgb_pp_tile_masks(const int32_t* gray_code, const int64_t* sorted_idx, int64_t n, int block, uint32_t* tile_masks,
                                 void* stream) {
  using namespace fgb;
  if (n < 0 || block < 8 || block > 1024 || (block & (block - 1))) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!gray_code || !sorted_idx || !tile_masks) return FGB_E_NULL;
  const int64_t ntiles = ceil_div(n, block);
  tile_mask_kernel<<<static_cast<unsigned>(ceil_div(ntiles * 32, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      gray_code, sorted_idx, n, block, ntiles, tile_masks);
  return launch_status();
}

extern "C" int fgb_pp_valid_kernel(const uint32_t* tile_masks, int64_t nblk, int32_t* valid_kernel, int32_t* valid_kernel_seg,
                                   void* stream) {
  using namespace fgb;
  if (nblk < 0 || nblk > (int64_t(1) << 24)) return FGB_E_SIZE;
  if (!valid_kernel_seg) return FGB_E_NULL;
  if (nblk > 0 && (!tile_masks || !valid_kernel)) return FGB_E_NULL;
  valid_kernel_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(tile_masks, static_cast<uint32_t>(nblk), valid_kernel,
                                                                         valid_kernel_seg);
  return launch_status();
}
