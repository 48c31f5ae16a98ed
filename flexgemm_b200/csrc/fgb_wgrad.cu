// Split-K weight gradient of the submanifold conv on sm_100a, plus the bias
// gradient and the fp32 -> dtype cast used after an all-reduce.
//
//   gW[co, v, ci] = sum_{p in segment v} gout[o_p, co] * x[i_p, ci]
//
// For one offset v this is a GEMM whose reduction runs over the pair list of
// the offset, and both operands are row gathers: shared-memory rows are pairs
// (the K index) holding 128 bytes of channels, i.e. both operands are MN-major
// for tcgen05.mma.  A CTA owns (offset, split, group of up to 256 output
// channels, tile of up to 256 input channels); its accumulators (one or two
// 128-row blocks) fill up to all 512 TMEM columns.  The pair range of an
// offset is cut into `splitk` parts; each CTA writes an fp32 partial slab and
// a second kernel adds the slabs in a fixed order.
//
// Warp roles (192 threads): warps 0-3 gather (cp.async 16 B, pair indices
// double-buffered in shared memory) and run the epilogue, warp 5 lane 0 issues
// the MMAs; warp 4 is idle (kept so the role layout matches the fprop kernel).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "fgb_common.cuh"
#include "fgb_umma.cuh"

namespace fgb {

constexpr int kWgThreads = 192;
constexpr int kWgMaxStages = 8;

struct WgradParams {
  const char* gout;  // [n, Co]
  const char* x;     // [n, Ci]
  const uint32_t* vs_i;
  const uint32_t* vs_o;
  const uint32_t* seg;  // [V + 1]
  float* partial;       // [splitk, Co, V, Ci]
  int Co, Ci, V;
  int splitk;
  int mt;         // 128-row accumulator blocks per CTA (1 or 2)
  int bn;         // input channels per CTA
  int co_groups;  // ceil(Co / (mt * 128))
  int ci_tiles;   // ceil(Ci / bn)
  int kb;         // pairs per stage
  int stages;
  int a_chunks;   // 128-byte column chunks of the A stage (mt * 128 * elem / 128)
  int b_chunks;
  uint32_t idesc;
  uint32_t tmem_cols;
  int order;  // CTA order: 0 = offset-major, 1 = split-major
  int32_t* status;
};

struct WgradSmem {
  uint64_t full[kWgMaxStages];
  uint64_t empty[kWgMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t pad[28];
  uint32_t idx[2][2][64];  // [buffer][0 = output rows (A), 1 = input rows (B)][pair]
};
static_assert(sizeof(WgradSmem) <= 2048, "control block too large");

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int kElem>
__global__ void __launch_bounds__(kWgThreads, 1) subm_wgrad_kernel(const WgradParams p) {
  constexpr bool kTF32 = (kElem == 4);
  constexpr int kUmmaK = 32 / kElem;      // 16 for 16-bit types, 8 for tf32
  constexpr int kChunkElems = 128 / kElem;
  // MN-major operands: 16-bit types use the plain 128-byte swizzle (8-row K groups, 1024 B apart);
  // tf32 needs the 32-byte-based variant (4-row K groups, 512 B apart)
  constexpr uint32_t kLayout = kElem == 2 ? kSwizzle128B : kSwizzle128B32;
  constexpr uint32_t kSbo = kElem == 2 ? 1024 : 512;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  WgradSmem* ctl = reinterpret_cast<WgradSmem*>(smem);
  uint8_t* stages = smem + 2048;
  const int chunk_bytes = p.kb * 128;
  const int a_bytes = p.a_chunks * chunk_bytes;
  const int stage_bytes = (p.a_chunks + p.b_chunks) * chunk_bytes;

  // A kernel that already reported a soft error makes the rest of the grid a
  // no-op.  One thread reads the word so that the whole CTA takes the same branch.
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = p.status != nullptr && *reinterpret_cast<volatile const int32_t*>(p.status) != 0;
  __syncthreads();
  if (s_skip) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // work item
  // Split-major order: CTAs that run at the same time work on the same slice of
  // the pair lists of all offsets.  The lists are sorted by output row and a
  // neighbour's row is close to its voxel's row, so the slice touches a narrow
  // band of rows of both gathered matrices and that band stays in L2.
  uint32_t bid = blockIdx.x;
  const int ci_tile = bid % p.ci_tiles;
  bid /= p.ci_tiles;
  const int co_group = bid % p.co_groups;
  bid /= p.co_groups;
  int v, split;
  if (p.order == 1) {
    v = bid % p.V;
    split = bid / p.V;
  } else {
    split = bid % p.splitk;
    v = bid / p.splitk;
  }
  const int co0 = co_group * p.mt * 128;
  const int ci0 = ci_tile * p.bn;

  const uint32_t seg_begin = __ldg(&p.seg[v]);
  const uint32_t seg_len = __ldg(&p.seg[v + 1]) - seg_begin;
  const uint32_t num_k = (seg_len + p.kb - 1) / p.kb;
  const uint32_t k_begin = static_cast<uint32_t>((uint64_t(num_k) * split + p.splitk - 1) / p.splitk);
  const uint32_t k_end = static_cast<uint32_t>((uint64_t(num_k) * (split + 1) + p.splitk - 1) / p.splitk);
  const int total = static_cast<int>(k_end - k_begin);
  const uint32_t seg_end = seg_begin + seg_len;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->full[s], 128);  // every gather thread, on completion of its copies
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->acc_full, 1);
    ctl->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc_dyn(&ctl->tmem_base, p.tmem_cols);
    tmem_relinquish();
  }
  // pair indices of the first stage
  if (tid < 128 && total > 0) {
    const int which = tid >> 6, j = tid & 63;
    if (j < p.kb) {
      const uint32_t pp = seg_begin + k_begin * p.kb + j;
      ctl->idx[0][which][j] = pp < seg_end ? __ldg(which ? &p.vs_i[pp] : &p.vs_o[pp]) : kInvalid;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < 4) {
    // ---------------------------------------------------------------- gather
    const int piece = lane & 7, sub = lane >> 3;
    const int nchunks = p.a_chunks + p.b_chunks;
    const int units = p.kb * nchunks;  // (pair row, 128-byte chunk) units per stage, 4 per warp instruction
    const int a_row_bytes = p.Co * kElem, b_row_bytes = p.Ci * kElem;
    for (int it = 0; it < total; ++it) {
      const int s = it % p.stages;
      const int buf = it & 1;
      // prefetch the next stage's pair indices into a register
      uint32_t next_idx = kInvalid;
      const int which = tid >> 6, j = tid & 63;
      if (it + 1 < total && j < p.kb) {
        const uint32_t pp = seg_begin + (k_begin + it + 1) * p.kb + j;
        if (pp < seg_end) next_idx = __ldg(which ? &p.vs_i[pp] : &p.vs_o[pp]);
      }
      mbar_wait(&ctl->empty[s], ((it / p.stages) & 1) ^ 1, abort_flag);
      const uint32_t st_base = smem_u32(stages + size_t(s) * stage_bytes);
      for (int u = warp * 4 + sub; u < units; u += 16) {
        const int row = u / nchunks, chunk = u - row * nchunks;
        const bool is_b = chunk >= p.a_chunks;
        const int c = is_b ? chunk - p.a_chunks : chunk;
        const uint32_t gidx = ctl->idx[buf][is_b ? 1 : 0][row];
        const int col_bytes = (is_b ? ci0 * kElem : co0 * kElem) + c * 128 + piece * 16;
        const bool ok = gidx != kInvalid && col_bytes < (is_b ? b_row_bytes : a_row_bytes);
        const char* base = is_b ? p.x : p.gout;
        const char* src = ok ? base + size_t(gidx) * (is_b ? b_row_bytes : a_row_bytes) + col_bytes : base;
        // 16-bit types: 16-byte pieces swizzled by (row & 7); tf32: 32-byte pieces swizzled by (row & 3)
        const int swz = kElem == 2 ? ((piece ^ (row & 7)) << 4) : (((((piece >> 1) ^ (row & 3)) << 1) | (piece & 1)) << 4);
        const uint32_t dst = st_base + (is_b ? a_bytes : 0) + c * chunk_bytes + row * 128 + swz;
        cp_async_16(dst, src, ok ? 16u : 0u);
      }
      cp_async_arrive(&ctl->full[s]);
      if (j < p.kb) ctl->idx[buf ^ 1][which][j] = next_idx;
      named_barrier_sync(1, 128);
    }

    // -------------------------------------------------------------- epilogue
    if (total > 0) mbar_wait(&ctl->acc_full, 0, abort_flag);
    tc_fence_after_sync();
    for (int mt = 0; mt < p.mt; ++mt) {
      const int co = co0 + mt * 128 + warp * 32 + lane;
      float* orow = p.partial + ((size_t(split) * p.Co + co) * p.V + v) * p.Ci;
      for (int c0 = 0; c0 < p.bn; c0 += 32) {
        uint32_t acc[32];
        if (total > 0) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + mt * p.bn + c0, acc);
          tmem_ld_wait();
        }
        if (co < p.Co) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int ci = ci0 + c0 + g * 4;
            if (ci < p.Ci) {
              float4 o = total > 0 ? make_float4(__uint_as_float(acc[g * 4]), __uint_as_float(acc[g * 4 + 1]),
                                                 __uint_as_float(acc[g * 4 + 2]), __uint_as_float(acc[g * 4 + 3]))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
              *reinterpret_cast<float4*>(orow + ci) = o;
            }
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------- MMA
    if (lane == 0) {
      uint32_t accumulate = 0;
      for (int it = 0; it < total; ++it) {
        const int s = it % p.stages;
        mbar_wait(&ctl->full[s], (it / p.stages) & 1, abort_flag);
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(stages + size_t(s) * stage_bytes);
        const uint32_t b_addr = a_addr + a_bytes;
        const int chunks_per_m = 128 / kChunkElems;  // 128-byte chunks per 128 accumulator rows
        for (int ks = 0; ks < p.kb / kUmmaK; ++ks) {
          const uint32_t koff = ks * kUmmaK * 128;  // kUmmaK pair rows of 128 bytes
          const uint64_t db = make_smem_desc(b_addr + koff, chunk_bytes, kSbo, kLayout);
          for (int mt = 0; mt < p.mt; ++mt) {
            const uint64_t da = make_smem_desc(a_addr + mt * chunks_per_m * chunk_bytes + koff, chunk_bytes, kSbo, kLayout);
            umma_ss<kTF32>(tmem_base + mt * p.bn, da, db, p.idesc, accumulate);
          }
          accumulate = 1;
        }
        umma_commit(&ctl->empty[s]);
      }
      if (total > 0) umma_commit(&ctl->acc_full);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (tid == 0 && ctl->abort_flag) report(p.status, FGB_S_WAIT_TIMEOUT);
}

// out[e] = sum_s partial[s][e], written as dtype and/or fp32
template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int splitk, int64_t count,
                                                            T* __restrict__ out, float* __restrict__ out_f32) {
  const int64_t i = (blockIdx.x * int64_t(256) + threadIdx.x) * 4;
  if (i >= count) return;
  float4 acc = __ldg(reinterpret_cast<const float4*>(partial + i));
  for (int s = 1; s < splitk; ++s) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(partial + int64_t(s) * count + i));
    acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
  }
  if (out_f32) *reinterpret_cast<float4*>(out_f32 + i) = acc;
  if (out) {
    if constexpr (std::is_same<T, float>::value) {
      *reinterpret_cast<float4*>(out + i) = acc;
    } else {
      T o[4] = {static_cast<T>(acc.x), static_cast<T>(acc.y), static_cast<T>(acc.z), static_cast<T>(acc.w)};
      *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<uint2*>(o);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t count) {
  const int64_t i = blockIdx.x * int64_t(256) + threadIdx.x;
  if (i < count) dst[i] = static_cast<T>(src[i]);
}

// ------------------------------------------------------------------ bias gradient
constexpr int kBiasBlocks = 592;  // 4 per SM on a 148-SM part
// partial[b, c] = sum of column c over the rows of block b.  When the row is a
// whole number of 16-byte vectors, a thread owns one vector column and every
// (256 / vectors-per-row)-th row of the block, and the row groups are added up
// through shared memory; otherwise one thread per column walks the rows.
template <typename T>
__global__ void __launch_bounds__(256) bias_partial_kernel(const T* __restrict__ g, int64_t n, int Co, float* __restrict__ partial) {
  constexpr int kVec = 16 / sizeof(T);
  __shared__ float s_acc[256 * kVec];
  const int64_t rows_per = (n + gridDim.x - 1) / gridDim.x;
  const int64_t r0 = blockIdx.x * rows_per, r1 = min(n, r0 + rows_per);
  const int ncg = Co / kVec;
  if (Co % kVec == 0 && ncg <= 256 && 256 % ncg == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0) {
    const int cg = threadIdx.x % ncg, rg = threadIdx.x / ncg, nrg = 256 / ncg;
    float acc[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] = 0.f;
    for (int64_t r = r0 + rg; r < r1; r += nrg) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(g + r * Co) + cg);
      const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
      for (int i = 0; i < kVec; ++i) acc[i] += static_cast<float>(e[i]);
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) s_acc[threadIdx.x * kVec + i] = acc[i];
    __syncthreads();
    for (int c = threadIdx.x; c < Co; c += 256) {
      float sum = 0.f;
      for (int k = 0; k < nrg; ++k) sum += s_acc[(k * ncg + c / kVec) * kVec + c % kVec];  // fixed order
      partial[size_t(blockIdx.x) * Co + c] = sum;
    }
  } else {
    for (int c = threadIdx.x; c < Co; c += 256) {
      float acc = 0.f;
      for (int64_t r = r0; r < r1; ++r) acc += static_cast<float>(g[r * Co + c]);
      partial[size_t(blockIdx.x) * Co + c] = acc;
    }
  }
}
// out[c] = sum_b partial[b, c]: 32 columns per CTA, 8 row groups added up in a fixed order
template <typename T>
__global__ void __launch_bounds__(256) bias_final_kernel(const float* __restrict__ partial, int nblk, int Co, T* __restrict__ out,
                                                         float* __restrict__ out_f32) {
  __shared__ float s_acc[8][32];
  const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (c < Co)
    for (int b = rg; b < nblk; b += 8) acc += partial[size_t(b) * Co + c];
  s_acc[rg][lane] = acc;
  __syncthreads();
  if (rg == 0 && c < Co) {
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += s_acc[k][lane];
    if (out_f32) out_f32[c] = sum;
    if (out) out[c] = static_cast<T>(sum);
  }
}

static int pick_bn(int c) {
  int bn = 32;
  while (bn < c && bn < 256) bn <<= 1;
  return bn;
}

struct WgradPlan {
  int mt, bn, co_groups, ci_tiles, kb, stages, a_chunks, b_chunks;
  uint32_t tmem_cols;
  size_t smem;
};

static WgradPlan plan_wgrad(int Ci, int Co, int eb) {
  WgradPlan w;
  w.bn = pick_bn(Ci);
  w.mt = (Co > 128 && w.bn * 2 <= 512) ? 2 : 1;
  w.co_groups = static_cast<int>(ceil_div(Co, w.mt * 128));
  w.ci_tiles = static_cast<int>(ceil_div(Ci, w.bn));
  w.kb = eb == 2 ? 64 : 32;
  w.a_chunks = w.mt * 128 * eb / 128;
  w.b_chunks = static_cast<int>(ceil_div(w.bn * eb, 128));
  const size_t stage = size_t(w.a_chunks + w.b_chunks) * w.kb * 128;
  const size_t budget = 200 * 1024;
  w.stages = static_cast<int>(budget / stage);
  if (w.stages > kWgMaxStages) w.stages = kWgMaxStages;
  if (w.stages < 2) w.stages = 2;
  uint32_t cols = 32;
  while (cols < uint32_t(w.mt * w.bn)) cols <<= 1;
  w.tmem_cols = cols;
  w.smem = 1024 + 2048 + stage * w.stages;
  return w;
}

}  // namespace fgb

extern "C" int fgb_wgrad_default_splitk(int64_t n_pairs, int Ci, int Co, int V, int dtype) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  const WgradPlan w = plan_wgrad(Ci, Co, eb);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t base = int64_t(V) * w.co_groups * w.ci_tiles;
  int64_t s = ceil_div(int64_t(3) * sms, base);
  // no more splits than stages of pairs per offset on average
  const int64_t max_s = n_pairs > 0 ? ceil_div(ceil_div(n_pairs, V), w.kb) : 1;
  if (s > max_s) s = max_s;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  return static_cast<int>(s);
}

extern "C" int64_t fgb_conv_workspace_bytes(int pass, int Ci, int Co, int V, int dtype, int splitk) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  const int64_t w_elems = int64_t(Ci) * V * Co;
  switch (pass) {
    case 0:
      return 0;
    case 1:
      return w_elems * eb;
    case 2:
      if (splitk < 1 || splitk > 1024) return FGB_E_SIZE;
      return w_elems * 4 * splitk;
    default:
      return FGB_E_SIZE;
  }
}

extern "C" int fgb_subm_conv_wgrad(const void* grad_out, const void* feats, const uint32_t* valid_signal_i,
                                   const uint32_t* valid_signal_o, const uint32_t* valid_signal_seg, void* grad_weight,
                                   float* grad_weight_f32, int64_t n, int Ci, int Co, int V, int dtype, int splitk,
                                   void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0 || dtype == FGB_F32_IEEE) return FGB_E_DTYPE;
  if (n < 0 || Ci <= 0 || Co <= 0 || V < 1 || V > 32 || splitk < 1 || splitk > 1024) return FGB_E_SIZE;
  if ((Ci * eb) % 16 || (Co * eb) % 16) return FGB_E_ALIGN;
  if (!valid_signal_seg || !workspace) return FGB_E_NULL;
  if (n > 0 && (!grad_out || !feats || !valid_signal_i || !valid_signal_o)) return FGB_E_NULL;
  if ((reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(feats) | reinterpret_cast<uintptr_t>(workspace) |
       reinterpret_cast<uintptr_t>(grad_weight) | reinterpret_cast<uintptr_t>(grad_weight_f32)) & 15)
    return FGB_E_ALIGN;
  const int64_t count = int64_t(Co) * V * Ci;
  if (workspace_bytes < count * 4 * splitk) return FGB_E_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const WgradPlan w = plan_wgrad(Ci, Co, eb);
  WgradParams p;
  p.gout = static_cast<const char*>(grad_out);
  p.x = static_cast<const char*>(feats);
  p.vs_i = valid_signal_i;
  p.vs_o = valid_signal_o;
  p.seg = valid_signal_seg;
  p.partial = static_cast<float*>(workspace);
  p.Co = Co, p.Ci = Ci, p.V = V, p.splitk = splitk;
  p.mt = w.mt, p.bn = w.bn, p.co_groups = w.co_groups, p.ci_tiles = w.ci_tiles;
  p.kb = w.kb, p.stages = w.stages, p.a_chunks = w.a_chunks, p.b_chunks = w.b_chunks;
  const uint32_t fmt = dtype == FGB_F16 ? kFmtF16 : dtype == FGB_BF16 ? kFmtBF16 : kFmtTF32;
  p.idesc = make_idesc(fmt, 128, w.bn, 1, 1);
  p.tmem_cols = w.tmem_cols;
  {
    const char* e = getenv("FGB_WGRAD_ORDER");
    p.order = e ? atoi(e) : 0;
  }
  p.status = status;
  const int64_t grid = int64_t(V) * splitk * w.co_groups * w.ci_tiles;
  cudaError_t e;
  if (eb == 2) {
    e = cudaFuncSetAttribute(subm_wgrad_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(w.smem));
    if (e != cudaSuccess) return cuda_status(e);
    subm_wgrad_kernel<2><<<static_cast<unsigned>(grid), kWgThreads, w.smem, s>>>(p);
  } else {
    e = cudaFuncSetAttribute(subm_wgrad_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(w.smem));
    if (e != cudaSuccess) return cuda_status(e);
    subm_wgrad_kernel<4><<<static_cast<unsigned>(grid), kWgThreads, w.smem, s>>>(p);
  }
  int rc = launch_status();
  if (rc != FGB_OK) return rc;
  const unsigned rblocks = static_cast<unsigned>(ceil_div(count, 1024));
  switch (dtype) {
    case FGB_F16:
      splitk_reduce_kernel<__half><<<rblocks, 256, 0, s>>>(p.partial, splitk, count, static_cast<__half*>(grad_weight), grad_weight_f32);
      break;
    case FGB_BF16:
      splitk_reduce_kernel<__nv_bfloat16><<<rblocks, 256, 0, s>>>(p.partial, splitk, count, static_cast<__nv_bfloat16*>(grad_weight), grad_weight_f32);
      break;
    default:
      splitk_reduce_kernel<float><<<rblocks, 256, 0, s>>>(p.partial, splitk, count, static_cast<float*>(grad_weight), grad_weight_f32);
  }
  return launch_status();
}

extern "C" int64_t fgb_bias_grad_workspace_bytes(int Co) { return Co <= 0 ? FGB_E_SIZE : int64_t(fgb::kBiasBlocks) * Co * 4; }

extern "C" int fgb_subm_conv_bias_grad(const void* grad_out, void* grad_bias, float* grad_bias_f32, int64_t n, int Co, int dtype,
                                       void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (n < 0 || Co <= 0) return FGB_E_SIZE;
  if (!workspace || (n > 0 && !grad_out)) return FGB_E_NULL;
  if (workspace_bytes < fgb_bias_grad_workspace_bytes(Co)) return FGB_E_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  const int nblk = static_cast<int>(n < kBiasBlocks ? (n > 0 ? n : 1) : kBiasBlocks);
  const unsigned fblocks = static_cast<unsigned>(ceil_div(Co, 32));
  switch (dtype) {
    case FGB_F16:
      bias_partial_kernel<__half><<<nblk, 256, 0, s>>>(static_cast<const __half*>(grad_out), n, Co, partial);
      bias_final_kernel<__half><<<fblocks, 256, 0, s>>>(partial, nblk, Co, static_cast<__half*>(grad_bias), grad_bias_f32);
      break;
    case FGB_BF16:
      bias_partial_kernel<__nv_bfloat16><<<nblk, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(grad_out), n, Co, partial);
      bias_final_kernel<__nv_bfloat16><<<fblocks, 256, 0, s>>>(partial, nblk, Co, static_cast<__nv_bfloat16*>(grad_bias), grad_bias_f32);
      break;
    default:
      bias_partial_kernel<float><<<nblk, 256, 0, s>>>(static_cast<const float*>(grad_out), n, Co, partial);
      bias_final_kernel<float><<<fblocks, 256, 0, s>>>(partial, nblk, Co, static_cast<float*>(grad_bias), grad_bias_f32);
  }
  return launch_status();
}

// ------------------------------------------------------------------ bias gradient without caller scratch
// Some callers may not allocate device memory at all: a host runtime that hands
// its plug-ins a fixed arena and forbids further allocations, or a service
// loop that cannot afford the device-wide synchronisation cudaMalloc implies.
// For them the partial sums of the bias gradient live in a buffer that is part
// of the library image itself.  Every GPU that loads the library carries these
// kBiasBlocks * kNoAllocMaxCo * 4 bytes (4.6 MiB) until the process exits.
constexpr int kNoAllocMaxCo = 2048;
static __device__ __align__(256) float g_bias_partials[size_t(fgb::kBiasBlocks) * kNoAllocMaxCo];

namespace {
// In host code `g_bias_partials` is only a handle for the runtime, not an
// address a kernel can use; the device address differs per GPU and is asked
// for once per device, with that device current.
int bias_partials_address(float** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float* addr[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fgb::cuda_status(e);
  if (dev < 0 || dev >= kMaxDevices) return FGB_E_SIZE;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_bias_partials);
    if (e != cudaSuccess) return fgb::cuda_status(e);
    if (p == nullptr) return FGB_E_DRIVER;
    addr[dev] = static_cast<float*>(p);
  }
  *out = addr[dev];
  return FGB_OK;
}
}  // namespace

extern "C" int fgb_noalloc_max_channels(void) { return kNoAllocMaxCo; }

extern "C" int fgb_subm_conv_bias_grad_noalloc(const void* grad_out, void* grad_bias, float* grad_bias_f32, int64_t n, int Co,
                                               int dtype, void* stream) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (n < 0 || Co <= 0) return FGB_E_SIZE;
  if (Co > kNoAllocMaxCo) return FGB_E_STATIC_LIMIT;
  if (n > 0 && !grad_out) return FGB_E_NULL;
  float* partial = nullptr;
  int rc = bias_partials_address(&partial);
  if (rc != FGB_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Nothing has to be cleared between calls: the first kernel overwrites every
  // partial sum that the second one reads (nblk rows of Co floats).
  const int nblk = static_cast<int>(n < kBiasBlocks ? (n > 0 ? n : 1) : kBiasBlocks);
  const unsigned fblocks = static_cast<unsigned>(ceil_div(Co, 32));
  switch (dtype) {
    case FGB_F16:
      bias_partial_kernel<__half><<<nblk, 256, 0, s>>>(static_cast<const __half*>(grad_out), n, Co, partial);
      bias_final_kernel<__half><<<fblocks, 256, 0, s>>>(partial, nblk, Co, static_cast<__half*>(grad_bias), grad_bias_f32);
      break;
    case FGB_BF16:
      bias_partial_kernel<__nv_bfloat16><<<nblk, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(grad_out), n, Co, partial);
      bias_final_kernel<__nv_bfloat16><<<fblocks, 256, 0, s>>>(partial, nblk, Co, static_cast<__nv_bfloat16*>(grad_bias), grad_bias_f32);
      break;
    default:
      bias_partial_kernel<float><<<nblk, 256, 0, s>>>(static_cast<const float*>(grad_out), n, Co, partial);
      bias_final_kernel<float><<<fblocks, 256, 0, s>>>(partial, nblk, Co, static_cast<float*>(grad_bias), grad_bias_f32);
  }
  return launch_status();
}

extern "C" int fgb_cast_from_f32(const float* src, void* dst, int64_t count, int dtype, void* stream) {
  using namespace fgb;
  if (count < 0) return FGB_E_SIZE;
  if (count == 0) return FGB_OK;
  if (!src || !dst) return FGB_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>(ceil_div(count, 256));
  switch (dtype) {
    case FGB_F16:
      cast_from_f32_kernel<__half><<<blocks, 256, 0, s>>>(src, static_cast<__half*>(dst), count);
      break;
    case FGB_BF16:
      cast_from_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(src, static_cast<__nv_bfloat16*>(dst), count);
      break;
    case FGB_F32_TF32:
    case FGB_F32_IEEE:
      cast_from_f32_kernel<float><<<blocks, 256, 0, s>>>(src, static_cast<float*>(dst), count);
      break;
    default:
      return FGB_E_DTYPE;
  }
  return launch_status();
}
