// Masked implicit GEMM for submanifold conv fprop and dgrad on sm_100a.
//
//   out[r, :] = bias + sum_{v in mask(tile(r))} x[nbr[r, v], :] . Wn[:, v, :]^T
//
// One CTA computes a tile of 128 sorted rows by BN output channels.  The
// accumulator lives in tensor memory; the reduction runs over the offsets set
// in the tile's mask times the 128-byte slices of the channel dimension.
//
// Warp roles (192 threads):
//   warps 0-3  gather the activation rows of the tile into a 128B-swizzled
//              K-major shared-memory stage with 16-byte cp.async (zero fill for
//              missing neighbours and past the channel count); each thread's
//              copies arrive on the stage's mbarrier when they land, so up to
//              all stages are in flight; afterwards the same warps
//              run the epilogue (tcgen05.ld -> +bias -> convert -> row store);
//   warp 4     one lane streams the dense weight tile [BN x 128 B] of the
//              current (offset, slice) with a tiled TMA load;
//   warp 5     owns the TMEM allocation; one lane issues tcgen05.mma and
//              commits stage releases to the mbarriers.
//
// dgrad is the same kernel: x = grad_out, the weight is first re-laid-out to
// [Ci, V, Co] and offset v reads weight slot V-1-v.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "fgb_common.cuh"
#include "fgb_umma.cuh"

namespace fgb {

constexpr int kTileM = 128;
constexpr int kStages = 4;
constexpr int kIgemmThreads = 192;
constexpr int kCtrlBytes = 1024;        // barriers, TMEM holder, abort flag, sorted rows
constexpr int kNbrTileBytes = kTileM * 32 * 4;
constexpr int kATileBytes = kTileM * 128;

struct IgemmParams {
  const char* x;             // [n, kc] gathered operand
  const void* bias;          // [nout] or null
  const uint32_t* nbr;       // [n, V]
  const int64_t* sorted_idx; // [n]
  const uint32_t* tile_masks;
  char* out;                 // [n, nout]
  uint32_t n;
  int kc;                    // reduction channels per offset
  int nout;                  // output channels
  int V;
  int bn;                    // output channels per CTA (32, 64, 128, 256)
  int n_tiles_n;
  int row_bytes;             // kc * element size
  int num_kb;                // 128-byte slices per row
  int flip;                  // weight slot = flip ? V-1-v : v
  int dtype;
  uint32_t idesc;
  int32_t* status;
};

struct IgemmSmem {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t pad[26];
  uint32_t srow[kTileM];  // original row of each tile row, kInvalid past the end
};
static_assert(sizeof(IgemmSmem) <= kCtrlBytes, "control block too large");

template <int kDtype>
__device__ __forceinline__ void store_row_chunk(char* dst, const uint32_t (&acc)[32], const void* bias, int col0, int nout,
                                                bool zero_acc) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = zero_acc ? 0.f : __uint_as_float(acc[i]);
  if constexpr (kDtype == FGB_F16 || kDtype == FGB_BF16) {
    using T = typename std::conditional<kDtype == FGB_F16, __half, __nv_bfloat16>::type;
#pragma unroll
    for (int g = 0; g < 4; ++g) {  // 8 columns = 16 bytes per store
      const int c = col0 + g * 8;
      if (c < nout) {
        if (bias != nullptr) {
          const uint4 bw = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(bias) + c));
          const T* bt = reinterpret_cast<const T*>(&bw);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[g * 8 + i] += static_cast<float>(bt[i]);
        }
        uint4 o;
        T* ot = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) ot[i] = static_cast<T>(v[g * 8 + i]);
        *reinterpret_cast<uint4*>(dst + size_t(c) * 2) = o;
      }
    }
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) {  // 4 columns = 16 bytes per store
      const int c = col0 + g * 4;
      if (c < nout) {
        float4 o = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
        if (bias != nullptr) {
          const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(bias) + c));
          o.x += b.x, o.y += b.y, o.z += b.z, o.w += b.w;
        }
        *reinterpret_cast<float4*>(dst + size_t(c) * 4) = o;
      }
    }
  }
}

template <int kDtype>
__global__ void __launch_bounds__(kIgemmThreads, 1)
    subm_igemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const IgemmParams p) {
  constexpr bool kTF32 = (kDtype == FGB_F32_TF32);
  constexpr int kElem = (kDtype == FGB_F16 || kDtype == FGB_BF16) ? 2 : 4;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: align by hand
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  IgemmSmem* ctl = reinterpret_cast<IgemmSmem*>(smem);
  uint32_t* s_nbr = reinterpret_cast<uint32_t*>(smem + kCtrlBytes);
  uint8_t* stages = smem + kCtrlBytes + kNbrTileBytes;
  const int stage_bytes = kATileBytes + p.bn * 128;

  // A kernel that already reported a soft error makes the rest of the grid a
  // no-op.  One thread reads the word so that the whole CTA takes the same branch.
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = p.status != nullptr && *reinterpret_cast<volatile const int32_t*>(p.status) != 0;
  __syncthreads();
  if (s_skip) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t n_tile = blockIdx.x % p.n_tiles_n;
  const uint32_t m_tile = blockIdx.x / p.n_tiles_n;
  const uint32_t m0 = m_tile * kTileM;
  const int n0 = n_tile * p.bn;
  const int V = p.V;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->full[s], 129);  // 128 gather threads (on completion of their copies) + the TMA lane's expect_tx arrive
      mbar_init(&ctl->empty[s], 1);  // one tcgen05.commit
    }
    mbar_init(&ctl->acc_full, 1);
    ctl->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 4 && lane == 0) tma_prefetch_desc(&tmap_w);
  if (warp == 5) {
    tmem_alloc_dyn(&ctl->tmem_base, static_cast<uint32_t>(p.bn));
    tmem_relinquish();
  }
  if (tid < kTileM) {
    const uint32_t r = m0 + tid;
    ctl->srow[tid] = r < p.n ? static_cast<uint32_t>(__ldg(&p.sorted_idx[r])) : kInvalid;
  }
  __syncthreads();
  for (int i = tid; i < kTileM * V; i += kIgemmThreads) {
    const int r = i / V, v = i - r * V;
    const uint32_t sr = ctl->srow[r];
    s_nbr[i] = sr != kInvalid ? __ldg(&p.nbr[size_t(sr) * V + v]) : kInvalid;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t mask = __ldg(&p.tile_masks[m_tile]);
  const int total = __popc(mask) * p.num_kb;

  if (warp < 4) {
    // ---------------------------------------------------------------- gather
    const int chunk = lane & 7;
    const int rsub = lane >> 3;
    int it = 0;
    uint32_t m = mask;
    while (m) {
      const int v = __ffs(m) - 1;
      m &= m - 1;
      // neighbour rows of this lane's 8 tile rows for offset v
      uint32_t idx[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) idx[j] = s_nbr[(warp * 32 + j * 4 + rsub) * V + v];
      for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
        const int s = it % kStages;
        mbar_wait(&ctl->empty[s], ((it / kStages) & 1) ^ 1, abort_flag);
        const uint32_t a_base = smem_u32(stages + size_t(s) * stage_bytes);
        const int col = kb * 128 + chunk * 16;
        const bool col_ok = col < p.row_bytes;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = warp * 32 + j * 4 + rsub;
          const bool ok = col_ok && idx[j] != kInvalid;
          const char* src = ok ? p.x + size_t(idx[j]) * p.row_bytes + col : p.x;
          cp_async_16(a_base + r * 128 + ((chunk ^ (r & 7)) << 4), src, ok ? 16u : 0u);
        }
        cp_async_arrive(&ctl->full[s]);
      }
    }

    // -------------------------------------------------------------- epilogue
    if (total > 0) mbar_wait(&ctl->acc_full, 0, abort_flag);
    tc_fence_after_sync();
    const uint32_t sr = ctl->srow[warp * 32 + lane];
    char* orow = p.out + size_t(sr) * p.nout * kElem;
    for (int c0 = 0; c0 < p.bn; c0 += 32) {
      uint32_t acc[32];
      if (total > 0) {
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c0, acc);
        tmem_ld_wait();
      }
      if (sr != kInvalid && n0 + c0 < p.nout) store_row_chunk<kDtype>(orow, acc, p.bias, n0 + c0, p.nout, total == 0);
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------ weight TMA
    if (lane == 0) {
      int it = 0;
      uint32_t m = mask;
      while (m) {
        const int v = __ffs(m) - 1;
        m &= m - 1;
        const int wv = p.flip ? V - 1 - v : v;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % kStages;
          mbar_wait(&ctl->empty[s], ((it / kStages) & 1) ^ 1, abort_flag);
          mbar_arrive_expect_tx(&ctl->full[s], static_cast<uint32_t>(p.bn) * 128u);
          tma_load_3d(smem_u32(stages + size_t(s) * stage_bytes + kATileBytes), &tmap_w, &ctl->full[s], kb * (128 / kElem), wv, n0);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------- MMA
    if (lane == 0) {
      uint32_t accumulate = 0;
      for (int it = 0; it < total; ++it) {
        const int s = it % kStages;
        const int kb = it % p.num_kb;
        mbar_wait(&ctl->full[s], (it / kStages) & 1, abort_flag);
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(stages + size_t(s) * stage_bytes);
        const uint64_t da = make_smem_desc(a_addr, 16, 1024);
        const uint64_t db = make_smem_desc(a_addr + kATileBytes, 16, 1024);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          if (kb * 128 + k4 * 32 < p.row_bytes) {
            umma_ss<kTF32>(tmem_base, da + uint64_t(k4 * 2), db + uint64_t(k4 * 2), p.idesc, accumulate);
            accumulate = 1;
          }
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
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.bn));
  }
  if (tid == 0 && ctl->abort_flag) report(p.status, FGB_S_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ weight re-layout for dgrad
// dst[ci, v, co] = src[co, v, ci]; 32x32 tiles through shared memory
template <typename T>
__global__ void __launch_bounds__(256) weight_transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int Co, int V, int Ci) {
  __shared__ T tile[32][33];
  const int v = blockIdx.z;
  const int ci0 = blockIdx.x * 32, co0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    const int co = co0 + j, ci = ci0 + tx;
    if (co < Co && ci < Ci) tile[j][tx] = src[(size_t(co) * V + v) * Ci + ci];
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int ci = ci0 + j, co = co0 + tx;
    if (co < Co && ci < Ci) dst[(size_t(ci) * V + v) * Co + co] = tile[tx][j];
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 3-D map over w[nout][V][kc]; box = 128 bytes of kc x 1 offset x bn rows, 128B swizzle
int make_weight_tmap(CUtensorMap* map, const void* w, int nout, int V, int kc, int bn, int dtype) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return FGB_E_DRIVER;
  const int eb = elem_bytes(dtype);
  const CUtensorMapDataType dt = dtype == FGB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : dtype == FGB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[3] = {cuuint64_t(kc), cuuint64_t(V), cuuint64_t(nout)};
  cuuint64_t strides[2] = {cuuint64_t(kc) * eb, cuuint64_t(V) * kc * eb};
  cuuint32_t box[3] = {cuuint32_t(128 / eb), 1u, cuuint32_t(bn)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FGB_OK : FGB_E_DRIVER;
}

static int pick_bn(int nout) {
  int bn = 32;
  while (bn < nout && bn < 256) bn <<= 1;
  return bn;
}

template <int kDtype>
static int launch_igemm(const CUtensorMap& tmap, const IgemmParams& p, cudaStream_t s) {
  const size_t smem = 1024 + kCtrlBytes + kNbrTileBytes + size_t(kStages) * (kATileBytes + p.bn * 128);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(subm_igemm_kernel<kDtype>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_status(e);
    configured = smem;
  }
  const int64_t m_tiles = ceil_div(p.n, kTileM);
  const int64_t grid = m_tiles * p.n_tiles_n;
  if (grid > 0x7FFFFFFF) return FGB_E_SIZE;
  subm_igemm_kernel<kDtype><<<static_cast<unsigned>(grid), kIgemmThreads, smem, s>>>(tmap, p);
  return launch_status();
}

// x [n, kc] gathered through nbr; w [nout, V, kc]; out [n, nout]
int run_igemm(const void* x, const void* w, const void* bias, const uint32_t* nbr, const int64_t* sorted_idx,
              const uint32_t* tile_masks, void* out, int64_t n, int kc, int nout, int V, int dtype, int flip, int32_t* status,
              cudaStream_t s) {
  const int eb = elem_bytes(dtype);
  if (eb == 0 || dtype == FGB_F32_IEEE) return FGB_E_DTYPE;
  if (n < 0 || n >= (int64_t(1) << 32) - 1 || kc <= 0 || nout <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!x || !w || !nbr || !sorted_idx || !tile_masks || !out) return FGB_E_NULL;
  if ((kc * eb) % 16 || (nout * eb) % 16) return FGB_E_ALIGN;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(bias)) & 15)
    return FGB_E_ALIGN;
  IgemmParams p;
  p.x = static_cast<const char*>(x);
  p.bias = bias;
  p.nbr = nbr;
  p.sorted_idx = sorted_idx;
  p.tile_masks = tile_masks;
  p.out = static_cast<char*>(out);
  p.n = static_cast<uint32_t>(n);
  p.kc = kc;
  p.nout = nout;
  p.V = V;
  p.bn = pick_bn(nout);
  p.n_tiles_n = static_cast<int>(ceil_div(nout, p.bn));
  p.row_bytes = kc * eb;
  p.num_kb = static_cast<int>(ceil_div(p.row_bytes, 128));
  p.flip = flip;
  p.dtype = dtype;
  const uint32_t fmt = dtype == FGB_F16 ? kFmtF16 : dtype == FGB_BF16 ? kFmtBF16 : kFmtTF32;
  p.idesc = make_idesc(fmt, kTileM, p.bn, 0, 0);
  p.status = status;
  CUtensorMap tmap;
  int rc = make_weight_tmap(&tmap, w, nout, V, kc, p.bn, dtype);
  if (rc != FGB_OK) return rc;
  switch (dtype) {
    case FGB_F16:
      return launch_igemm<FGB_F16>(tmap, p, s);
    case FGB_BF16:
      return launch_igemm<FGB_BF16>(tmap, p, s);
    default:
      return launch_igemm<FGB_F32_TF32>(tmap, p, s);
  }
}

}  // namespace fgb

extern "C" int fgb_conv_tile_rows(void) { return fgb::kTileM; }

extern "C" int fgb_subm_conv_fprop(const void* feats, const void* weight, const void* bias, const uint32_t* neighbor_map,
                                   const int64_t* sorted_idx, const uint32_t* tile_masks, void* out, int64_t n, int Ci, int Co,
                                   int V, int dtype, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  return fgb::run_igemm(feats, weight, bias, neighbor_map, sorted_idx, tile_masks, out, n, Ci, Co, V, dtype, 0, status,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int fgb_subm_conv_dgrad(const void* grad_out, const void* weight, const uint32_t* neighbor_map,
                                   const int64_t* sorted_idx, const uint32_t* tile_masks, void* grad_feats, int64_t n, int Ci,
                                   int Co, int V, int dtype, void* workspace, int64_t workspace_bytes, int32_t* status,
                                   void* stream) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!weight || !workspace) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FGB_E_ALIGN;
  if (workspace_bytes < int64_t(Ci) * V * Co * eb) return FGB_E_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>(ceil_div(Ci, 32)), static_cast<unsigned>(ceil_div(Co, 32)), V);
  if (eb == 2)
    weight_transpose_kernel<uint16_t><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(weight), static_cast<uint16_t*>(workspace), Co, V, Ci);
  else
    weight_transpose_kernel<uint32_t><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(weight), static_cast<uint32_t*>(workspace), Co, V, Ci);
  int rc = launch_status();
  if (rc != FGB_OK) return rc;
  return run_igemm(grad_out, workspace, nullptr, neighbor_map, sorted_idx, tile_masks, grad_feats, n, Co, Ci, V, dtype, 1, status, s);
}
