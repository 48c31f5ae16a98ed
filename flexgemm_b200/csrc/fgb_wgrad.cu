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
// 128-row blocks) fill up to all 512 TMEM columns.  The pair lists are cut into
// units of equal length (about `splitk` per offset on average, an offset with
// more pairs gets more units); each CTA writes an fp32 partial slab and a
// second kernel adds the slabs of an offset in a fixed order.
//
// Warp roles (416 threads): warps 0-3 epilogue (tcgen05.ld -> fp32 slab),
// warp 4 owns the TMEM allocation and lane 0 issues the MMAs, warps 5-12 gather
// both operands (cp.async 16 B, pair indices prefetched into registers one stage
// ahead, completion signalled per thread on the stage's mbarrier).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <type_traits>

#include "fgb_common.cuh"
#include "fgb_device.cuh"
#include "fgb_precision.cuh"
#include "fgb_umma.cuh"

namespace fgb {

constexpr int kWgThreads = 416;   // 4 epilogue warps, 1 MMA warp, 8 gather warps
constexpr int kWgGatherWarp0 = 5;
constexpr int kWgGatherThreads = 256;
constexpr int kWgMaxStages = 8;
constexpr int kWgRowsMax = 4;  // pair rows of a stage per gather thread: stages hold up to 128 pairs
constexpr int kWgMaxBands = 64;

struct WgradParams {
  const char* gout;  // [n, Co]
  const char* x;     // [n, Ci]
  const uint32_t* vs_i;
  const uint32_t* vs_o;
  const uint32_t* seg;  // [V + 1]
  const uint32_t* block_offsets;  // [V, nblk]: pairs of offset v in the 256-row map blocks before block k; null = one band
  uint32_t nblk;        // 256-row map blocks of the output rows
  uint32_t band_blocks; // map blocks per row band
  int bands;            // row bands (1 .. kWgMaxBands)
  float* partial;       // [units, Co, Ci] slabs
  int Co, Ci, V;
  int target_units;  // the kernel cuts the pair lists into at most this many units (see wg_plan_unit_kb)
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
  int order;      // unit enumeration: 0 = offset-major, 1 = chunk-major
  int32_t* status;
};

struct WgradSmem {
  uint64_t full[kWgMaxStages];
  uint64_t empty[kWgMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  uint32_t abort_flag;
  int unit_v, unit_j;  // the unit this CTA works on (offset, chunk index), -1 if none
  int unit_kb;         // k-blocks per unit, planned from the segment table
  int total;           // k-blocks (stages) of this CTA over all bands
  // this CTA's share of each row band: first pair, k-blocks, and the band's end in the pair list
  uint32_t band_begin[kWgMaxBands], band_cnt[kWgMaxBands], band_end[kWgMaxBands];
};
static_assert(sizeof(WgradSmem) <= 1024, "control block too large");

// k-blocks per unit: the smallest length for which the offsets' pair lists (nk_v k-blocks each) make at most `target`
// units, sum_v ceil(nk_v / unit_kb) <= target.  The host knows only the total pair count; planning from the segment
// table itself lets the grid be exactly the number of CTAs that run together (one wave, or a whole number of waves)
// instead of a worst-case bound whose overshoot would run as a short extra wave.  Called by all 32 lanes of a warp
// (lane v looks at offset v); every CTA and the reduction compute the same value from the same table.
__device__ __forceinline__ uint32_t wg_plan_unit_kb(const uint32_t* seg, int V, int kb, uint32_t target, int lane) {
  uint32_t nk = 0;
  if (lane < V) nk = (__ldg(&seg[lane + 1]) - __ldg(&seg[lane]) + kb - 1) / kb;
  uint32_t lo = 1, hi = __reduce_max_sync(0xffffffffu, nk);
  if (hi < 1u) hi = 1u;
  while (lo < hi) {  // sum of ceilings does not increase with the unit length; at hi every non-empty offset is one unit
    const uint32_t mid = lo + ((hi - lo) >> 1);
    const uint32_t units = __reduce_add_sync(0xffffffffu, (nk + mid - 1) / mid);
    if (units <= target) hi = mid;
    else lo = mid + 1;
  }
  return lo;
}

// Units: offset v is cut into ceil(nk_v / unit_kb) chunks of unit_kb k-blocks
// (nk_v = k-blocks of the offset's pair list).  Unit ids enumerate (v, chunk)
// either offset-major or chunk-major.  Returns false when `u` is past the end.
__device__ __forceinline__ uint32_t wg_chunks_of(const uint32_t* seg, int v, int kb, int unit_kb) {
  const uint32_t len = __ldg(&seg[v + 1]) - __ldg(&seg[v]);
  const uint32_t nk = (len + kb - 1) / kb;
  return (nk + unit_kb - 1) / unit_kb;
}
__device__ bool wg_find_unit(const uint32_t* seg, int V, int kb, int unit_kb, int order, uint32_t u, int* v_out, int* j_out) {
  if (order == 0) {
    for (int v = 0; v < V; ++v) {
      const uint32_t c = wg_chunks_of(seg, v, kb, unit_kb);
      if (u < c) {
        *v_out = v, *j_out = static_cast<int>(u);
        return true;
      }
      u -= c;
    }
    return false;
  }
  for (uint32_t j = 0;; ++j) {
    uint32_t alive = 0;
    for (int v = 0; v < V; ++v) {
      if (wg_chunks_of(seg, v, kb, unit_kb) > j) {
        if (u == alive) {
          *v_out = v, *j_out = static_cast<int>(j);
          return true;
        }
        ++alive;
      }
    }
    if (alive == 0) return false;
    u -= alive;
  }
}
// slab index of unit (v, j): units are stored offset-major whatever the launch order
__device__ __forceinline__ uint32_t wg_slab_of(const uint32_t* seg, int kb, int unit_kb, int v, int j) {
  uint32_t base = 0;
  for (int t = 0; t < v; ++t) base += wg_chunks_of(seg, t, kb, unit_kb);
  return base + j;
}

// ------------------------------------------------------------------ row bands
// The pair list of an offset is in ascending output-row order, and the input row of a pair lies near its output
// row.  Cutting EVERY offset's list at the same output rows (bands of `band_blocks` 256-row map blocks) and letting
// every CTA of an offset take its share of every band, band after band, makes all CTAs of the launch read the same
// band of rows of both matrices at the same time: the band is fetched from HBM once and the other offsets find it
// in L2.  (With each CTA walking one contiguous piece of one list, the 148 CTAs are spread over the whole row range
// at any moment and every offset streams both matrices from HBM again.)
//
// Position in the pair list where band b of offset v starts; b == bands gives the end of the list.
__host__ __device__ __forceinline__ uint32_t wg_band_pos(const uint32_t* seg, const uint32_t* block_offsets, uint32_t nblk,
                                                         uint32_t band_blocks, int bands, int v, int b) {
  if (b <= 0) return seg[v];
  const uint64_t blk = uint64_t(b) * band_blocks;
  if (b >= bands || blk >= nblk || block_offsets == nullptr) return seg[v + 1];
  return seg[v] + block_offsets[size_t(v) * nblk + blk];
}
// Share of CTA `k` (of K for the offset) in a band of `nkb` k-blocks.  The K CTAs get nkb / K blocks each and the
// remainder goes to nkb % K of them, dealt round-robin from where the previous bands stopped (`rot` = sum of the
// earlier bands' remainders), so that over all bands the CTAs' totals differ by at most one block.
// Returns the count; *first = index of the CTA's first block within the band.
__host__ __device__ __forceinline__ uint32_t wg_band_share(uint32_t nkb, uint32_t K, uint32_t k, uint32_t rot, uint32_t* first) {
  const uint32_t base = nkb / K, rem = nkb - base * K;
  const uint32_t q = (k + K - rot % K) % K;  // position of this CTA in the band's dealing order
  *first = q * base + (q < rem ? q : rem);
  return base + (q < rem ? 1u : 0u);
}

// kRows = pairs of a stage / 32 = pair rows per gather thread.  kBanded: the CTA walks its share of every row band (see
// above); otherwise one contiguous run of k-blocks of its offset's list, without the per-band tables in the gather loop
// (that loop's bookkeeping alone costs 2-3 % where bands bring nothing).
template <int kElem, int kRows, bool kBanded>
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
  uint8_t* stages = smem + 1024;
  chain_release();  // the ordered sum that follows is launched chained: its CTAs plan their slabs while this kernel runs
  const int chunk_bytes = p.kb * 128;
  const int a_bytes = p.a_chunks * chunk_bytes;
  const int stage_bytes = (p.a_chunks + p.b_chunks) * chunk_bytes;
  const int S = p.stages;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // work item: (unit, output-channel group, input-channel tile)
  uint32_t bid = blockIdx.x;
  const int ci_tile = bid % p.ci_tiles;
  bid /= p.ci_tiles;
  const int co_group = bid % p.co_groups;
  bid /= p.co_groups;
  if (warp == 0) {
    const uint32_t ukb = wg_plan_unit_kb(p.seg, p.V, p.kb, static_cast<uint32_t>(p.target_units), lane);
    int v = -1, j = -1;
    if (lane == 0) {
      const bool skip = p.status != nullptr && *reinterpret_cast<volatile const int32_t*>(p.status) != 0;
      if (skip || !wg_find_unit(p.seg, p.V, p.kb, static_cast<int>(ukb), p.order, bid, &v, &j)) v = j = -1;
      ctl->unit_v = v, ctl->unit_j = j, ctl->unit_kb = static_cast<int>(ukb);
    }
    v = __shfl_sync(0xffffffffu, v, 0), j = __shfl_sync(0xffffffffu, j, 0);
    if (kBanded && v >= 0) {
      // this CTA's share of every row band (lane b looks at band b, 32 bands per round)
      const uint32_t K = wg_chunks_of(p.seg, v, p.kb, static_cast<int>(ukb));
      uint32_t rot = 0, total = 0;
      for (int b0 = 0; b0 < p.bands; b0 += 32) {
        const int b = b0 + lane;
        uint32_t begin = 0, end = 0, nkb = 0;
        if (b < p.bands) {
          begin = wg_band_pos(p.seg, p.block_offsets, p.nblk, p.band_blocks, p.bands, v, b);
          end = wg_band_pos(p.seg, p.block_offsets, p.nblk, p.band_blocks, p.bands, v, b + 1);
          nkb = (end - begin + p.kb - 1) / p.kb;
        }
        // exclusive prefix of the remainders over the bands before this one
        const uint32_t rem = nkb % K;
        uint32_t inc = rem;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const uint32_t y = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += y;
        }
        uint32_t first = 0;
        const uint32_t cnt = wg_band_share(nkb, K, static_cast<uint32_t>(j), rot + inc - rem, &first);
        if (b < p.bands) {
          ctl->band_begin[b] = begin + first * p.kb;
          ctl->band_cnt[b] = cnt;
          ctl->band_end[b] = end;
        }
        total += __reduce_add_sync(0xffffffffu, cnt);
        rot += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) ctl->total = static_cast<int>(total);
    }
  }
  __syncthreads();
  const int v = ctl->unit_v, unit_j = ctl->unit_j, unit_kb = ctl->unit_kb;
  if (v < 0) return;  // grid is sized for the worst case; also the no-op path after a soft error
  const int co0 = co_group * p.mt * 128;
  const int ci0 = ci_tile * p.bn;
  // contiguous walk: k-blocks [k_begin, k_begin + total) of the offset's list, full units and a shorter last one
  const uint32_t seg_begin = __ldg(&p.seg[v]);
  const uint32_t seg_end = __ldg(&p.seg[v + 1]);
  const uint32_t num_k = (seg_end - seg_begin + p.kb - 1) / p.kb;
  const uint32_t k_begin = static_cast<uint32_t>(unit_j) * unit_kb;
  // banded: may be 0 for a CTA of a very short offset, which then writes a slab of zeros
  const int total = kBanded ? ctl->total : static_cast<int>(min(num_k, k_begin + unit_kb) - k_begin);
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&ctl->full[s], kWgGatherThreads);  // every gather thread, on completion of its copies
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->acc_full, 1);
    ctl->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 4) {
    tmem_alloc_dyn(&ctl->tmem_base, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp >= kWgGatherWarp0) {
    // ---------------------------------------------------------------- gather
    // Eight lanes move one 128-byte chunk of one pair row; a thread owns rows
    // g, g+32, ... of every stage and walks over the chunks of both operands.
    const int piece = lane & 7;
    const int g = (warp - kWgGatherWarp0) * 4 + (lane >> 3);  // 0..31
    const int a_row_bytes = p.Co * kElem, b_row_bytes = p.Ci * kElem;
    uint32_t row_off[kRows];
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const int row = g + 32 * j;
      // 16-bit types: 16-byte pieces swizzled by (row & 7); tf32: 32-byte pieces swizzled by (row & 3)
      const int swz = kElem == 2 ? ((piece ^ (row & 7)) << 4) : (((((piece >> 1) ^ (row & 3)) << 1) | (piece & 1)) << 4);
      row_off[j] = row * 128 + swz;
    }
    // walks the CTA's k-blocks band by band: (band, block within the CTA's share of the band)
    int band = 0;
    uint32_t blk = 0;
    auto skip_empty = [&]() {
      while (band < p.bands && blk >= ctl->band_cnt[band]) ++band, blk = 0;
    };
    uint32_t next_kblk = k_begin;  // contiguous walk: the next k-block of the list
    auto load_pairs = [&](uint32_t (&io)[kRows], uint32_t (&ii)[kRows]) {  // pairs of the next block, then advance
      uint32_t first, end;
      if constexpr (kBanded) {
        first = ctl->band_begin[band] + blk * p.kb, end = ctl->band_end[band];
      } else {
        first = seg_begin + next_kblk * p.kb, end = seg_end;
      }
#pragma unroll
      for (int j = 0; j < kRows; ++j) {
        const uint32_t pp = first + g + 32 * j;
        const bool ok = pp < end;
        io[j] = ok ? __ldg(&p.vs_o[pp]) : kInvalid;
        ii[j] = ok ? __ldg(&p.vs_i[pp]) : kInvalid;
      }
      if constexpr (kBanded) {
        ++blk;
        skip_empty();
      } else {
        ++next_kblk;
      }
    };
    uint32_t io[kRows], ii[kRows], nio[kRows], nii[kRows];
    if constexpr (kBanded) skip_empty();
    if (total > 0) load_pairs(nio, nii);
    int s = 0;
    uint32_t ph = 0;  // ring position and phase bit, advanced by hand (no division by the runtime stage count per stage)
    for (int it = 0; it < total; ++it) {
#pragma unroll
      for (int j = 0; j < kRows; ++j) io[j] = nio[j], ii[j] = nii[j];
      if (it + 1 < total) load_pairs(nio, nii);  // one stage ahead
      const char* srca[kRows];
      const char* srcb[kRows];
#pragma unroll
      for (int j = 0; j < kRows; ++j) {
        srca[j] = p.gout + size_t(io[j] != kInvalid ? io[j] : 0u) * a_row_bytes + co0 * kElem + piece * 16;
        srcb[j] = p.x + size_t(ii[j] != kInvalid ? ii[j] : 0u) * b_row_bytes + ci0 * kElem + piece * 16;
      }
      mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag);
      const uint32_t st_base = smem_u32(stages + size_t(s) * stage_bytes);
      for (int c = 0; c < p.a_chunks; ++c) {
        const bool col_ok = co0 * kElem + c * 128 + piece * 16 < a_row_bytes;
#pragma unroll
        for (int j = 0; j < kRows; ++j)
          cp_async_16(st_base + c * chunk_bytes + row_off[j], srca[j] + c * 128, (col_ok && io[j] != kInvalid) ? 16u : 0u);
      }
      for (int c = 0; c < p.b_chunks; ++c) {
        const bool col_ok = ci0 * kElem + c * 128 + piece * 16 < b_row_bytes;
#pragma unroll
        for (int j = 0; j < kRows; ++j)
          cp_async_16(st_base + a_bytes + c * chunk_bytes + row_off[j], srcb[j] + c * 128, (col_ok && ii[j] != kInvalid) ? 16u : 0u);
      }
      cp_async_arrive(&ctl->full[s]);
      if (++s == S) s = 0, ph ^= 1;
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------- MMA
    if (lane == 0) {
      uint32_t accumulate = 0;
      const int chunks_per_m = 128 / kChunkElems;  // 128-byte chunks per 128 accumulator rows
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < total; ++it) {
        mbar_wait(&ctl->full[s], ph, abort_flag);
        // both operands were written by cp.async (generic proxy), the MMA reads them through the async proxy
        fence_proxy_async_smem();
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(stages + size_t(s) * stage_bytes);
        const uint32_t b_addr = a_addr + a_bytes;
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
        if (++s == S) s = 0, ph ^= 1;
      }
      if (total > 0) umma_commit(&ctl->acc_full);
      else mbar_arrive(&ctl->acc_full);  // nothing was issued: the epilogue writes zeros
    }
  } else {
    // -------------------------------------------------------------- epilogue
    // Thread `lane` of warp w holds accumulator row 32 w + lane.  32 columns at a time go through a 4 KB staging
    // buffer per warp (the pipeline's first stage: once the accumulator is complete every stage has been consumed
    // and nothing is in flight), 16-byte pieces XOR-swizzled by the row, and come back so that eight consecutive
    // lanes hold one row's 128 contiguous bytes: every store instruction then writes four whole lines of the slab
    // instead of one 16-byte piece in each of 32 lines.
    const uint32_t slab = wg_slab_of(p.seg, p.kb, unit_kb, v, unit_j);
    mbar_wait(&ctl->acc_full, 0, abort_flag);
    tc_fence_after_sync();
    uint8_t* stage_out = stages + warp * 4096;
    for (int mt = 0; mt < p.mt; ++mt) {
      const int co_base = co0 + mt * 128 + warp * 32;
      float* obase = p.partial + (size_t(slab) * p.Co + co_base) * p.Ci;
      for (int c0 = 0; c0 < p.bn; c0 += 32) {
        uint32_t acc[32];
        if (total > 0) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + mt * p.bn + c0, acc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = 0u;
        }
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4)
          *reinterpret_cast<uint4*>(stage_out + lane * 128 + ((g4 ^ (lane & 7)) << 4)) =
              make_uint4(acc[g4 * 4], acc[g4 * 4 + 1], acc[g4 * 4 + 2], acc[g4 * 4 + 3]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = i * 4 + (lane >> 3), piece = lane & 7;
          const int ci = ci0 + c0 + piece * 4;
          const uint4 val = *reinterpret_cast<const uint4*>(stage_out + row * 128 + ((piece ^ (row & 7)) << 4));
          if (co_base + row < p.Co && ci < p.Ci) *reinterpret_cast<uint4*>(obase + size_t(row) * p.Ci + ci) = val;
        }
        __syncwarp();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (tid == 0 && ctl->abort_flag) report(p.status, FGB_S_WAIT_TIMEOUT);
}

// out[co, v, ci] = sum over the slabs of offset v, in slab order; written as dtype and/or fp32
template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, const uint32_t* __restrict__ seg, int kb,
                                                            int target_units, int Co, int V, int Ci, T* __restrict__ out,
                                                            float* __restrict__ out_f32, int accumulate) {
  __shared__ int s_unit_kb;
  chain_release();
  // the plan depends on the segment table only (written by the cache build): it is made while the wgrad kernel runs
  if (threadIdx.x < 32) {
    const uint32_t ukb = wg_plan_unit_kb(seg, V, kb, static_cast<uint32_t>(target_units), threadIdx.x);
    if (threadIdx.x == 0) s_unit_kb = static_cast<int>(ukb);
  }
  __syncthreads();
  const int unit_kb = s_unit_kb;
  const int v = blockIdx.y;
  const int64_t e = (blockIdx.x * int64_t(256) + threadIdx.x) * 4;  // element of the [Co, Ci] slab
  const uint32_t first = wg_slab_of(seg, kb, unit_kb, v, 0);
  const uint32_t count = wg_chunks_of(seg, v, kb, unit_kb);
  chain_wait();  // the slabs are complete
  if (e >= int64_t(Co) * Ci) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* src = partial + size_t(first) * Co * Ci + e;
  const size_t slab = size_t(Co) * Ci;
  uint32_t s = 0;
  for (; s + 4 <= count; s += 4) {  // four loads in flight, added in slab order
    const float4 t0 = __ldg(reinterpret_cast<const float4*>(src + (s + 0) * slab));
    const float4 t1 = __ldg(reinterpret_cast<const float4*>(src + (s + 1) * slab));
    const float4 t2 = __ldg(reinterpret_cast<const float4*>(src + (s + 2) * slab));
    const float4 t3 = __ldg(reinterpret_cast<const float4*>(src + (s + 3) * slab));
    acc.x += t0.x, acc.y += t0.y, acc.z += t0.z, acc.w += t0.w;
    acc.x += t1.x, acc.y += t1.y, acc.z += t1.z, acc.w += t1.w;
    acc.x += t2.x, acc.y += t2.y, acc.z += t2.z, acc.w += t2.w;
    acc.x += t3.x, acc.y += t3.y, acc.z += t3.z, acc.w += t3.w;
  }
  for (; s < count; ++s) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(src + s * slab));
    acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
  }
  const int co = static_cast<int>(e / Ci), ci = static_cast<int>(e % Ci);
  const int64_t o = (int64_t(co) * V + v) * Ci + ci;
  if (accumulate) {  // later passes of the fp32-accurate mode add to what an earlier pass wrote (fp32 outputs only)
    const float* prev = out_f32 ? out_f32 : reinterpret_cast<const float*>(out);
    const float4 t = *reinterpret_cast<const float4*>(prev + o);
    acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
  }
  if (out_f32) *reinterpret_cast<float4*>(out_f32 + o) = acc;
  if (out) {
    if constexpr (std::is_same<T, float>::value) {
      *reinterpret_cast<float4*>(out + o) = acc;
    } else {
      T t4[4] = {static_cast<T>(acc.x), static_cast<T>(acc.y), static_cast<T>(acc.z), static_cast<T>(acc.w)};
      *reinterpret_cast<uint2*>(out + o) = *reinterpret_cast<uint2*>(t4);
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
  w.a_chunks = w.mt * 128 * eb / 128;
  w.b_chunks = static_cast<int>(ceil_div(w.bn * eb, 128));
  // pairs per stage: as many as keep a stage near 64 KB (more pairs per stage for narrow channel counts, so that the
  // fixed cost of a stage hand-over is spread over enough bytes); a multiple of 32 (one row per gather lane group)
  w.kb = 32;
  while (w.kb < 32 * kWgRowsMax && size_t(w.a_chunks + w.b_chunks) * (w.kb * 2) * 128 <= 64 * 1024) w.kb *= 2;
  const size_t stage = size_t(w.a_chunks + w.b_chunks) * w.kb * 128;
  const size_t budget = 224 * 1024;
  w.stages = static_cast<int>(budget / stage);
  if (w.stages > kWgMaxStages) w.stages = kWgMaxStages;
  if (w.stages < 2) w.stages = 2;
  uint32_t cols = 32;
  while (cols < uint32_t(w.mt * w.bn)) cols <<= 1;
  w.tmem_cols = cols;
  w.smem = 1024 + 1024 + stage * w.stages;
  return w;
}

// CTAs of one (output-channel group, input-channel tile) that run together: one per SM
static int wave_units(const WgradPlan& w) {
  const int sms = device_sm_count();
  const int per_wave = sms / (w.co_groups * w.ci_tiles);
  return per_wave > 0 ? per_wave : 1;
}

// Units to cut the pair lists into for `splitk` parts per offset on average: the workspace holds (splitk + 1) * V
// slabs; of those, a whole number of waves when that is at least one wave (a unit count just above a multiple of the
// wave runs as one more, nearly empty wave: measured 248 -> 388 us from 5 to 6 parts at RES=256, C=256).
static int target_units(const WgradPlan& w, int V, int splitk) {
  const int64_t budget = (int64_t(splitk) + 1) * V;
  const int64_t wave = wave_units(w);
  const int64_t t = budget >= wave ? budget / wave * wave : budget;
  return static_cast<int>(t);
}

// Row bands of the pair-list walk (see wg_band_pos): bands of about 8 MB of rows of both matrices, so that the band the
// CTAs are working on -- and the one they drift into -- stay in L2; never so many that the partial k-block at the end of
// every (offset, band) piece adds up to more than ~2 % of the blocks; at most kWgMaxBands.  0 = automatic.
static std::atomic<int> g_row_bands{0};

static void plan_bands(int64_t n_out, int64_t n_in, int64_t n_pairs, int Ci, int Co, int V, int eb, int kb, bool have_offsets,
                       bool whole_channels, int* bands, uint32_t* nblk, uint32_t* band_blocks) {
  const int64_t blocks = ceil_div(n_out > 0 ? n_out : 1, kMapBlock);
  int64_t b = 1;
  if (have_offsets) {
    const int forced = g_row_bands.load(std::memory_order_relaxed);
    if (forced > 0) {
      b = forced;
    } else if (!whole_channels) {
      // several CTAs per unit (channel counts above 256): measured 2-4 % slower with bands (RES=64 x 4, C=512; RES=128,
      // C=1024), so the lists are walked in one piece there
      b = 1;
    } else {
      const int64_t row_bytes = (n_out * Co + n_in * Ci) * eb;
      // rows that fit L2 (126 MB) are shared by the offsets anyway: bands only cost their partial blocks there
      b = row_bytes > (int64_t(126) << 20) ? row_bytes / (int64_t(8) << 20) : 1;
      const int64_t waste_cap = n_pairs / (int64_t(25) * kb * V);  // 0.5 * V * bands <= 2 % of n_pairs / kb
      if (b > waste_cap) b = waste_cap;
    }
    if (b > kWgMaxBands) b = kWgMaxBands;
    if (b > blocks) b = blocks;
    if (b < 1) b = 1;
  }
  const int64_t per = ceil_div(blocks, b);
  *bands = static_cast<int>(ceil_div(blocks, per));
  *nblk = static_cast<uint32_t>(blocks);
  *band_blocks = static_cast<uint32_t>(per);
}

}  // namespace fgb

extern "C" int fgb_wgrad_set_row_bands(int bands) {
  if (bands < 0 || bands > fgb::kWgMaxBands) return FGB_E_SIZE;
  return fgb::g_row_bands.exchange(bands, std::memory_order_relaxed);
}

extern "C" int fgb_wgrad_default_splitk(int64_t n_pairs, int Ci, int Co, int V, int dtype) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  const WgradPlan w = plan_wgrad(Ci, Co, eb);
  // One wave of CTAs, one per SM, whatever the input size: the kernel plans the unit length from the segment table so
  // that the unit count fills the wave exactly, and splitk only has to make room for it.  (Two waves were best while
  // the slab write-out was slow; with whole-line stores one wave wins at every size measured -- RES=256 C=256 248
  // against 271 us, RES=128 C=256 86 against 104, RES=128 C=64 46 against 53, RES=1024 C=64 1650 against 1698 for
  // five waves -- and every further wave costs a little more: partial slabs and a write-out pause per unit.)
  const int64_t wave = wave_units(w);
  int64_t s = ceil_div(wave, V) - 1;  // (s + 1) * V >= wave
  // no more splits than stages of pairs per offset on average
  const int64_t max_s = n_pairs > 0 ? ceil_div(ceil_div(n_pairs, V), w.kb) : 1;
  if (s > max_s) s = max_s;
  if (s > 1024) s = 1024;
  if (s < 1) s = 1;
  return static_cast<int>(s);
}

extern "C" int64_t fgb_conv_workspace_bytes(int pass, int64_t n, int Ci, int Co, int V, int dtype, int splitk) {
  return fgb_sparse_conv_workspace_bytes(pass, n, n, Ci, Co, V, dtype, splitk);
}

extern "C" int64_t fgb_sparse_conv_workspace_bytes(int pass, int64_t n_out, int64_t n_in, int Ci, int Co, int V, int dtype, int splitk) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (n_out < 0 || n_in < 0 || Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  const int64_t w_elems = int64_t(Ci) * V * Co;
  const bool ieee = dtype == FGB_F32_IEEE;
  switch (pass) {
    case 0:  // header with the ticket counter (+ fp32-accurate mode: tripled activations and weights; + split-K slabs of a small launch)
      return 256 + (ieee ? align256(n_in * 3 * Ci * 4) + align256(w_elems * 3 * 4) : 0) + igemm_partial_bytes(n_out, Co, V);
    case 1:  // header, re-laid-out weight (+ its tripled copy and the tripled grad_out; + split-K slabs)
      return 256 + align256(w_elems * eb) + (ieee ? align256(w_elems * 3 * 4) + align256(n_out * 3 * Co * 4) : 0) +
             igemm_partial_bytes(n_in, Ci, V);
    case 2:  // slabs [Co, Ci] for up to (splitk + 1) * V units (+ hi/lo copies of both operands)
      if (splitk < 1 || splitk > 1024) return FGB_E_SIZE;
      return align256(w_elems * 4 * (int64_t(splitk) + 1)) + (ieee ? 2 * align256(n_in * Ci * 4) + 2 * align256(n_out * Co * 4) : 0);
    default:
      return FGB_E_SIZE;
  }
}

namespace fgb {
// One launcher per kernel instance: the dynamic shared-memory limit is a property of (kernel, device), and all
// instances share one function-pointer type, so the table must hang on the template arguments, not on the type.
template <int kElem, int kRows, bool kBanded>
static int launch_wgrad_instance(int64_t grid, size_t smem, const WgradParams& p, cudaStream_t s) {
  static PerDeviceTable configured;
  const int rc = ensure_dynamic_smem(configured, subm_wgrad_kernel<kElem, kRows, kBanded>, smem);
  if (rc != FGB_OK) return rc;
  subm_wgrad_kernel<kElem, kRows, kBanded><<<static_cast<unsigned>(grid), kWgThreads, smem, s>>>(p);
  return launch_status();
}
template <int kElem, int kRows>
static int launch_wgrad(int64_t grid, size_t smem, const WgradParams& p, cudaStream_t s) {
  return p.bands > 1 ? launch_wgrad_instance<kElem, kRows, true>(grid, smem, p, s) : launch_wgrad_instance<kElem, kRows, false>(grid, smem, p, s);
}

// one wgrad pass over operands of element type `dtype` (never FGB_F32_IEEE): partial slabs, then the ordered sum
static int wgrad_pass(const void* grad_out, const void* feats, const uint32_t* vs_i, const uint32_t* vs_o, const uint32_t* seg,
                      const uint32_t* block_offsets, void* grad_weight, float* grad_weight_f32, int64_t n_out, int64_t n_in,
                      int64_t n_pairs, int Ci, int Co, int V, int dtype, int splitk, float* slabs, int accumulate, int32_t* status,
                      cudaStream_t s) {
  const int eb = elem_bytes(dtype);
  const WgradPlan w = plan_wgrad(Ci, Co, eb);
  WgradParams p;
  p.gout = static_cast<const char*>(grad_out);
  p.x = static_cast<const char*>(feats);
  p.vs_i = vs_i;
  p.vs_o = vs_o;
  p.seg = seg;
  p.block_offsets = block_offsets;
  plan_bands(n_out, n_in, n_pairs, Ci, Co, V, eb, w.kb, block_offsets != nullptr, w.co_groups * w.ci_tiles == 1, &p.bands, &p.nblk,
             &p.band_blocks);
  p.partial = slabs;
  p.Co = Co, p.Ci = Ci, p.V = V;
  p.target_units = target_units(w, V, splitk);
  const int64_t max_units = p.target_units;
  p.mt = w.mt, p.bn = w.bn, p.co_groups = w.co_groups, p.ci_tiles = w.ci_tiles;
  p.kb = w.kb, p.stages = w.stages, p.a_chunks = w.a_chunks, p.b_chunks = w.b_chunks;
  const uint32_t fmt = dtype == FGB_F16 ? kFmtF16 : dtype == FGB_BF16 ? kFmtBF16 : kFmtTF32;
  p.idesc = make_idesc(fmt, 128, w.bn, 1, 1);
  p.tmem_cols = w.tmem_cols;
  p.order = 0;  // offset-major: measured faster than chunk-major on B200 (chunk-major makes every SM stream the same rows at once)
  p.status = status;
  const int64_t grid = max_units * w.co_groups * w.ci_tiles;
  if (grid > 0x7FFFFFFF) return FGB_E_SIZE;
  const int rows = w.kb / 32;
  int rc;
  if (eb == 2) rc = rows == 4 ? launch_wgrad<2, 4>(grid, w.smem, p, s) : rows == 2 ? launch_wgrad<2, 2>(grid, w.smem, p, s) : launch_wgrad<2, 1>(grid, w.smem, p, s);
  else rc = rows == 4 ? launch_wgrad<4, 4>(grid, w.smem, p, s) : rows == 2 ? launch_wgrad<4, 2>(grid, w.smem, p, s) : launch_wgrad<4, 1>(grid, w.smem, p, s);
  if (rc != FGB_OK) return rc;
  const dim3 rgrid(static_cast<unsigned>(ceil_div(int64_t(Co) * Ci, 1024)), static_cast<unsigned>(V));
  switch (dtype) {
    case FGB_F16:
      rc = cuda_status(launch_chained(splitk_reduce_kernel<__half>, rgrid, dim3(256), 0, s, static_cast<const float*>(slabs), seg, p.kb,
                                      p.target_units, Co, V, Ci, static_cast<__half*>(grad_weight), grad_weight_f32, 0));
      break;
    case FGB_BF16:
      rc = cuda_status(launch_chained(splitk_reduce_kernel<__nv_bfloat16>, rgrid, dim3(256), 0, s, static_cast<const float*>(slabs), seg,
                                      p.kb, p.target_units, Co, V, Ci, static_cast<__nv_bfloat16*>(grad_weight), grad_weight_f32, 0));
      break;
    default:
      rc = cuda_status(launch_chained(splitk_reduce_kernel<float>, rgrid, dim3(256), 0, s, static_cast<const float*>(slabs), seg, p.kb,
                                      p.target_units, Co, V, Ci, static_cast<float*>(grad_weight), grad_weight_f32, accumulate));
  }
  return rc != FGB_OK ? rc : launch_status();
}
}  // namespace fgb

extern "C" int fgb_subm_conv_wgrad(const void* grad_out, const void* feats, const uint32_t* valid_signal_i,
                                   const uint32_t* valid_signal_o, const uint32_t* valid_signal_seg, const uint32_t* block_offsets,
                                   void* grad_weight, float* grad_weight_f32, int64_t n, int64_t n_pairs, int Ci, int Co, int V,
                                   int dtype, int splitk, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  return fgb_sparse_conv_wgrad(grad_out, feats, valid_signal_i, valid_signal_o, valid_signal_seg, block_offsets, grad_weight,
                               grad_weight_f32, n, n, n_pairs, Ci, Co, V, dtype, splitk, workspace, workspace_bytes, status, stream);
}

extern "C" int fgb_sparse_conv_wgrad(const void* grad_out, const void* feats, const uint32_t* valid_signal_i,
                                     const uint32_t* valid_signal_o, const uint32_t* valid_signal_seg, const uint32_t* block_offsets,
                                     void* grad_weight, float* grad_weight_f32, int64_t n_out, int64_t n_in, int64_t n_pairs, int Ci,
                                     int Co, int V, int dtype, int splitk, void* workspace, int64_t workspace_bytes, int32_t* status,
                                     void* stream) {
  using namespace fgb;
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (n_out < 0 || n_in < 0 || n_pairs < 0 || n_pairs > n_out * V || Ci <= 0 || Co <= 0 || V < 1 || V > 32 || splitk < 1 || splitk > 1024)
    return FGB_E_SIZE;
  if ((Ci * eb) % 16 || (Co * eb) % 16) return FGB_E_ALIGN;
  if (!valid_signal_seg || !workspace) return FGB_E_NULL;
  if (n_pairs > 0 && (!grad_out || !feats || !valid_signal_i || !valid_signal_o)) return FGB_E_NULL;
  if (!grad_weight && !grad_weight_f32) return FGB_E_NULL;
  if ((reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(feats) | reinterpret_cast<uintptr_t>(grad_weight) |
       reinterpret_cast<uintptr_t>(grad_weight_f32)) & 15)
    return FGB_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FGB_E_ALIGN;
  if (workspace_bytes < fgb_sparse_conv_workspace_bytes(2, n_out, n_in, Ci, Co, V, dtype, splitk)) return FGB_E_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* slabs = static_cast<float*>(workspace);
  if (dtype != FGB_F32_IEEE)
    return wgrad_pass(grad_out, feats, valid_signal_i, valid_signal_o, valid_signal_seg, block_offsets, grad_weight, grad_weight_f32,
                      n_out, n_in, n_pairs, Ci, Co, V, dtype, splitk, slabs, 0, status, s);
  // fp32-accurate: g_hi*x_hi + g_hi*x_lo + g_lo*x_hi, three passes adding into the fp32 output
  char* base = static_cast<char*>(workspace) + align256(int64_t(Ci) * V * Co * 4 * (int64_t(splitk) + 1));
  float* x_hi = reinterpret_cast<float*>(base);
  float* x_lo = reinterpret_cast<float*>(base + align256(n_in * Ci * 4));
  float* g_hi = reinterpret_cast<float*>(base + 2 * align256(n_in * Ci * 4));
  float* g_lo = reinterpret_cast<float*>(base + 2 * align256(n_in * Ci * 4) + align256(n_out * Co * 4));
  int rc = FGB_OK;
  if (n_in > 0) rc = launch_split2(static_cast<const float*>(feats), x_hi, x_lo, n_in * Ci, s);
  if (rc != FGB_OK) return rc;
  if (n_out > 0) rc = launch_split2(static_cast<const float*>(grad_out), g_hi, g_lo, n_out * Co, s);
  if (rc != FGB_OK) return rc;
  const float* ga[3] = {g_hi, g_hi, g_lo};
  const float* xa[3] = {x_hi, x_lo, x_hi};
  for (int pass = 0; pass < 3; ++pass) {
    rc = wgrad_pass(ga[pass], xa[pass], valid_signal_i, valid_signal_o, valid_signal_seg, block_offsets, grad_weight, grad_weight_f32,
                    n_out, n_in, n_pairs, Ci, Co, V, FGB_F32_TF32, splitk, slabs, pass > 0, status, s);
    if (rc != FGB_OK) return rc;
  }
  return FGB_OK;
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

// Host-side replay of the kernel's work split, for tests: which pairs each CTA of a wgrad launch would read.
// seg and block_offsets are HOST arrays here.  For every unit u (offset-major, as the slabs are stored) and band b,
// plan[(u * bands + b) * 3 + {0, 1, 2}] = first pair, k-blocks, end of the band in the pair list.  Returns the number
// of units, or a negative code; *bands_out and *kb_out receive the band count and the pairs per k-block.
extern "C" int fgb_wgrad_plan_host(const uint32_t* seg, const uint32_t* block_offsets, int64_t n_out, int64_t n_in, int Ci, int Co, int V,
                                   int dtype, int splitk, uint32_t* plan, int64_t plan_capacity, int* bands_out, int* kb_out) {
  using namespace fgb;
  const int eb = elem_bytes(dtype == FGB_F32_IEEE ? FGB_F32_TF32 : dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (!seg || !plan || !bands_out || !kb_out) return FGB_E_NULL;
  if (n_out < 0 || n_in < 0 || Ci <= 0 || Co <= 0 || V < 1 || V > 32 || splitk < 1 || splitk > 1024) return FGB_E_SIZE;
  const WgradPlan w = plan_wgrad(Ci, Co, eb);
  const uint32_t target = static_cast<uint32_t>(target_units(w, V, splitk));
  const int64_t n_pairs = seg[V];
  int bands = 1;
  uint32_t nblk = 0, band_blocks = 0;
  plan_bands(n_out, n_in, n_pairs, Ci, Co, V, eb, w.kb, block_offsets != nullptr, w.co_groups * w.ci_tiles == 1, &bands, &nblk, &band_blocks);
  // the kernel's bisection (wg_plan_unit_kb) with loops in place of warp reductions
  uint32_t nk[32], hi = 1;
  for (int v = 0; v < V; ++v) {
    nk[v] = (seg[v + 1] - seg[v] + w.kb - 1) / w.kb;
    if (nk[v] > hi) hi = nk[v];
  }
  uint32_t lo = 1;
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    uint32_t units = 0;
    for (int v = 0; v < V; ++v) units += (nk[v] + mid - 1) / mid;
    if (units <= target) hi = mid;
    else lo = mid + 1;
  }
  const uint32_t unit_kb = lo;
  int u = 0;
  for (int v = 0; v < V; ++v) {
    const uint32_t K = (nk[v] + unit_kb - 1) / unit_kb;
    for (uint32_t k = 0; k < K; ++k, ++u) {
      if (int64_t(u + 1) * bands * 3 > plan_capacity) return FGB_E_WORKSPACE;
      uint32_t rot = 0;
      for (int b = 0; b < bands; ++b) {
        const uint32_t begin = wg_band_pos(seg, block_offsets, nblk, band_blocks, bands, v, b);
        const uint32_t end = wg_band_pos(seg, block_offsets, nblk, band_blocks, bands, v, b + 1);
        const uint32_t nkb = (end - begin + w.kb - 1) / w.kb;
        uint32_t first = 0;
        uint32_t cnt;
        if (bands == 1) {
          first = k * unit_kb;
          cnt = first < nkb ? std::min(nkb - first, unit_kb) : 0u;
        } else {
          cnt = wg_band_share(nkb, K, k, rot, &first);
        }
        rot += nkb % K;
        uint32_t* e = plan + (size_t(u) * bands + b) * 3;
        e[0] = begin + first * w.kb, e[1] = cnt, e[2] = end;
      }
    }
  }
  *bands_out = bands;
  *kb_out = w.kb;
  return u;
}
