// Masked implicit GEMM for submanifold conv fprop and dgrad on sm_100a.
//
//   out[r, :] = bias + sum_{v in mask(tile(r))} x[nbr[r, v], :] . Wn[:, v, :]^T
//
// Persistent kernel: one CTA per SM walks over work items (a block of 256
// sorted rows x BN output channels).  The block is two 128-row halves with one
// TMEM accumulator each; both halves multiply the same dense weight tile, so a
// weight tile fetched once feeds two MMAs, and each half skips the offsets that
// are absent from its own 27-bit mask (no gather, no MMA for it).
//
// Warp roles (576 threads):
//   warps 0-3, 14-17
//               epilogue: tcgen05.ld -> +bias -> convert -> staged through a
//               small swizzled shared-memory buffer so that every global store
//               instruction writes whole 128-byte lines of out[sorted_idx[row]];
//               runs while the next block is gathered.  Two warps per quarter
//               of the accumulator rows, alternating 64-column passes: the MMA
//               lane waits for the drain (one accumulator pair fills TMEM at
//               BN = 256), so halving it is worth the extra warps;
//   warp 4      one lane streams the dense weight tile [BN x 128 B] of the
//               current (offset, channel slice) with a tiled TMA load;
//   warp 5      owns the TMEM allocation; one lane issues tcgen05.mma and
//               releases stages / publishes accumulators with tcgen05.commit;
//   warps 6-13  gather the activation rows of both halves into a 128B-swizzled
//               K-major stage with 16-byte cp.async (zero fill for missing
//               neighbours and past the channel count).  Neighbour indices are
//               read straight from the map into registers one offset ahead;
//               each thread's copies arrive on the stage's mbarrier when they
//               land, so every stage can be in flight at once.
//   (A TMA row gather -- tile::gather4 -- was measured for the activation rows:
//    correct, zero-fills missing rows, but ~2.4x slower than cp.async for
//    128-byte rows, so the copies stay on the LSU path.)
//
// dgrad is the same kernel: x = grad_out, the weight is first re-laid-out to
// [Ci, V, Co] and offset v reads weight slot V-1-v.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

#include "fgb_common.cuh"
#include "fgb_device.cuh"
#include "fgb_precision.cuh"
#include "fgb_umma.cuh"

namespace fgb {

constexpr int kTileM = 128;             // rows per accumulator (and per tile mask)
constexpr int kBlockM = 2 * kTileM;     // rows per work item
constexpr int kMaxStages = 6;
constexpr int kSchedRing = 16;  // deeper than the gather front can ever run ahead of the epilogue (stages + accumulator sets + 1 blocks)
constexpr int kSchedReaders = 18;  // 8 gather warps, the TMA lane, the MMA lane, 8 epilogue warps
constexpr int kIgemmThreads = 576;
constexpr int kEpilogueWarp1 = 14;  // second group of epilogue warps: 14..17 (the first is 0..3)
constexpr int kGatherWarp0 = 6;
constexpr int kGatherThreads = 256;
constexpr int kStoreStageBytes = 8 * 4096;  // per epilogue warp: 32 rows x 128 bytes
constexpr int kCtrlBytes = 1024;        // barriers, TMEM holder, abort flag
constexpr int kATileBytes = kTileM * 128;
constexpr int kSmemBudget = 226 * 1024;

struct IgemmParams {
  const char* x;             // [n, kc] gathered operand
  const void* bias;          // [nout] or null
  const uint32_t* nbr;       // [n, V]
  const int64_t* sorted_idx; // [n]
  const uint32_t* tile_masks; // one mask per 128 sorted rows
  const uint32_t* block_order; // row blocks in descending cost order, or null for natural order
  uint32_t* ticket;          // zeroed counter: the next position of the block list to hand out
  char* out;                 // [n, nout]
  uint32_t n;
  uint32_t num_tiles;        // ceil(n / 128)
  uint32_t num_blocks;       // ceil(n / 256)
  int kc;                    // reduction channels per offset
  int nout;                  // output channels
  int V;
  int bn;                    // output channels per work item (32, 64, 128, 256)
  int n_tiles_n;
  int splits;                // split-K: shares of a block's offsets that run as separate work items (1 = off)
  int items_per_block;       // n_tiles_n * splits
  int row_bytes;             // kc * element size
  int num_kb;                // 128-byte slices per row
  int flip;                  // bit 0: weight slot = V-1-v instead of v; bit 1: the weight operand is MN-major (below)
  int stages;
  int acc_sets;              // accumulator pairs that fit in TMEM (1 or 2)
  uint32_t idesc;
  int32_t* status;
};

// what the fused epilogue adds (a kernel parameter of its own: the plain kernel's parameter block, and with it its
// register allocation, stays as tuned)
struct FusedEpilogue {
  const char* residual;      // fused epilogue: [n, nout] added after the activation, or null
  char* preact;              // fused epilogue: [n, nout] copy of the result before the activation, or null
  int act;                   // fused epilogue: FGB_ACT_NONE / FGB_ACT_SILU
};

struct IgemmSmem {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sched_full[kSchedRing];   // work entry published
  uint64_t sched_empty[kSchedRing];  // work entry read by every role
  uint32_t sched_entry[kSchedRing];  // block * items_per_block + (column tile * splits + split), or kInvalid = no more work
  uint32_t tmem_base;
  uint32_t abort_flag;
};
static_assert(sizeof(IgemmSmem) <= kCtrlBytes, "control block too large");

// Converts 32 accumulator columns of one row, adds the bias and writes them as
// 16-byte pieces into the warp's staging buffer: row `lane`, pieces
// chunk*4 .. chunk*4+3 (16-bit types: two chunks fill a 128-byte row) or 0 .. 7
// (fp32: one chunk is a whole 128-byte row); piece p of row r sits at p ^ (r & 7).
// 16-bit types: two columns are rounded per instruction and the bias is added to
// the rounded pair in the output type (what a bias add after the conversion does);
// fp32 adds in fp32.  The epilogue runs while the MMA lane waits for the
// accumulator, so its length in instructions is time the tensor pipe idles.
template <int kDtype>
__device__ __forceinline__ void stage_row_chunk(uint8_t* stage, int lane, int chunk, const uint32_t (&acc)[32], const void* bias,
                                                int col0, int nout) {
  uint8_t* row = stage + lane * 128;
  if constexpr (kDtype == FGB_F16 || kDtype == FGB_BF16) {
    using T = typename std::conditional<kDtype == FGB_F16, __half, __nv_bfloat16>::type;
    using T2 = typename std::conditional<kDtype == FGB_F16, __half2, __nv_bfloat162>::type;
#pragma unroll
    for (int g = 0; g < 4; ++g) {  // 8 columns = 16 bytes
      const int c = col0 + g * 8;
      uint4 o;
      T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __uint_as_float(acc[g * 8 + 2 * i]), hi = __uint_as_float(acc[g * 8 + 2 * i + 1]);
        if constexpr (kDtype == FGB_F16) o2[i] = __floats2half2_rn(lo, hi);
        else o2[i] = __floats2bfloat162_rn(lo, hi);
      }
      if (bias != nullptr && c < nout) {
        const uint4 bw = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(bias) + c));
        const T2* b2 = reinterpret_cast<const T2*>(&bw);
#pragma unroll
        for (int i = 0; i < 4; ++i) o2[i] = __hadd2(o2[i], b2[i]);
      }
      *reinterpret_cast<uint4*>(row + (((chunk * 4 + g) ^ (lane & 7)) << 4)) = o;
    }
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) {  // 4 columns = 16 bytes
      const int c = col0 + g * 4;
      float4 o = make_float4(__uint_as_float(acc[g * 4]), __uint_as_float(acc[g * 4 + 1]), __uint_as_float(acc[g * 4 + 2]),
                             __uint_as_float(acc[g * 4 + 3]));
      if (bias != nullptr && c < nout) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(bias) + c));
        o.x += b.x, o.y += b.y, o.z += b.z, o.w += b.w;
      }
      *reinterpret_cast<float4*>(row + ((g ^ (lane & 7)) << 4)) = o;
    }
  }
}

// Fused epilogue on one 16-byte piece of an output row (8 values of a 16-bit type, 4 of fp32), already rounded to the
// output type: optionally keeps a copy (what a backward pass of the activation needs), applies the activation in
// fp32, adds the residual piece, rounds again -- the roundings of the unfused sequence conv -> activation -> add.
template <int kDtype>
__device__ __forceinline__ uint4 fuse_piece(uint4 val, int act, const char* residual, char* preact, size_t byte_off) {
  if (preact != nullptr) *reinterpret_cast<uint4*>(preact + byte_off) = val;
  uint4 res = make_uint4(0, 0, 0, 0);
  if (residual != nullptr) res = __ldg(reinterpret_cast<const uint4*>(residual + byte_off));
  auto f = [&](float x, float r) {
    if (act == FGB_ACT_SILU) x = x / (1.f + __expf(-x));
    return x + r;
  };
  uint4 o;
  if constexpr (kDtype == FGB_F16 || kDtype == FGB_BF16) {
    using T = typename std::conditional<kDtype == FGB_F16, __half, __nv_bfloat16>::type;
    const T* vt = reinterpret_cast<const T*>(&val);
    const T* rt = reinterpret_cast<const T*>(&res);
    T* ot = reinterpret_cast<T*>(&o);
    const bool two_roundings = act != FGB_ACT_NONE && residual != nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float x = static_cast<float>(vt[i]);
      if (two_roundings) {  // activation output rounded to the type before the add, as a separate activation kernel would
        x = static_cast<float>(static_cast<T>(f(x, 0.f)));
        ot[i] = static_cast<T>(x + static_cast<float>(rt[i]));
      } else {
        ot[i] = static_cast<T>(f(x, residual != nullptr ? static_cast<float>(rt[i]) : 0.f));
      }
    }
  } else {
    const float* vt = reinterpret_cast<const float*>(&val);
    const float* rt = reinterpret_cast<const float*>(&res);
    float* ot = reinterpret_cast<float*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) ot[i] = f(vt[i], residual != nullptr ? rt[i] : 0.f);
  }
  return o;
}

// kMode: kPlain -- the epilogue adds the bias and writes `out` in the operand type; kFusedEp -- the same plus
// activation / residual / pre-activation copy; kSplitK -- the work item covers only a share of the block's offsets and
// the epilogue writes the raw fp32 accumulators into its split's slab of a partial buffer (summed by a second kernel).
enum { kPlain = 0, kFusedEp = 1, kSplitK = 2 };

template <int kDtype, int kMode>
__global__ void __launch_bounds__(kIgemmThreads, 1)
    subm_igemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const IgemmParams p, const FusedEpilogue fe) {
  constexpr bool kTF32 = (kDtype == FGB_F32_TF32);
  constexpr bool kFused = kMode == kFusedEp;
  constexpr bool kSplit = kMode == kSplitK;
  constexpr int kElem = (kDtype == FGB_F16 || kDtype == FGB_BF16) ? 2 : 4;
  constexpr int kOutDtype = kSplit ? FGB_F32_TF32 : kDtype;  // element type the epilogue writes
  constexpr int kElemOut = kSplit ? 4 : kElem;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: align by hand
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  IgemmSmem* ctl = reinterpret_cast<IgemmSmem*>(smem);
  uint8_t* stages = smem + kCtrlBytes;
  const int stage_bytes = 2 * kATileBytes + p.bn * 128;  // A half 0 | A half 1 | B
  const int S = p.stages;

  // Launched chained (fgb_device.cuh): the CTA may be on its SM before the kernel ahead in the stream has finished.
  chain_release();
  chain_wait();
  // A kernel that already reported a soft error makes the rest of the grid a
  // no-op.  One thread reads the word so that the whole CTA takes the same branch.
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = p.status != nullptr && *reinterpret_cast<volatile const int32_t*>(p.status) != 0;
  __syncthreads();
  if (s_skip) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int V = p.V;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&ctl->full[s], kGatherThreads + 1);  // every gather thread (when its copies land) + the TMA lane
      mbar_init(&ctl->empty[s], 1);                  // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&ctl->acc_full[a], 1);   // tcgen05.commit after the block's last MMA
      mbar_init(&ctl->acc_empty[a], 8);  // the eight epilogue warps
    }
    for (int k = 0; k < kSchedRing; ++k) {
      mbar_init(&ctl->sched_full[k], 1);
      mbar_init(&ctl->sched_empty[k], kSchedReaders);
    }
    ctl->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 4 && lane == 0) tma_prefetch_desc(&tmap_w);
  if (warp == 5) {
    tmem_alloc_dyn(&ctl->tmem_base, 512u);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  // Work distribution.  Work items (row block x column tile x split-K share) are handed out
  // dynamically, blocks in descending cost order, from a global ticket counter: lane 0 of the first gather warp
  // claims the ticket of the CTA's next item when the gather front is about to
  // finish the current one, and publishes it (or "no more work") in a
  // small shared-memory ring that every role reads in order.  So each role walks
  // the same sequence of work items, an SM that got cheap blocks simply takes
  // more of them, and within an item all roles enumerate the offsets of the
  // union mask in ascending order, num_kb slices each.
  const uint32_t none = 0xFFFFFFFFu;  // "no more work" (kInvalid as a plain value, usable in conditional expressions)
  auto publish_work = [&](uint32_t k, uint32_t& pub_block, uint32_t& pub_ntile) {  // one thread
    const uint32_t slot = k % kSchedRing;
    mbar_wait(&ctl->sched_empty[slot], ((k / kSchedRing) & 1) ^ 1, abort_flag);
    // one ticket = one work item; the items of a block (its column tiles and split-K shares) have consecutive tickets,
    // so they run at about the same time on different SMs and find the block's gathered rows in L2
    const uint32_t ipb = static_cast<uint32_t>(p.items_per_block);
    const uint32_t t = pub_block == none ? none : atomicAdd(p.ticket, 1u);
    if (t == none || t / ipb >= p.num_blocks) {
      pub_block = none;  // stays "no more work"
    } else {
      const uint32_t pos = ipb == 1 ? t : t / ipb;
      pub_block = p.block_order != nullptr ? __ldg(&p.block_order[pos]) : pos;
      pub_ntile = t - pos * ipb;
    }
    ctl->sched_entry[slot] = (pub_block == none || *abort_flag) ? none : pub_block * ipb + pub_ntile;
    mbar_arrive(&ctl->sched_full[slot]);
  };
  // k-th work item of this CTA; every reader (a whole warp, or a single lane when
  // `one_lane`) calls it exactly once per k, in order, until it returns false
  auto work_of = [&](uint32_t k, uint32_t& mblk, uint32_t& ntile, bool one_lane) -> bool {
    const uint32_t slot = k % kSchedRing;
    const bool ok = mbar_wait(&ctl->sched_full[slot], (k / kSchedRing) & 1, abort_flag);
    const uint32_t e = ok ? *reinterpret_cast<volatile uint32_t*>(&ctl->sched_entry[slot]) : none;
    if (!one_lane) __syncwarp();
    if (one_lane || lane == 0) mbar_arrive(&ctl->sched_empty[slot]);
    if (e == kInvalid) return false;
    mblk = p.items_per_block == 1 ? e : e / p.items_per_block;  // once per work item
    ntile = e - mblk * p.items_per_block;  // column tile * splits + split
    return true;
  };
  // column tile and split of a work item's sub-index
  auto tile_of = [&](uint32_t sub) -> uint32_t { return kSplit ? sub / static_cast<uint32_t>(p.splits) : sub; };
  auto split_of = [&](uint32_t sub) -> uint32_t { return kSplit ? sub % static_cast<uint32_t>(p.splits) : 0u; };
  // Offset masks of the two halves of a work item.  With split-K the item keeps only its share of the block's
  // offsets: the set bits of the union mask, in ascending order, are dealt to the splits in equal runs (a split beyond
  // the number of offsets gets none and writes zeros).  Every role derives the same masks from the same words.
  auto masks_of = [&](uint32_t mblk, uint32_t sub, uint32_t& m0, uint32_t& m1) {
    const uint32_t t0 = mblk * 2;
    m0 = __ldg(&p.tile_masks[t0]);
    m1 = t0 + 1 < p.num_tiles ? __ldg(&p.tile_masks[t0 + 1]) : 0u;
    if constexpr (kSplit) {
      const uint32_t un = m0 | m1, count = __popc(un), sp = split_of(sub), S = static_cast<uint32_t>(p.splits);
      const uint32_t first = sp * count / S, last = (sp + 1) * count / S;
      uint32_t keep = 0, rank = 0;
      for (uint32_t u = un; u != 0u; u &= u - 1u, ++rank) {
        if (rank >= first && rank < last) keep |= u & (0u - u);
      }
      m0 &= keep, m1 &= keep;
    }
  };

  if (warp >= kGatherWarp0 && warp < kEpilogueWarp1) {
    // ---------------------------------------------------------------- gather
    const int piece = lane & 7;
    const int g = (warp - kGatherWarp0) * 4 + (lane >> 3);  // 0..31: rows g, g+32, ... of the block
    // shared-memory offset of this thread's 16 bytes for each of its 8 rows (j < 4: half 0)
    uint32_t dst_off[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = g + 32 * (j & 3);
      dst_off[j] = (j >> 2) * kATileBytes + r * 128 + ((piece ^ (r & 7)) << 4);
    }
    auto load_rows = [&](uint32_t mblk, uint32_t (&rows)[8]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t r = mblk * kBlockM + (j >> 2) * kTileM + g + 32 * (j & 3);
        rows[j] = r < p.n ? static_cast<uint32_t>(__ldg(&p.sorted_idx[r])) : kInvalid;
      }
    };
    auto load_idx = [&](const uint32_t (&rows)[8], int v, uint32_t m0, uint32_t m1, uint32_t (&idx)[8]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool need = ((j < 4 ? m0 : m1) >> v) & 1u;
        idx[j] = (need && rows[j] != kInvalid) ? __ldg(&p.nbr[size_t(rows[j]) * V + v]) : kInvalid;
      }
    };
    // ring position of the next stage and its phase bit, advanced by hand: a division by the runtime stage count
    // in this loop costs several XU-pipe instructions per stage and starves the epilogue's conversions
    uint32_t s = 0, ph = 0;
    uint32_t rows[8], nrows[8], idx[8], nidx[8];
    uint32_t m0 = 0, m1 = 0, nm0 = 0, nm1 = 0;
    uint32_t mblk = 0, ntile = 0;
    const bool publisher = warp == kGatherWarp0 && lane == 0;
    uint32_t pub_block = 0, pub_ntile = 0;  // pub_block turns `none` once the tickets are used up
    if (publisher) publish_work(0, pub_block, pub_ntile);
    bool has_work = work_of(0, mblk, ntile, false);
    if (has_work) {
      masks_of(mblk, ntile, m0, m1);
      load_rows(mblk, rows);
      if (m0 | m1) load_idx(rows, __ffs(m0 | m1) - 1, m0, m1, nidx);
    }
    for (uint32_t pass = 0; has_work; ++pass) {
      // The next work item is claimed late -- when at most one more offset of the current block is left to
      // gather -- so that near the end of the launch no CTA sits on a block while another SM is already idle;
      // its rows and masks then arrive while the last offsets are gathered.
      uint32_t mblk_n = 0, ntile_n = 0;
      bool has_next = false, claimed = false;
      auto claim_next = [&]() {
        if (publisher) publish_work(pass + 1, pub_block, pub_ntile);
        has_next = work_of(pass + 1, mblk_n, ntile_n, false);
        if (has_next) {
          masks_of(mblk_n, ntile_n, nm0, nm1);
          load_rows(mblk_n, nrows);
        }
        claimed = true;
      };
      uint32_t un = m0 | m1;
      while (un) {
        const int v = __ffs(un) - 1;
        un &= un - 1;
#pragma unroll
        for (int j = 0; j < 8; ++j) idx[j] = nidx[j];
        if (!claimed && (un & (un - 1)) == 0u) claim_next();
        // neighbour indices one offset ahead (or the first offset of the next block)
        if (un) {
          load_idx(rows, __ffs(un) - 1, m0, m1, nidx);
        } else if (has_next && (nm0 | nm1)) {
          load_idx(nrows, __ffs(nm0 | nm1) - 1, nm0, nm1, nidx);
        }
        const bool need0 = (m0 >> v) & 1u, need1 = (m1 >> v) & 1u;
        const char* src[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) src[j] = p.x + size_t(idx[j] != kInvalid ? idx[j] : 0u) * p.row_bytes + piece * 16;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag);
          const uint32_t a_base = smem_u32(stages + size_t(s) * stage_bytes);
          const bool col_ok = kb * 128 + piece * 16 < p.row_bytes;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j < 4 ? need0 : need1) {
              const bool ok = col_ok && idx[j] != kInvalid;
              cp_async_16(a_base + dst_off[j], src[j] + kb * 128, ok ? 16u : 0u);
            }
          }
          cp_async_arrive(&ctl->full[s]);
          if (++s == static_cast<uint32_t>(S)) s = 0, ph ^= 1;
        }
      }
      if (!claimed) {  // a block without any offset (rows with no neighbour at all)
        claim_next();
        if (has_next && (nm0 | nm1)) load_idx(nrows, __ffs(nm0 | nm1) - 1, nm0, nm1, nidx);
      }
      m0 = nm0, m1 = nm1;
#pragma unroll
      for (int j = 0; j < 8; ++j) rows[j] = nrows[j];
      has_work = has_next;
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------ weight TMA
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      uint32_t mblk = 0, ntile = 0;
      for (uint32_t pass = 0; work_of(pass, mblk, ntile, true); ++pass) {
        const int n0 = static_cast<int>(tile_of(ntile)) * p.bn;
        uint32_t m0, m1;
        masks_of(mblk, ntile, m0, m1);
        uint32_t un = m0 | m1;
        while (un) {
          const int v = __ffs(un) - 1;
          un &= un - 1;
          const int wv = (p.flip & 1) ? V - 1 - v : v;
          for (int kb = 0; kb < p.num_kb; ++kb) {
            mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag);
            mbar_arrive_expect_tx(&ctl->full[s], static_cast<uint32_t>(p.bn) * 128u);
            const uint32_t b_dst = smem_u32(stages + size_t(s) * stage_bytes + 2 * kATileBytes);
            if (p.flip & 2) {
              // MN-major weights (dgrad of 16-bit types reads the weight as stored, [Co][V][Ci]): rows of the stage are
              // reduction channels, 128 bytes = 64 output channels per row, one 8 KB chunk per 64 output channels
              for (int c = 0; c < p.bn / 64; ++c) tma_load_3d(b_dst + c * 8192, &tmap_w, &ctl->full[s], n0 + c * 64, wv, kb * 64);
            } else {
              tma_load_3d(b_dst, &tmap_w, &ctl->full[s], kb * (128 / kElem), wv, n0);
            }
            if (++s == static_cast<uint32_t>(S)) s = 0, ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------- MMA
    if (lane == 0) {
      uint32_t s = 0, ph = 0, item = 0;
      uint32_t set = 0, set_ph = 0;  // accumulator set of the item and its phase bit
      uint32_t mblk = 0, ntile = 0;
      for (; work_of(item, mblk, ntile, true); ++item) {
        uint32_t m0, m1;
        masks_of(mblk, ntile, m0, m1);
        const uint32_t acc_tmem = tmem_base + set * 2 * p.bn;
        // the epilogue must have drained this accumulator pair
        mbar_wait(&ctl->acc_empty[set], set_ph ^ 1, abort_flag);
        tc_fence_after_sync();
        uint32_t acc0 = 0, acc1 = 0;
        uint32_t un = m0 | m1;
        while (un) {
          const int v = __ffs(un) - 1;
          un &= un - 1;
          const bool need0 = (m0 >> v) & 1u, need1 = (m1 >> v) & 1u;
          for (int kb = 0; kb < p.num_kb; ++kb) {
            mbar_wait(&ctl->full[s], ph, abort_flag);
            // the activation rows were written by cp.async (generic proxy), the MMA reads them through the async proxy
            fence_proxy_async_smem();
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(stages + size_t(s) * stage_bytes);
            const uint64_t da0 = make_smem_desc(a_addr, 16, 1024);
            const uint64_t da1 = make_smem_desc(a_addr + kATileBytes, 16, 1024);
            // K-major weights: a k-step is 32 bytes along the row; MN-major: 16 rows of 128 bytes, chunks 8 KB apart
            const bool b_mn = (p.flip & 2) != 0;
            const uint64_t db = make_smem_desc(a_addr + 2 * kATileBytes, b_mn ? 8192 : 16, 1024);
            const uint32_t b_step = b_mn ? 128u : 2u;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              if (kb * 128 + k4 * 32 < p.row_bytes) {
                if (need0) {
                  umma_ss<kTF32>(acc_tmem, da0 + uint64_t(k4 * 2), db + uint64_t(k4 * b_step), p.idesc, acc0);
                  acc0 = 1;
                }
                if (need1) {
                  umma_ss<kTF32>(acc_tmem + p.bn, da1 + uint64_t(k4 * 2), db + uint64_t(k4 * b_step), p.idesc, acc1);
                  acc1 = 1;
                }
              }
            }
            umma_commit(&ctl->empty[s]);
            if (++s == static_cast<uint32_t>(S)) s = 0, ph ^= 1;
          }
        }
        umma_commit(&ctl->acc_full[set]);
        if (++set == static_cast<uint32_t>(p.acc_sets)) set = 0, set_ph ^= 1;
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue
    // Thread `lane` of warp w owns accumulator row 32w + lane.  64 columns at a
    // time go through a per-warp staging buffer [32 rows][128 or 256 bytes] whose
    // 16-byte pieces are XOR-swizzled, and come back so that eight (fp32: sixteen)
    // consecutive lanes hold one row's contiguous bytes.
    // Two warps share each quarter of the accumulator rows (a warp reads TMEM lanes 32 * (warp % 4) ...): the
    // first group takes the even 64-column passes, the second the odd ones.
    const int quarter = warp & 3;
    const int group = warp >= kEpilogueWarp1 ? 1 : 0;
    uint8_t* stage_out = smem + kCtrlBytes + size_t(S) * stage_bytes + (group * 4 + quarter) * 4096;
    constexpr int kColsPerPass = 4096 / 32 / kElemOut;  // 64 columns of 16-bit, 32 columns of fp32: 128 bytes per row
    constexpr int kChunksPerPass = kColsPerPass / 32 > 0 ? kColsPerPass / 32 : 1;
    uint32_t item = 0;
    uint32_t set = 0, set_ph = 0;
    uint32_t mblk = 0, ntile = 0;
    for (; work_of(item, mblk, ntile, false); ++item) {
      const int n0 = static_cast<int>(tile_of(ntile)) * p.bn;
      uint32_t m0, m1;
      masks_of(mblk, ntile, m0, m1);
      // split-K: this item's slab [n, nout] of fp32 partial sums
      char* const out_base = kSplit ? p.out + size_t(split_of(ntile)) * p.n * p.nout * 4 : p.out;
      uint32_t sr[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t r = mblk * kBlockM + h * kTileM + quarter * 32 + lane;
        sr[h] = r < p.n ? static_cast<uint32_t>(__ldg(&p.sorted_idx[r])) : kInvalid;
      }
      mbar_wait(&ctl->acc_full[set], set_ph, abort_flag);
      tc_fence_after_sync();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const bool has_acc = (h == 0 ? m0 : m1) != 0u;  // a half without offsets holds no rows
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + set * 2 * p.bn + h * p.bn;
        for (int c0 = group * kColsPerPass; c0 < p.bn; c0 += 2 * kColsPerPass) {
          uint32_t acc[kChunksPerPass][32];
          if (has_acc) {
#pragma unroll
            for (int cc = 0; cc < kChunksPerPass; ++cc) tmem_ld_32x32(t_addr + c0 + cc * 32, acc[cc]);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int cc = 0; cc < kChunksPerPass; ++cc)
#pragma unroll
              for (int i = 0; i < 32; ++i) acc[cc][i] = 0u;
          }
#pragma unroll
          for (int cc = 0; cc < kChunksPerPass; ++cc)
            stage_row_chunk<kOutDtype>(stage_out, lane, cc, acc[cc], kSplit ? nullptr : p.bias, n0 + c0 + cc * 32, p.nout);
          __syncwarp();
          {
            // 128 bytes per row: lane -> (row = 4 i + lane / 8, piece = lane % 8)
            const int piece = lane & 7;
            const int col = n0 + c0 + piece * (16 / kElemOut);
            const bool col_ok = col < p.nout;
            const uint8_t* src = stage_out + (lane >> 3) * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = i * 4 + (lane >> 3);
              const uint32_t orow = __shfl_sync(0xffffffffu, sr[h], row);  // output row of staging row `row`
              const uint4 val = *reinterpret_cast<const uint4*>(src + i * 512 + ((piece ^ (row & 7)) << 4));
              if constexpr (kFused) {
                if (orow != kInvalid && col_ok) {
                  const size_t byte_off = (size_t(orow) * p.nout + col) * kElemOut;
                  *reinterpret_cast<uint4*>(out_base + byte_off) = fuse_piece<kDtype>(val, fe.act, fe.residual, fe.preact, byte_off);
                }
              } else {
                if (orow != kInvalid && col_ok) *reinterpret_cast<uint4*>(out_base + (size_t(orow) * p.nout + col) * kElemOut) = val;
              }
            }
          }
          __syncwarp();
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[set]);
      if (++set == static_cast<uint32_t>(p.acc_sets)) set = 0, set_ph ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512u);
  }
  if (tid == 0 && ctl->abort_flag) report(p.status, FGB_S_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ block schedule
// order[] = row blocks (pairs of 128-row tiles) sorted by descending cost, the
// cost of a block being the number of (tile, offset) products it runs.  One CTA;
// a counting sort over the 65 possible costs.  Blocks of equal cost may come out
// in any order: the order only decides which SM computes a block, never a result.
__global__ void __launch_bounds__(1024) block_schedule_kernel(const uint32_t* __restrict__ masks, uint32_t num_tiles, uint32_t nb,
                                                              uint32_t* __restrict__ order) {
  __shared__ uint32_t s_count[65];
  __shared__ uint32_t s_start[65];
  const int t = threadIdx.x;
  if (t < 65) s_count[t] = 0;
  __syncthreads();
  auto cost_of = [&](uint32_t b) {
    const uint32_t t0 = 2 * b;
    return __popc(__ldg(&masks[t0])) + (t0 + 1 < num_tiles ? __popc(__ldg(&masks[t0 + 1])) : 0);
  };
  for (uint32_t b = t; b < nb; b += 1024) atomicAdd(&s_count[cost_of(b)], 1u);
  __syncthreads();
  if (t == 0) {
    uint32_t acc = 0;
    for (int c = 64; c >= 0; --c) {
      s_start[c] = acc;
      acc += s_count[c];
    }
  }
  __syncthreads();
  for (uint32_t b = t; b < nb; b += 1024) order[atomicAdd(&s_start[cost_of(b)], 1u)] = b;
}

// ------------------------------------------------------------------ weight re-layout for dgrad
// dst[ci, v, co] = src[co, v, ci]; 32x32 tiles through shared memory
template <typename T>
__global__ void __launch_bounds__(256) weight_transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int Co, int V, int Ci) {
  __shared__ T tile[32][33];
  chain_release();  // the conv kernel that reads dst is launched chained
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

// 3-D map over the weight as stored, w[Co][V][Ci] of 16-bit elements, for dgrad: box = 64 input channels (128 bytes) x 1
// offset x 64 output channels -- one MN-major chunk of a stage (rows = reduction channels), 128B swizzle
int make_weight_tmap_mn(CUtensorMap* map, const void* w, int Co, int V, int Ci, int dtype) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return FGB_E_DRIVER;
  const CUtensorMapDataType dt = dtype == FGB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t dims[3] = {cuuint64_t(Ci), cuuint64_t(V), cuuint64_t(Co)};
  cuuint64_t strides[2] = {cuuint64_t(Ci) * 2, cuuint64_t(V) * Ci * 2};
  cuuint32_t box[3] = {64u, 1u, 64u};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FGB_OK : FGB_E_DRIVER;
}

// 2-D map over rows[n_rows][row_elems] of 16-bit elements; box = 128 bytes of one row, 128B swizzle (the box TMA
// tile::gather4 wants: it takes four row coordinates per instruction)
int make_rows_tmap(CUtensorMap* map, const void* rows, int64_t n_rows, int row_elems) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return FGB_E_DRIVER;
  cuuint64_t dims[2] = {cuuint64_t(row_elems), cuuint64_t(n_rows)};
  cuuint64_t strides[1] = {cuuint64_t(row_elems) * 2};
  cuuint32_t box[2] = {64u, 1u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(rows), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FGB_OK : FGB_E_DRIVER;
}

static int pick_bn(int nout) {
  int bn = 32;
  while (bn < nout && bn < 256) bn <<= 1;
  return bn;
}

// Upper bound on the CTAs (= SMs) of the persistent conv kernels; 0 = all.  A caller that has a collective running
// beside a conv kernel leaves it some SMs this way: the conv CTAs fill their SMs completely (shared memory and
// registers), so a kernel launched beside them would otherwise wait for the first of them to finish.
static std::atomic<int> g_cta_limit{0};

template <int kDtype, int kMode>
static int launch_igemm_variant(const CUtensorMap& tmap, const IgemmParams& p, const FusedEpilogue& fe, cudaStream_t s) {
  const size_t smem = 1024 + kCtrlBytes + size_t(p.stages) * (2 * kATileBytes + p.bn * 128) + kStoreStageBytes;
  static PerDeviceTable configured;  // the attribute belongs to (kernel instance, device)
  const int rc = ensure_dynamic_smem(configured, subm_igemm_kernel<kDtype, kMode>, smem);
  if (rc != FGB_OK) return rc;
  const int64_t work = int64_t(p.num_blocks) * p.items_per_block;
  int ctas = device_sm_count();
  const int limit = g_cta_limit.load(std::memory_order_relaxed);
  if (limit > 0 && limit < ctas) ctas = limit;
  const unsigned grid = static_cast<unsigned>(work < ctas ? work : ctas);
  const cudaError_t e = launch_chained(subm_igemm_kernel<kDtype, kMode>, dim3(grid), dim3(kIgemmThreads), smem, s, tmap, p, fe);
  return e != cudaSuccess ? cuda_status(e) : launch_status();
}

// the plain kernel carries no trace of the fused epilogue (its register allocation is the tuned one)
template <int kDtype>
static int launch_igemm(const CUtensorMap& tmap, const IgemmParams& p, const FusedEpilogue& fe, cudaStream_t s) {
  if (p.splits > 1) return launch_igemm_variant<kDtype, kSplitK>(tmap, p, fe, s);
  if (fe.act != FGB_ACT_NONE || fe.residual != nullptr || fe.preact != nullptr) return launch_igemm_variant<kDtype, kFusedEp>(tmap, p, fe, s);
  return launch_igemm_variant<kDtype, kPlain>(tmap, p, fe, s);
}

// ------------------------------------------------------------------ split-K for small inputs
// A launch with fewer work items (row blocks x column tiles) than SMs leaves most of the device idle: each item walks
// up to V offsets x kc/64 slices on its own.  Then every item is cut into `splits` shares of its offsets, the shares
// run as separate work items into fp32 slabs, and a second kernel adds the slabs in a fixed order, adds the bias and
// converts.  (The reference splits the same way when tiles * SPLITK < number of SMs:
// sparse_submanifold_conv_fwd_masked_implicit_gemm_splitk.py:109-121.)
static std::atomic<int> g_dgrad_relayout{0};  // 1 = dgrad always works on the re-laid-out copy of the weight (measurement / test knob)
static std::atomic<int> g_force_splits{0};  // 0 = by the rule below, 1 = never split, k = k shares (capped at V)

int igemm_splits(int64_t n, int nout, int V) {
  if (n <= 0) return 1;
  const int forced = g_force_splits.load(std::memory_order_relaxed);
  if (forced > 0) return forced < V ? forced : V;
  const int64_t items = ceil_div(n, kBlockM) * ceil_div(nout, pick_bn(nout));
  const int64_t sms = device_sm_count();
  if (items * 2 > sms) return 1;
  int64_t sp = sms / items;
  if (sp > V) sp = V;
  return static_cast<int>(sp < 1 ? 1 : sp);
}
int64_t igemm_partial_bytes(int64_t n, int nout, int V) {
  const int sp = igemm_splits(n, nout, V);
  return sp > 1 ? align256(int64_t(sp) * n * nout * 4) : 0;
}

// out[r, c] = sum_s partial[s, r, c] (+ bias[c]) in split order, converted to T
template <typename T>
__global__ void __launch_bounds__(256) splitk_rows_reduce_kernel(const float* __restrict__ partial, int splits, int64_t elems, int nout,
                                                                 const T* __restrict__ bias, T* __restrict__ out) {
  const int64_t e = (blockIdx.x * int64_t(256) + threadIdx.x) * 4;
  if (e >= elems) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp = 0; sp < splits; ++sp) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(partial + size_t(sp) * elems + e));
    acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
  }
  float v[4] = {acc.x, acc.y, acc.z, acc.w};
  const int c = static_cast<int>(e % nout);  // nout is a multiple of 4: the four values share a row
  T o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // same roundings as the unsplit epilogue: 16-bit types round the sum, then add the bias in the type
    if constexpr (std::is_same<T, float>::value) o[i] = v[i] + (bias ? bias[c + i] : 0.f);
    else o[i] = bias ? static_cast<T>(static_cast<T>(v[i]) + bias[c + i]) : static_cast<T>(v[i]);
  }
  if constexpr (std::is_same<T, float>::value) *reinterpret_cast<float4*>(out + e) = make_float4(o[0], o[1], o[2], o[3]);
  else *reinterpret_cast<uint2*>(out + e) = *reinterpret_cast<const uint2*>(o);
}

// x [n, kc] gathered through nbr; w [nout, V, kc]; out [n, nout]
int run_igemm(const void* x, const void* w, const void* bias, const uint32_t* nbr, const int64_t* sorted_idx,
              const uint32_t* tile_masks, const uint32_t* block_order, uint32_t* ticket, void* out, int64_t n, int kc, int nout, int V, int dtype, int flip, int32_t* status,
              cudaStream_t s, float* partial = nullptr, int act = FGB_ACT_NONE, const void* residual = nullptr, void* preact = nullptr,
              bool ticket_zeroed = false) {
  const int eb = elem_bytes(dtype);
  if (eb == 0 || dtype == FGB_F32_IEEE) return FGB_E_DTYPE;  // callers expand fp32-accurate mode to TF32 operands
  if (n < 0 || n >= (int64_t(1) << 32) - 1 || kc <= 0 || nout <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!x || !w || !nbr || !sorted_idx || !tile_masks || !out) return FGB_E_NULL;
  if ((kc * eb) % 16 || (nout * eb) % 16) return FGB_E_ALIGN;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(preact)) & 15)
    return FGB_E_ALIGN;
  if (act != FGB_ACT_NONE && act != FGB_ACT_SILU) return FGB_E_SIZE;
  FusedEpilogue fe;
  fe.residual = static_cast<const char*>(residual);
  fe.preact = static_cast<char*>(preact);
  fe.act = act;
  IgemmParams p;
  p.x = static_cast<const char*>(x);
  p.bias = bias;
  p.nbr = nbr;
  p.sorted_idx = sorted_idx;
  p.tile_masks = tile_masks;
  p.block_order = block_order;
  p.ticket = ticket;
  p.out = static_cast<char*>(out);
  p.n = static_cast<uint32_t>(n);
  p.kc = kc;
  p.nout = nout;
  p.V = V;
  p.bn = pick_bn(nout);
  p.n_tiles_n = static_cast<int>(ceil_div(nout, p.bn));
  // split-K when the caller gave room for the partial sums and the plain epilogue is asked for
  const bool fused = act != FGB_ACT_NONE || residual != nullptr || preact != nullptr;
  p.splits = (partial != nullptr && !fused) ? igemm_splits(n, nout, V) : 1;
  p.items_per_block = p.n_tiles_n * p.splits;
  if (p.splits > 1) p.out = reinterpret_cast<char*>(partial);
  p.row_bytes = kc * eb;
  p.num_kb = static_cast<int>(ceil_div(p.row_bytes, 128));
  p.flip = flip;
  p.num_tiles = static_cast<uint32_t>(ceil_div(n, kTileM));
  p.num_blocks = static_cast<uint32_t>(ceil_div(n, kBlockM));
  const int stage_bytes = 2 * kATileBytes + p.bn * 128;
  p.stages = (kSmemBudget - 1024 - kCtrlBytes - kStoreStageBytes) / stage_bytes;
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  p.acc_sets = 2 * p.bn * 2 <= 512 ? 2 : 1;
  const uint32_t fmt = dtype == FGB_F16 ? kFmtF16 : dtype == FGB_BF16 ? kFmtBF16 : kFmtTF32;
  const bool b_mn = (flip & 2) != 0;  // the weight operand as stored for the other direction: w [kc, V, nout]
  p.idesc = make_idesc(fmt, kTileM, p.bn, 0, b_mn ? 1 : 0);
  p.status = status;
  if (!ticket) return FGB_E_NULL;
  // the work counter starts at zero; a caller that launches kernels of its own right before this one zeroes it ahead of
  // them, so that the conv kernel follows a kernel in the stream and its chained launch takes effect
  int rc = ticket_zeroed ? FGB_OK : cuda_status(cudaMemsetAsync(ticket, 0, sizeof(uint32_t), s));
  if (rc != FGB_OK) return rc;
  CUtensorMap tmap;
  rc = b_mn ? make_weight_tmap_mn(&tmap, w, kc, V, nout, dtype) : make_weight_tmap(&tmap, w, nout, V, kc, p.bn, dtype);
  if (rc != FGB_OK) return rc;
  switch (dtype) {
    case FGB_F16:
      rc = launch_igemm<FGB_F16>(tmap, p, fe, s);
      break;
    case FGB_BF16:
      rc = launch_igemm<FGB_BF16>(tmap, p, fe, s);
      break;
    default:
      rc = launch_igemm<FGB_F32_TF32>(tmap, p, fe, s);
  }
  if (rc != FGB_OK || p.splits == 1) return rc;
  const int64_t elems = n * nout;
  const unsigned grid = static_cast<unsigned>(ceil_div(elems, 1024));
  switch (dtype) {
    case FGB_F16:
      splitk_rows_reduce_kernel<__half><<<grid, 256, 0, s>>>(partial, p.splits, elems, nout, static_cast<const __half*>(bias), static_cast<__half*>(out));
      break;
    case FGB_BF16:
      splitk_rows_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(partial, p.splits, elems, nout, static_cast<const __nv_bfloat16*>(bias),
                                                                    static_cast<__nv_bfloat16*>(out));
      break;
    default:
      splitk_rows_reduce_kernel<float><<<grid, 256, 0, s>>>(partial, p.splits, elems, nout, static_cast<const float*>(bias), static_cast<float*>(out));
  }
  return launch_status();
}

}  // namespace fgb

extern "C" int fgb_conv_tile_rows(void) { return fgb::kTileM; }

extern "C" int fgb_conv_set_cta_limit(int max_ctas) {
  if (max_ctas < 0) return FGB_E_SIZE;
  return fgb::g_cta_limit.exchange(max_ctas, std::memory_order_relaxed);
}

extern "C" int fgb_conv_set_splitk(int splits) {
  if (splits < 0 || splits > 32) return FGB_E_SIZE;
  return fgb::g_force_splits.exchange(splits, std::memory_order_relaxed);
}

extern "C" int fgb_conv_set_dgrad_relayout(int on) {
  if (on != 0 && on != 1) return FGB_E_SIZE;
  return fgb::g_dgrad_relayout.exchange(on, std::memory_order_relaxed);
}

extern "C" int fgb_conv_block_schedule(const uint32_t* tile_masks, int64_t num_tiles, uint32_t* block_order, void* stream) {
  using namespace fgb;
  if (num_tiles < 0 || num_tiles > 0x7FFFFFFF) return FGB_E_SIZE;
  if (num_tiles == 0) return FGB_OK;
  if (!tile_masks || !block_order) return FGB_E_NULL;
  const uint32_t nb = static_cast<uint32_t>(ceil_div(num_tiles, 2));
  block_schedule_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(tile_masks, static_cast<uint32_t>(num_tiles), nb, block_order);
  return launch_status();
}

// Every conv workspace starts with a 256-byte header whose first word is the
// ticket counter of the persistent kernel; the pass-specific scratch follows.
constexpr int64_t kWsHeader = 256;

namespace fgb {

// n rows of the map / of `out`; n_src rows of `feats` (equal for a submanifold conv)
static int fprop_impl(const void* feats, const void* weight, const void* bias, const uint32_t* neighbor_map, const int64_t* sorted_idx,
                      const uint32_t* tile_masks, const uint32_t* block_order, void* out, int64_t n, int64_t n_src, int Ci, int Co, int V,
                      int dtype, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream, int act = FGB_ACT_NONE,
                      const void* residual = nullptr, void* preact = nullptr) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n < 0 || n_src < 0 || Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!workspace) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FGB_E_ALIGN;
  if (workspace_bytes < kWsHeader) return FGB_E_WORKSPACE;
  uint32_t* ticket = static_cast<uint32_t*>(workspace);
  char* scratch = static_cast<char*>(workspace) + kWsHeader;
  const bool fused = act != FGB_ACT_NONE || residual != nullptr || preact != nullptr;  // the fused epilogue is never split
  const int64_t part_bytes = fused ? 0 : igemm_partial_bytes(n, Co, V);
  if (dtype != FGB_F32_IEEE) {
    if (workspace_bytes < kWsHeader + part_bytes) return FGB_E_WORKSPACE;
    return run_igemm(feats, weight, bias, neighbor_map, sorted_idx, tile_masks, block_order, ticket, out, n, Ci, Co, V, dtype, 0, status, s,
                     part_bytes ? reinterpret_cast<float*>(scratch) : nullptr, act, residual, preact);
  }
  // fp32-accurate: one TF32 run over the tripled channel dimension
  if (!feats || !weight) return FGB_E_NULL;
  const int64_t x_bytes = align256(n_src * 3 * Ci * 4), w_bytes = align256(int64_t(Co) * V * 3 * Ci * 4);
  if (workspace_bytes < kWsHeader + x_bytes + w_bytes + part_bytes) return FGB_E_WORKSPACE;
  float* x3 = reinterpret_cast<float*>(scratch);
  float* w3 = reinterpret_cast<float*>(scratch + x_bytes);
  float* part = part_bytes ? reinterpret_cast<float*>(scratch + x_bytes + w_bytes) : nullptr;
  int rc = FGB_OK;
  if (n_src > 0) rc = launch_split3(static_cast<const float*>(feats), x3, n_src, Ci, kSplitActivations, s);
  if (rc != FGB_OK) return rc;
  rc = launch_split3(static_cast<const float*>(weight), w3, int64_t(Co) * V, Ci, kSplitWeights, s);
  if (rc != FGB_OK) return rc;
  return run_igemm(x3, w3, bias, neighbor_map, sorted_idx, tile_masks, block_order, ticket, out, n, 3 * Ci, Co, V, FGB_F32_TF32, 0, status, s,
                   part, act, residual, preact);
}

}  // namespace fgb

extern "C" int fgb_subm_conv_fprop(const void* feats, const void* weight, const void* bias, const uint32_t* neighbor_map,
                                   const int64_t* sorted_idx, const uint32_t* tile_masks, const uint32_t* block_order, void* out,
                                   int64_t n, int Ci, int Co, int V, int dtype, void* workspace, int64_t workspace_bytes,
                                   int32_t* status, void* stream) {
  return fgb::fprop_impl(feats, weight, bias, neighbor_map, sorted_idx, tile_masks, block_order, out, n, n, Ci, Co, V, dtype, workspace,
                         workspace_bytes, status, stream);
}

extern "C" int fgb_sparse_conv_fprop(const void* feats, const void* weight, const void* bias, const uint32_t* neighbor_map,
                                     const int64_t* sorted_idx, const uint32_t* tile_masks, const uint32_t* block_order, void* out,
                                     int64_t n_out, int64_t n_in, int Ci, int Co, int V, int dtype, void* workspace,
                                     int64_t workspace_bytes, int32_t* status, void* stream) {
  return fgb::fprop_impl(feats, weight, bias, neighbor_map, sorted_idx, tile_masks, block_order, out, n_out, n_in, Ci, Co, V, dtype,
                         workspace, workspace_bytes, status, stream);
}

extern "C" int fgb_subm_conv_fprop_fused(const void* feats, const void* weight, const void* bias, const void* residual,
                                         const uint32_t* neighbor_map, const int64_t* sorted_idx, const uint32_t* tile_masks,
                                         const uint32_t* block_order, void* out, void* preact_out, int64_t n, int Ci, int Co, int V,
                                         int dtype, int activation, void* workspace, int64_t workspace_bytes, int32_t* status,
                                         void* stream) {
  if (activation != FGB_ACT_NONE && activation != FGB_ACT_SILU) return FGB_E_SIZE;
  return fgb::fprop_impl(feats, weight, bias, neighbor_map, sorted_idx, tile_masks, block_order, out, n, n, Ci, Co, V, dtype, workspace,
                         workspace_bytes, status, stream, activation, residual, preact_out);
}

namespace fgb {

// n rows of the map / of `grad_feats`; n_src rows of `grad_out`; mirror = the map is the forward map of a submanifold
// conv, whose row for offset v is the backward map's row for offset V-1-v
static int dgrad_impl(const void* grad_out, const void* weight, const uint32_t* neighbor_map, const int64_t* sorted_idx,
                      const uint32_t* tile_masks, const uint32_t* block_order, void* grad_feats, int64_t n, int64_t n_src, int Ci, int Co,
                      int V, int dtype, int mirror, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  const int eb = elem_bytes(dtype);
  if (eb == 0) return FGB_E_DTYPE;
  if (n < 0 || n_src < 0 || Ci <= 0 || Co <= 0 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!weight || !workspace) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FGB_E_ALIGN;
  const int64_t wt_bytes = align256(int64_t(Ci) * V * Co * eb);
  const bool ieee = dtype == FGB_F32_IEEE;
  const int64_t w3_bytes = ieee ? align256(int64_t(Ci) * V * 3 * Co * 4) : 0;
  const int64_t g3_bytes = ieee ? align256(n_src * 3 * Co * 4) : 0;
  const int64_t part_bytes = igemm_partial_bytes(n, Ci, V);
  if (workspace_bytes < kWsHeader + wt_bytes + w3_bytes + g3_bytes + part_bytes) return FGB_E_WORKSPACE;
  float* part = part_bytes ? reinterpret_cast<float*>(static_cast<char*>(workspace) + kWsHeader + wt_bytes + w3_bytes + g3_bytes) : nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* ticket = static_cast<uint32_t*>(workspace);
  char* wt = static_cast<char*>(workspace) + kWsHeader;
  // 16-bit types read the weight as it is stored, [Co][V][Ci], as an MN-major operand (rows = reduction channels): no
  // re-layout pass.  Column tiles narrower than one 64-channel chunk, and the 32-bit types (whose MN-major layout TMA
  // does not produce), go through the re-laid-out copy.
  if (eb == 2 && !g_dgrad_relayout.load(std::memory_order_relaxed) && pick_bn(Ci) % 64 == 0)
    return run_igemm(grad_out, weight, nullptr, neighbor_map, sorted_idx, tile_masks, block_order, ticket, grad_feats, n, Co, Ci, V, dtype,
                     mirror | 2, status, s, part);
  dim3 grid(static_cast<unsigned>(ceil_div(Ci, 32)), static_cast<unsigned>(ceil_div(Co, 32)), V);
  {
    const cudaError_t e = cudaMemsetAsync(ticket, 0, sizeof(uint32_t), s);  // ahead of the re-layout: see run_igemm
    if (e != cudaSuccess) return cuda_status(e);
  }
  if (eb == 2)
    weight_transpose_kernel<uint16_t><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(weight), reinterpret_cast<uint16_t*>(wt), Co, V, Ci);
  else
    weight_transpose_kernel<uint32_t><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(weight), reinterpret_cast<uint32_t*>(wt), Co, V, Ci);
  int rc = launch_status();
  if (rc != FGB_OK) return rc;
  if (!ieee)
    return run_igemm(grad_out, wt, nullptr, neighbor_map, sorted_idx, tile_masks, block_order, ticket, grad_feats, n, Co, Ci, V, dtype,
                     mirror, status, s, part, FGB_ACT_NONE, nullptr, nullptr, true);
  if (!grad_out) return FGB_E_NULL;
  float* w3 = reinterpret_cast<float*>(wt + wt_bytes);
  float* g3 = reinterpret_cast<float*>(wt + wt_bytes + w3_bytes);
  rc = launch_split3(reinterpret_cast<const float*>(wt), w3, int64_t(Ci) * V, Co, kSplitWeights, s);
  if (rc != FGB_OK) return rc;
  if (n_src > 0) rc = launch_split3(static_cast<const float*>(grad_out), g3, n_src, Co, kSplitActivations, s);
  if (rc != FGB_OK) return rc;
  return run_igemm(g3, w3, nullptr, neighbor_map, sorted_idx, tile_masks, block_order, ticket, grad_feats, n, 3 * Co, Ci, V, FGB_F32_TF32,
                   mirror, status, s, part, FGB_ACT_NONE, nullptr, nullptr, true);
}

}  // namespace fgb

extern "C" int fgb_subm_conv_dgrad(const void* grad_out, const void* weight, const uint32_t* neighbor_map,
                                   const int64_t* sorted_idx, const uint32_t* tile_masks, const uint32_t* block_order,
                                   void* grad_feats, int64_t n, int Ci, int Co, int V, int dtype, void* workspace,
                                   int64_t workspace_bytes, int32_t* status, void* stream) {
  return fgb::dgrad_impl(grad_out, weight, neighbor_map, sorted_idx, tile_masks, block_order, grad_feats, n, n, Ci, Co, V, dtype, 1,
                         workspace, workspace_bytes, status, stream);
}

extern "C" int fgb_sparse_conv_dgrad(const void* grad_out, const void* weight, const uint32_t* neighbor_map_bwd,
                                     const int64_t* sorted_idx_bwd, const uint32_t* tile_masks_bwd, const uint32_t* block_order_bwd,
                                     void* grad_feats, int64_t n_in, int64_t n_out, int Ci, int Co, int V, int dtype, void* workspace,
                                     int64_t workspace_bytes, int32_t* status, void* stream) {
  return fgb::dgrad_impl(grad_out, weight, neighbor_map_bwd, sorted_idx_bwd, tile_masks_bwd, block_order_bwd, grad_feats, n_in, n_out, Ci,
                         Co, V, dtype, 0, workspace, workspace_bytes, status, stream);
}
