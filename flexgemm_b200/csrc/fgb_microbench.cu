// Pipeline microbenchmark: the operand traffic and the MMAs of one stage of the masked implicit GEMM, isolated from
// the conv kernel, to measure what one SM can sustain.  (No counterpart in the reference.)
//
// A stage is what fprop / dgrad move and compute per 64 input channels of one kernel offset at Ci = Co = 256, 16-bit:
//   * 32 KB of gathered activation rows: 256 rows x 128 bytes taken at random from an [n_rows, row_bytes] matrix, by
//     cp.async (16 bytes per thread, 256 threads) or by TMA tile::gather4 (4 rows per instruction, two warps);
//   * 32 KB of the dense operand by one TMA bulk copy from a small, L2-resident buffer (16 KB per CTA with CTA pairs);
//   * 8 MMAs 128 x 256 x 16 (two 128-row halves x four k-steps) on whatever the stage buffers hold.
// The streams run either independently (every stage buffer is freed as soon as it is full) or coupled like in the conv
// kernel: the MMA lane waits for a full stage, the producers wait for the commit of the MMAs that read a buffer.  With
// CTA pairs (tcgen05 cta_group::2) the leader CTA issues M = 256 MMAs over the rows of both CTAs; the peer's MMA lane
// relays "my operands of this stage have landed" to the leader's barrier.
//
// All waits are bounded (fgb_umma.cuh); a wait that gives up sets *status.
#include <cuda.h>

#include "fgb_common.cuh"
#include "fgb_device.cuh"
#include "fgb_umma.cuh"

namespace fgb {
namespace {

constexpr int kMbMaxStages = 6;
constexpr int kMbAChunk = 32 * 1024;   // gathered rows per stage and CTA
constexpr int kMbThreads = 352;        // warps 0-7 gather, 8 TMA lane, 9 consumer / relay, 10 MMA lane and TMEM owner

enum : int {
  kMbTma = 1, kMbGather = 2, kMbMma = 4, kMbCoupled = 8, kMbGather4 = 16, kMbPair = 32, kMbLean = 64,
  kMbM64 = 128,         // the MMAs are 64 x 256 x 16
  kMbStore = 256,       // instead of the gather: the epilogue's output stream, 32 KB per stage to random rows of `rows`,
                        // 16-byte stores that cover four 128-byte lines per warp instruction
  kMbStoreBulk128 = 512,   // ... as bulk async copies shared -> global of 128 bytes (one per row piece and lane)
  kMbStoreBulk512 = 1024,  // ... as bulk async copies of whole 512-byte rows
};

struct MbParams {
  const char* dense;
  unsigned long long dense_bytes;
  const char* rows;
  uint32_t n_rows;
  int row_bytes;
  int iters;
  int mode;
  int stages_a, stages_b;
  int b_chunk;  // 32 KB, 16 KB with CTA pairs
  int issue_delay;  // cycles the MMA lane idles before each stage's MMAs
  unsigned long long* counters;  // [8], written by CTA 0: MMA lane's cycles waiting for the dense / gathered operand,
                                 // number of such waits (2 values), total cycles of its loop
  int32_t* status;
};

struct MbSmem {
  uint64_t full_t[kMbMaxStages], full_g[kMbMaxStages], empty_t[kMbMaxStages], empty_g[kMbMaxStages], mma_bar[4];
  uint32_t abort_flag, tmem_base;
};

template <bool kCluster>
__device__ __forceinline__ bool mb_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if constexpr (kCluster) return mbar_wait_cluster(bar, parity, abort_flag);
  else return mbar_wait(bar, parity, abort_flag);
}
template <bool kCluster>
__device__ __forceinline__ void mb_timed_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned long long& cycles,
                                              unsigned long long& waits) {
  if (kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return;
  const long long t0 = clock64();
  mb_wait<kCluster>(bar, parity, abort_flag);
  cycles += static_cast<unsigned long long>(clock64() - t0);
  ++waits;
}
__device__ __forceinline__ void mb_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mb_gather4(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int col, const int (&r)[4]) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(col), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(smem_u32(bar))
      : "memory");
}

// kPair: launched as clusters of two CTAs
template <bool kPair>
__global__ void __launch_bounds__(kMbThreads, 1) microbench_kernel(const __grid_constant__ CUtensorMap tmap_rows, const MbParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  MbSmem* ctl = reinterpret_cast<MbSmem*>(smem);
  uint8_t* tbuf = smem + 1024;
  uint8_t* gbuf = tbuf + size_t(p.stages_b) * p.b_chunk;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mode = p.mode, SA = p.stages_a, SB = p.stages_b;
  const bool coupled = (mode & kMbCoupled) != 0;
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;
  const bool leader = rank == 0u;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  if (tid == 0) {
    for (int s = 0; s < SB; ++s) {
      mbar_init(&ctl->full_t[s], 1);
      mbar_init(&ctl->empty_t[s], 1);
    }
    for (int s = 0; s < SA; ++s) {
      // cp.async: every gather thread; gather4: one lane of each of the two warps; leader of a pair: + the peer's relay
      mbar_init(&ctl->full_g[s], ((mode & kMbGather4) ? 2 : 256) + ((kPair && leader) ? 1 : 0));
      mbar_init(&ctl->empty_g[s], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&ctl->mma_bar[i], 1);
    ctl->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 10) {
    if constexpr (kPair) {
      tmem_alloc_pair(&ctl->tmem_base, 512u);
    } else {
      tmem_alloc_dyn(&ctl->tmem_base, 512u);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < 8 && (mode & (kMbStore | kMbStoreBulk128 | kMbStoreBulk512))) {
    // ------------------------------------------------------------ output stream (what an epilogue writes)
    // Every warp owns 4 KB of the first gathered stage as its staging buffer and writes it out p.iters times: 32 KB per
    // "stage" and CTA.  The destination rows are random rows of `rows` (the benchmark's scratch).
    uint32_t state = blockIdx.x * 2654435761u + tid * 40503u + 777u;
    uint8_t* stage_out = gbuf + warp * 4096;
    char* out = const_cast<char*>(p.rows);
    const int pieces_per_row = p.row_bytes / 128;
    for (int it = 0; it < p.iters; ++it) {
      const int kb = it % pieces_per_row;
      if (mode & kMbStore) {
        // lane -> (row = 4 i + lane / 8, piece = lane % 8): eight lanes write one 128-byte line
        state = state * 1664525u + 1013904223u;
        const uint32_t my_row = (state >> 4) % p.n_rows;  // row of staging row `lane`
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = i * 4 + (lane >> 3), piece = lane & 7;
          const uint32_t orow = __shfl_sync(0xffffffffu, my_row, row);
          const uint4 val = *reinterpret_cast<const uint4*>(stage_out + row * 128 + ((piece ^ (row & 7)) << 4));
          *reinterpret_cast<uint4*>(out + size_t(orow) * p.row_bytes + kb * 128 + piece * 16) = val;
        }
      } else if (mode & kMbStoreBulk128) {
        state = state * 1664525u + 1013904223u;
        const uint32_t orow = (state >> 4) % p.n_rows;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 128;" ::"l"(out + size_t(orow) * p.row_bytes + kb * 128),
                     "r"(smem_u32(stage_out + lane * 128))
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        if ((it & 3) == 3) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      } else {
        // 4 KB per warp and stage = eight whole rows of 512 bytes: lanes 0-7 issue one copy each
        state = state * 1664525u + 1013904223u;
        const uint32_t orow = (state >> 4) % p.n_rows;
        if (lane < 8 && p.row_bytes >= 512)
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 512;" ::"l"(out + size_t(orow) * p.row_bytes),
                       "r"(smem_u32(stage_out + lane * 512))
                       : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        if ((it & 3) == 3) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else if (warp < 8) {
    // ------------------------------------------------------------ gathered operand
    if ((mode & kMbGather) && (mode & kMbGather4)) {
      if (warp < 2) {  // lane l of warp h: rows 4l .. 4l+3 of half h, 512 bytes per instruction
        uint32_t state = blockIdx.x * 2654435761u + tid * 40503u + 12345u;
        const int pieces_per_row = p.row_bytes / 128;
        uint32_t s = 0, ph = 0;
        for (int it = 0; it < p.iters; ++it) {
          mb_wait<kPair>(&ctl->empty_g[s], ph ^ 1, abort_flag);
          int r[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            state = state * 1664525u + 1013904223u;
            r[j] = static_cast<int>((state >> 4) % p.n_rows);
          }
          if (lane == 0) mbar_arrive_expect_tx(&ctl->full_g[s], 16384u);
          __syncwarp();
          // x = multiple of 64 16-bit elements: 128-byte aligned
          mb_gather4(smem_u32(gbuf + size_t(s) * kMbAChunk) + warp * 16384 + lane * 512, &tmap_rows, &ctl->full_g[s],
                     (it % pieces_per_row) * 64, r);
          if (++s == static_cast<uint32_t>(SA)) s = 0, ph ^= 1;
        }
      }
    } else if (mode & kMbGather) {
      uint32_t state = blockIdx.x * 2654435761u + (tid / 8) * 40503u + 12345u;
      const int piece = lane & 7;
      const int pieces_per_row = p.row_bytes / 128;
      uint32_t s = 0, ph = 0;
      for (int it = 0; it < p.iters; ++it) {
        mb_wait<kPair>(&ctl->empty_g[s], ph ^ 1, abort_flag);
        const uint32_t base = smem_u32(gbuf + size_t(s) * kMbAChunk);
        const int kb = it % pieces_per_row;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          state = state * 1664525u + 1013904223u;
          const uint32_t r = (state >> 4) % p.n_rows;
          cp_async_16(base + ((tid / 8) * 8 + j) * 128 + piece * 16, p.rows + size_t(r) * p.row_bytes + kb * 128 + piece * 16, 16u);
        }
        cp_async_arrive(&ctl->full_g[s]);
        if (++s == static_cast<uint32_t>(SA)) s = 0, ph ^= 1;
      }
    }
  } else if (warp == 8) {
    // --------------------------------------------------------------- dense operand
    if ((mode & kMbTma) && lane == 0) {
      uint32_t s = 0, ph = 0;
      size_t off = (size_t(blockIdx.x) * 7 * p.b_chunk) % p.dense_bytes;
      for (int it = 0; it < p.iters; ++it) {
        mb_wait<kPair>(&ctl->empty_t[s], ph ^ 1, abort_flag);
        mbar_arrive_expect_tx(&ctl->full_t[s], static_cast<uint32_t>(p.b_chunk));
        mb_bulk_load(smem_u32(tbuf + size_t(s) * p.b_chunk), p.dense + off, static_cast<uint32_t>(p.b_chunk), &ctl->full_t[s]);
        off += p.b_chunk;
        if (off + p.b_chunk > p.dense_bytes) off = 0;
        if (++s == static_cast<uint32_t>(SB)) s = 0, ph ^= 1;
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      if (kPair && !leader) {
        // relay: this CTA's operands of a stage have landed -> one arrival on the leader's barrier
        uint32_t s = 0, ph = 0, sb = 0, phb = 0;
        for (int it = 0; it < p.iters; ++it) {
          mb_wait<true>(&ctl->full_t[sb], phb, abort_flag);
          mb_wait<true>(&ctl->full_g[s], ph, abort_flag);
          fence_proxy_async_smem();
          mbar_arrive_cluster(cluster_map(smem_u32(&ctl->full_g[s]), 0));
          if (++s == static_cast<uint32_t>(SA)) s = 0, ph ^= 1;
          if (++sb == static_cast<uint32_t>(SB)) sb = 0, phb ^= 1;
        }
      } else if (!kPair && !coupled) {
        // independent streams: a full stage is free again at once
        uint32_t s = 0, ph = 0, sb = 0, phb = 0;
        for (int it = 0; it < p.iters; ++it) {
          if (mode & kMbTma) {
            mbar_wait(&ctl->full_t[sb], phb, abort_flag);
            mbar_arrive(&ctl->empty_t[sb]);
          }
          if (mode & kMbGather) {
            mbar_wait(&ctl->full_g[s], ph, abort_flag);
            mbar_arrive(&ctl->empty_g[s]);
          }
          if (++s == static_cast<uint32_t>(SA)) s = 0, ph ^= 1;
          if (++sb == static_cast<uint32_t>(SB)) sb = 0, phb ^= 1;
        }
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------------ MMA
    if (!kPair && (mode & kMbLean) && coupled && lane == 0) {
      // Lean MMA lane: the instructions between the last MMA of a stage and the first of the next are what the tensor
      // pipe cannot hide (it holds one MMA beyond the running one).  Descriptors advance by one add per stage, the next
      // stage's barriers are probed and the fences issued in the shadow of the current stage's last MMAs.
      const uint32_t idesc = make_idesc(kFmtF16, 128, 256, 0, 0);
      unsigned long long cyc_t = 0, n_t = 0, cyc_g = 0, n_g = 0;
      const long long t_begin = clock64();
      const uint64_t da_base = make_smem_desc(smem_u32(gbuf), 16, 1024), db_base = make_smem_desc(smem_u32(tbuf), 16, 1024);
      const bool use_t = (mode & kMbTma) != 0, use_g = (mode & kMbGather) != 0;
      uint32_t s = 0, ph = 0, sb = 0, phb = 0;
      if (use_t) mbar_wait(&ctl->full_t[0], 0, abort_flag);
      if (use_g) mbar_wait(&ctl->full_g[0], 0, abort_flag);
      fence_proxy_async_smem();
      tc_fence_after_sync();
      for (int it = 0; it < p.iters; ++it) {
        const uint64_t da0 = da_base + uint64_t(s * (kMbAChunk >> 4)), da1 = da0 + uint64_t(16384 >> 4);
        const uint64_t db = db_base + uint64_t(sb * (32768 >> 4));
        uint32_t ns = s + 1, nph = ph, nsb = sb + 1, nphb = phb;
        if (ns == static_cast<uint32_t>(SA)) ns = 0, nph ^= 1;
        if (nsb == static_cast<uint32_t>(SB)) nsb = 0, nphb ^= 1;
        bool ready = false;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          umma_ss<false>(tmem_base, da0 + uint64_t(k4 * 2), db + uint64_t(k4 * 2), idesc, 1);
          if (k4 == 3) {  // between the last two MMAs: is the next stage there already?
            ready = (!use_t || mbar_try_wait(&ctl->full_t[nsb], nphb)) && (!use_g || mbar_try_wait(&ctl->full_g[ns], nph));
            if (ready) fence_proxy_async_smem();
          }
          umma_ss<false>(tmem_base + 256, da1 + uint64_t(k4 * 2), db + uint64_t(k4 * 2), idesc, 1);
        }
        if (use_t) umma_commit(&ctl->empty_t[sb]);
        if (use_g) umma_commit(&ctl->empty_g[s]);
        if (it + 1 < p.iters && !ready) {
          if (use_t) mb_timed_wait<false>(&ctl->full_t[nsb], nphb, abort_flag, cyc_t, n_t);
          if (use_g) mb_timed_wait<false>(&ctl->full_g[ns], nph, abort_flag, cyc_g, n_g);
          fence_proxy_async_smem();
        }
        tc_fence_after_sync();
        s = ns, ph = nph, sb = nsb, phb = nphb;
      }
      umma_commit(&ctl->mma_bar[0]);
      mbar_wait(&ctl->mma_bar[0], 0, abort_flag);
      if (blockIdx.x == 0 && p.counters != nullptr) {
        p.counters[0] = cyc_t, p.counters[1] = n_t, p.counters[2] = cyc_g, p.counters[3] = n_g;
        p.counters[4] = static_cast<unsigned long long>(clock64() - t_begin);
      }
    } else if ((mode & kMbMma) && lane == 0 && leader) {
      const uint32_t idesc = make_idesc(kFmtF16, kPair ? 256 : ((mode & kMbM64) ? 64 : 128), 256, 0, 0);
      unsigned long long cyc_t = 0, n_t = 0, cyc_g = 0, n_g = 0;
      const long long t_begin = clock64();
      // ring positions advanced by hand: a division by the run-time depth here would sit between two stages' MMAs
      uint32_t s = 0, ph = 0, sb = 0, phb = 0;
      for (int it = 0; it < p.iters; ++it) {
        if (p.issue_delay > 0) {  // stand-in for instructions between the MMAs of two stages
          const long long t0 = clock64();
          while (clock64() - t0 < p.issue_delay) {
          }
        }
        if (coupled) {
          if (mode & kMbTma) mb_timed_wait<kPair>(&ctl->full_t[sb], phb, abort_flag, cyc_t, n_t);
          if (mode & kMbGather) mb_timed_wait<kPair>(&ctl->full_g[s], ph, abort_flag, cyc_g, n_g);
          fence_proxy_async_smem();
          tc_fence_after_sync();
        } else if (it >= 3) {
          mbar_wait(&ctl->mma_bar[(it - 3) & 3], ((it - 3) >> 2) & 1, abort_flag);  // at most three stages of MMAs queued
        }
        const uint32_t a_addr = smem_u32(gbuf + size_t(s) * kMbAChunk), b_addr = smem_u32(tbuf + size_t(sb) * p.b_chunk);
        const uint64_t da0 = make_smem_desc(a_addr, 16, 1024), da1 = make_smem_desc(a_addr + 16384, 16, 1024);
        const uint64_t db = make_smem_desc(b_addr, 16, 1024);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          if constexpr (kPair) {
            umma_ss_pair(tmem_base, da0 + uint64_t(k4 * 2), db + uint64_t(k4 * 2), idesc, 1);
            umma_ss_pair(tmem_base + 256, da1 + uint64_t(k4 * 2), db + uint64_t(k4 * 2), idesc, 1);
          } else {
            umma_ss<false>(tmem_base, da0 + uint64_t(k4 * 2), db + uint64_t(k4 * 2), idesc, 1);
            umma_ss<false>(tmem_base + 256, da1 + uint64_t(k4 * 2), db + uint64_t(k4 * 2), idesc, 1);
          }
        }
        if constexpr (kPair) {
          const uint32_t eg = smem_u32(&ctl->empty_g[s]), et = smem_u32(&ctl->empty_t[sb]);
          umma_commit_pair(eg);
          umma_commit_pair(cluster_map(eg, 1));
          umma_commit_pair(et);
          umma_commit_pair(cluster_map(et, 1));
          umma_commit_pair(smem_u32(&ctl->mma_bar[it & 3]));
        } else {
          if (coupled) {
            if (mode & kMbTma) umma_commit(&ctl->empty_t[sb]);
            if (mode & kMbGather) umma_commit(&ctl->empty_g[s]);
          }
          umma_commit(&ctl->mma_bar[it & 3]);
        }
        if (++s == static_cast<uint32_t>(SA)) s = 0, ph ^= 1;
        if (++sb == static_cast<uint32_t>(SB)) sb = 0, phb ^= 1;
      }
      for (int it = p.iters > 3 ? p.iters - 3 : 0; it < p.iters; ++it) mb_wait<kPair>(&ctl->mma_bar[it & 3], (it >> 2) & 1, abort_flag);
      if (blockIdx.x == 0 && p.counters != nullptr) {
        p.counters[0] = cyc_t, p.counters[1] = n_t, p.counters[2] = cyc_g, p.counters[3] = n_g;
        p.counters[4] = static_cast<unsigned long long>(clock64() - t_begin);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();  // no CTA leaves while its peer may still arrive on its barriers or read its operands
  if (warp == 10) {
    tc_fence_after_sync();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, 512u);
    else tmem_dealloc(tmem_base, 512u);
  }
  if (tid == 0 && ctl->abort_flag) report(p.status, FGB_S_WAIT_TIMEOUT);
}

}  // namespace
}  // namespace fgb

using namespace fgb;

extern "C" int fgb_microbench_pipeline(int mode, int stages_a, int stages_b, int iters, int issue_delay, const void* rows, int64_t n_rows, int row_bytes,
                                       const void* dense, int64_t dense_bytes, float* ms_out, uint64_t* counters, int32_t* status,
                                       void* stream) {
  if (!rows || !dense || !ms_out) return FGB_E_NULL;
  const bool pair = (mode & kMbPair) != 0;
  if (pair) mode |= kMbTma | kMbGather | kMbMma | kMbCoupled;
  if (issue_delay < 0 || issue_delay > 100000) return FGB_E_SIZE;
  if (iters < 1 || n_rows < 1 || n_rows >= (int64_t(1) << 31) || row_bytes < 128 || row_bytes % 128 != 0) return FGB_E_SIZE;
  if (stages_a < 1 || stages_a > kMbMaxStages || stages_b < 1 || stages_b > kMbMaxStages) return FGB_E_SIZE;
  if ((mode & kMbCoupled) && !(mode & kMbMma)) return FGB_E_SIZE;
  if ((mode & (kMbStore | kMbStoreBulk128 | kMbStoreBulk512)) && (mode & (kMbGather | kMbCoupled | kMbPair))) return FGB_E_SIZE;
  if ((mode & kMbM64) && (mode & (kMbPair | kMbLean))) return FGB_E_SIZE;
  if ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(dense)) & 15u) return FGB_E_ALIGN;
  MbParams p{};
  p.b_chunk = pair ? 16 * 1024 : 32 * 1024;
  if (dense_bytes < 2 * p.b_chunk) return FGB_E_SIZE;
  p.dense = static_cast<const char*>(dense);
  p.dense_bytes = static_cast<unsigned long long>(dense_bytes / p.b_chunk * p.b_chunk);
  p.rows = static_cast<const char*>(rows);
  p.n_rows = static_cast<uint32_t>(n_rows);
  p.row_bytes = row_bytes;
  p.iters = iters;
  p.issue_delay = issue_delay;
  p.mode = mode;
  p.stages_a = stages_a;
  p.stages_b = stages_b;
  p.status = status;
  const size_t smem = 1024 + 1024 + size_t(stages_a) * kMbAChunk + size_t(stages_b) * p.b_chunk;
  if (smem > 227 * 1024) return FGB_E_SIZE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap tmap;
  int rc = make_rows_tmap(&tmap, rows, n_rows, row_bytes / 2);
  if (rc != FGB_OK) return rc;
  unsigned long long* d_counters = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  rc = cuda_status(cudaMalloc(&d_counters, 8 * sizeof(unsigned long long)));
  if (rc == FGB_OK) rc = cuda_status(cudaMemsetAsync(d_counters, 0, 8 * sizeof(unsigned long long), s));
  if (rc == FGB_OK) rc = cuda_status(cudaEventCreate(&e0));
  if (rc == FGB_OK) rc = cuda_status(cudaEventCreate(&e1));
  p.counters = d_counters;
  int sms = device_sm_count();
  sms -= sms % 2;
  if (rc == FGB_OK) {
    if (pair) {
      static PerDeviceTable configured;
      rc = ensure_dynamic_smem(configured, microbench_kernel<true>, smem);
      if (rc == FGB_OK) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(sms);
        cfg.blockDim = dim3(kMbThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        rc = cuda_status(cudaEventRecord(e0, s));
        if (rc == FGB_OK) rc = cuda_status(cudaLaunchKernelEx(&cfg, microbench_kernel<true>, tmap, p));
      }
    } else {
      static PerDeviceTable configured;
      rc = ensure_dynamic_smem(configured, microbench_kernel<false>, smem);
      if (rc == FGB_OK) rc = cuda_status(cudaEventRecord(e0, s));
      if (rc == FGB_OK) {
        microbench_kernel<false><<<sms, kMbThreads, smem, s>>>(tmap, p);
        rc = launch_status();
      }
    }
  }
  if (rc == FGB_OK) rc = cuda_status(cudaEventRecord(e1, s));
  if (rc == FGB_OK) rc = cuda_status(cudaEventSynchronize(e1));
  if (rc == FGB_OK) rc = cuda_status(cudaEventElapsedTime(ms_out, e0, e1));
  if (rc == FGB_OK && counters != nullptr) {
    unsigned long long h[8];
    rc = cuda_status(cudaMemcpy(h, d_counters, sizeof(h), cudaMemcpyDeviceToHost));
    for (int i = 0; i < 8; ++i) counters[i] = h[i];
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (d_counters) cudaFree(d_counters);
  return rc;
}
