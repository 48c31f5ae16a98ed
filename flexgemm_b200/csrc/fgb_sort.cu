// Stable argsort of the per-voxel binary codes: sorted_idx for the masked implicit GEMM.
//
// A least-significant-digit radix sort of (code, row) pairs with 9-bit digits:
// three passes cover the 27 bits of a 3x3x3 mask (a library radix sort with
// 8-bit digits needs four, plus a pass to write the row numbers).  One kernel
// first counts, for every pass at once, how many codes carry each digit value.
// Each pass then is ONE kernel: a CTA takes a tile of keys (dealt by a ticket
// counter, so that a tile's predecessors are always running or done), ranks
// its keys by digit in a stable way (warp match + per-warp digit counters), and
// learns how many keys of each digit the earlier tiles hold by looking back
// over their published counts -- every tile first publishes its own count, and
// later the inclusive prefix, per digit, in one 32-bit word (2 flag bits + 30
// bits), so a look-back stops at the first tile whose prefix is known.  The
// keys of the first pass are read straight from the codes (the row number is
// the position), the last pass writes only the int64 row numbers.
//
// Waits are bounded: a look-back that stays unanswered records
// FGB_S_WAIT_TIMEOUT, publishes what it has and goes on, so the kernel always
// ends (its output is then meaningless, which the status word says).
#include <algorithm>

#include "fgb_common.cuh"
#include "fgb_device.cuh"

namespace fgb {

constexpr int kDigitBits = 9;
constexpr int kDigits = 1 << kDigitBits;   // 512
constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortMaxPasses = 4;          // 32 bits / 9
constexpr uint32_t kFlagAggregate = 1u << 30, kFlagPrefix = 2u << 30, kCountMask = (1u << 30) - 1u;
constexpr uint32_t kLookbackPolls = 1u << 22;   // of >= 32 ns each: far beyond any legitimate wait

// hist[p * 512 + d] += number of codes whose digit p is d, for every pass p < passes
__global__ void __launch_bounds__(kSortThreads) sort_histogram_kernel(const int32_t* __restrict__ codes, uint32_t n, int passes, uint32_t flip,
                                                                      uint32_t* __restrict__ hist) {
  __shared__ uint32_t s_h[kSortMaxPasses * kDigits];
  chain_release();
  for (int i = threadIdx.x; i < passes * kDigits; i += kSortThreads) s_h[i] = 0;
  chain_wait();  // set-up above overlaps the tail of the kernel before; global memory only from here on
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const uint32_t per = (n + gridDim.x - 1) / gridDim.x;
  const uint32_t begin = blockIdx.x * per, end = min(n, begin + per);
  // whole warps walk the range so that every lane takes part in the votes
  for (uint32_t i0 = begin + (threadIdx.x & ~31u); i0 < end; i0 += kSortThreads) {
    const uint32_t i = i0 + lane;
    const bool ok = i < end;
    const uint32_t key = ok ? static_cast<uint32_t>(__ldg(&codes[i])) ^ flip : 0u;
    const unsigned valid = __ballot_sync(0xffffffffu, ok);  // a prefix of the lanes
    // neighbouring voxels mostly share their code: the warp's keys are cut into runs of equal keys, and the first
    // lane of a run adds the run's length to the key's bin of every pass (equal keys share all their digits)
    const uint32_t prev = __shfl_up_sync(0xffffffffu, key, 1);
    const bool head = ok && (lane == 0 || key != prev);
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    if (head) {
      const unsigned later = heads & ~((2u << lane) - 1u);  // run heads above this lane
      const int next = later != 0u ? __ffs(later) - 1 : __popc(valid);
      const uint32_t len = static_cast<uint32_t>(next - lane);
      for (int p = 0; p < passes; ++p) atomicAdd(&s_h[p * kDigits + ((key >> (p * kDigitBits)) & (kDigits - 1))], len);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < passes * kDigits; i += kSortThreads) {
    const uint32_t c = s_h[i];
    if (c != 0u) atomicAdd(&hist[i], c);
  }
}

__device__ __forceinline__ uint32_t load_status(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_status(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One pass.  kItems keys per thread, a tile = 256 * kItems keys.  Order of the keys inside a tile: warp w holds the
// keys [w * 32 * kItems, (w + 1) * 32 * kItems) of the tile, item j of lane l is key w * 32 * kItems + j * 32 + l.
template <int kItems, bool kFirst, bool kLast>
__global__ void __launch_bounds__(kSortThreads)
    sort_pass_kernel(const int32_t* __restrict__ codes, const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                     uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t* __restrict__ idx_out, uint32_t n, int shift,
                     uint32_t flip, const uint32_t* __restrict__ hist, uint32_t* __restrict__ ticket, uint32_t* __restrict__ status,
                     int32_t* err) {
  __shared__ uint32_t s_cnt[kSortWarps][kDigits];  // per-warp digit counts, then each warp's offset inside the tile's digit run
  __shared__ uint32_t s_base[kDigits];             // output position of the tile's first key of each digit
  __shared__ uint32_t s_scan[kSortWarps];
  __shared__ uint32_t s_tile;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  chain_release();
  for (int i = tid; i < kSortWarps * kDigits; i += kSortThreads) (&s_cnt[0][0])[i] = 0;
  chain_wait();  // the pass before (or the histogram) has completed; global memory only from here on
  if (tid == 0) s_tile = atomicAdd(ticket, 1u);
  __syncthreads();
  const uint32_t tile = s_tile;
  const uint32_t base = tile * (kSortThreads * kItems) + w * (32 * kItems);

  uint32_t key[kItems], val[kItems], rank[kItems];
  bool ok[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const uint32_t i = base + j * 32 + lane;
    ok[j] = i < n;
    if constexpr (kFirst) {
      key[j] = ok[j] ? static_cast<uint32_t>(__ldg(&codes[i])) ^ flip : 0u;
      val[j] = i;
    } else {
      key[j] = ok[j] ? __ldg(&keys_in[i]) : 0u;
      val[j] = ok[j] ? __ldg(&vals_in[i]) : 0u;
    }
  }
  // stable rank of every key among the keys of its digit in this warp's chunk: items in order, lanes in order
  const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const uint32_t d = (key[j] >> shift) & (kDigits - 1);
    const unsigned valid = __ballot_sync(0xffffffffu, ok[j]);
    const unsigned peers = __match_any_sync(0xffffffffu, d) & valid;
    const int leader = __ffs(peers) - 1;
    uint32_t before = 0;
    if (ok[j] && lane == leader) {
      before = s_cnt[w][d];
      s_cnt[w][d] = before + static_cast<uint32_t>(__popc(peers));
    }
    before = __shfl_sync(0xffffffffu, before, leader < 0 ? 0 : leader);
    rank[j] = before + static_cast<uint32_t>(__popc(peers & lt));
    __syncwarp();
  }
  __syncthreads();

  // thread t owns digits 2t and 2t + 1: counts of the tile, exclusive scan of the global histogram over the digits,
  // and the look-back over the earlier tiles
  uint32_t count[2], first_of_digit[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int d = 2 * tid + k;
    uint32_t acc = 0;
#pragma unroll
    for (int ww = 0; ww < kSortWarps; ++ww) {
      const uint32_t c = s_cnt[ww][d];
      s_cnt[ww][d] = acc;
      acc += c;
    }
    count[k] = acc;
  }
  {
    const uint32_t h0 = __ldg(&hist[2 * tid]), h1 = __ldg(&hist[2 * tid + 1]);
    uint32_t inc = h0 + h1;
#pragma unroll
    for (int dlt = 1; dlt < 32; dlt <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, inc, dlt);
      if (lane >= dlt) inc += y;
    }
    if (lane == 31) s_scan[w] = inc;
    __syncthreads();
    uint32_t warp_base = 0;
    for (int ww = 0; ww < w; ++ww) warp_base += s_scan[ww];
    first_of_digit[0] = warp_base + inc - (h0 + h1);
    first_of_digit[1] = first_of_digit[0] + h0;
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int d = 2 * tid + k;
    uint32_t* mine = status + size_t(tile) * kDigits + d;
    uint32_t before = 0;
    if (tile == 0) {
      store_status(mine, count[k] | kFlagPrefix);
    } else {
      store_status(mine, count[k] | kFlagAggregate);
      for (uint32_t t = tile; t-- > 0;) {
        const uint32_t* theirs = status + size_t(t) * kDigits + d;
        uint32_t v = load_status(theirs);
        for (uint32_t polls = 0; (v >> 30) == 0u; ++polls) {
          if (polls >= kLookbackPolls) {
            report(err, FGB_S_WAIT_TIMEOUT);
            v = kFlagPrefix;  // give up on this digit: the output is void, the kernel still ends
            break;
          }
          __nanosleep(32);
          v = load_status(theirs);
        }
        before += v & kCountMask;
        if (v & kFlagPrefix) break;
      }
      store_status(mine, ((before + count[k]) & kCountMask) | kFlagPrefix);
    }
    s_base[d] = first_of_digit[k] + before;
  }
  __syncthreads();

#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    if (!ok[j]) continue;
    const uint32_t d = (key[j] >> shift) & (kDigits - 1);
    const uint32_t pos = s_base[d] + s_cnt[w][d] + rank[j];
    if (pos >= n) continue;  // only after a timed-out look-back
    if constexpr (kLast) {
      idx_out[pos] = static_cast<int64_t>(val[j]);
    } else {
      keys_out[pos] = key[j];
      vals_out[pos] = val[j];
    }
  }
}

struct SortLayout {
  size_t keys_a, vals_a, keys_b, vals_b, control, status, total;
  uint32_t tiles;
  int items;
};

// Tiles of 4096 keys for long inputs (the per-tile bookkeeping -- 512 counters published and looked back over the
// earlier tiles -- is then small beside the keys), of 2048 keys up to 400 k keys (measured: 52 against 58 us at 164 k keys,
// 79 against 76 us at 660 k) and of 1024 keys for very short inputs, so that more CTAs share the work.
static SortLayout sort_layout(int64_t n) {
  auto align = [](size_t x) { return (x + 255) & ~size_t(255); };
  SortLayout L;
  L.items = n <= (int64_t(1) << 15) ? 4 : n <= 400000 ? 8 : 16;
  L.tiles = static_cast<uint32_t>(ceil_div(n > 0 ? n : 1, int64_t(kSortThreads) * L.items));
  const size_t arr = align(size_t(n) * 4);
  L.keys_a = 0, L.vals_a = arr, L.keys_b = 2 * arr, L.vals_b = 3 * arr;
  L.control = 4 * arr;                                                     // histograms [4][512], then the tickets [4]
  L.status = L.control + align((kSortMaxPasses * kDigits + kSortMaxPasses) * 4);
  L.total = L.status + align(size_t(kSortMaxPasses) * L.tiles * kDigits * 4);
  return L;
}

template <int kItems>
static cudaError_t launch_pass(int pass, int passes, const int32_t* codes, char* ws, const SortLayout& L, uint32_t n, uint32_t flip, int64_t* out,
                        int32_t* err, cudaStream_t s) {
  uint32_t* ka = reinterpret_cast<uint32_t*>(ws + L.keys_a);
  uint32_t* va = reinterpret_cast<uint32_t*>(ws + L.vals_a);
  uint32_t* kb = reinterpret_cast<uint32_t*>(ws + L.keys_b);
  uint32_t* vb = reinterpret_cast<uint32_t*>(ws + L.vals_b);
  uint32_t* hist = reinterpret_cast<uint32_t*>(ws + L.control) + pass * kDigits;
  uint32_t* ticket = reinterpret_cast<uint32_t*>(ws + L.control) + kSortMaxPasses * kDigits + pass;
  uint32_t* status = reinterpret_cast<uint32_t*>(ws + L.status) + size_t(pass) * L.tiles * kDigits;
  // passes alternate between the two buffer pairs: pass 0 writes a, pass 1 reads a and writes b, ...
  const uint32_t* kin = (pass & 1) ? ka : kb;
  const uint32_t* vin = (pass & 1) ? va : vb;
  uint32_t* kout = (pass & 1) ? kb : ka;
  uint32_t* vout = (pass & 1) ? vb : va;
  const int shift = pass * kDigitBits;
  const bool first = pass == 0, last = pass == passes - 1;
  cudaError_t rc;
  if (first && last)
    rc = launch_chained(sort_pass_kernel<kItems, true, true>, dim3(L.tiles), dim3(kSortThreads), 0, s, codes, kin, vin, kout, vout, out, n, shift, flip, hist, ticket, status, err);
  else if (first)
    rc = launch_chained(sort_pass_kernel<kItems, true, false>, dim3(L.tiles), dim3(kSortThreads), 0, s, codes, kin, vin, kout, vout, out, n, shift, flip, hist, ticket, status, err);
  else if (last)
    rc = launch_chained(sort_pass_kernel<kItems, false, true>, dim3(L.tiles), dim3(kSortThreads), 0, s, codes, kin, vin, kout, vout, out, n, shift, flip, hist, ticket, status, err);
  else
    rc = launch_chained(sort_pass_kernel<kItems, false, false>, dim3(L.tiles), dim3(kSortThreads), 0, s, codes, kin, vin, kout, vout, out, n, shift, flip, hist, ticket, status, err);
  return rc;
}

}  // namespace fgb

extern "C" int64_t fgb_pp_sorted_idx_workspace_bytes(int64_t n) {
  if (n < 0 || n >= (int64_t(1) << 30)) return FGB_E_SIZE;
  return static_cast<int64_t>(fgb::sort_layout(n).total);
}

extern "C" int fgb_pp_sorted_idx(const int32_t* binary_code, int64_t n, int key_bits, int64_t* sorted_idx, void* workspace,
                                 int64_t workspace_bytes, int32_t* status, void* stream) {
  using namespace fgb;
  if (n < 0 || n >= (int64_t(1) << 30)) return FGB_E_SIZE;
  if (key_bits < 1 || key_bits > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!binary_code || !sorted_idx || !workspace) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FGB_E_ALIGN;
  const SortLayout L = sort_layout(n);
  if (workspace_bytes < static_cast<int64_t>(L.total)) return FGB_E_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  const int passes = (key_bits + kDigitBits - 1) / kDigitBits;
  // Codes with fewer than 32 significant bits are non-negative; with 32 bits they are signed, and flipping the top
  // bit makes the unsigned digit order the signed order.
  const uint32_t flip = key_bits == 32 ? 0x80000000u : 0u;
  // histograms, tickets and the look-back words start at zero
  int rc = cuda_status(cudaMemsetAsync(ws + L.control, 0, L.total - L.control, s));
  if (rc != FGB_OK) return rc;
  // keys per CTA of the histogram: 1024 up to 400 k keys, 2048 beyond (measured: 42 / 43.5 / 46.5 us for the whole sort at
  // 164 k keys with 1024 / 2048 / 4096; 70.5 / 68.7 / 70.6 us at 660 k), at most eight CTAs per SM
  const unsigned hist_grid = static_cast<unsigned>(std::min<int64_t>(ceil_div(n, n <= 400000 ? 1024 : 2048), 148 * 8));
  sort_histogram_kernel<<<hist_grid, kSortThreads, 0, s>>>(binary_code, static_cast<uint32_t>(n), passes, flip,
                                                          reinterpret_cast<uint32_t*>(ws + L.control));
  for (int pass = 0; pass < passes; ++pass) {
    cudaError_t e;
    if (L.items == 16) e = launch_pass<16>(pass, passes, binary_code, ws, L, static_cast<uint32_t>(n), flip, sorted_idx, status, s);
    else if (L.items == 8) e = launch_pass<8>(pass, passes, binary_code, ws, L, static_cast<uint32_t>(n), flip, sorted_idx, status, s);
    else e = launch_pass<4>(pass, passes, binary_code, ws, L, static_cast<uint32_t>(n), flip, sorted_idx, status, s);
    if (e != cudaSuccess) return cuda_status(e);
  }
  return launch_status();
}
