// GPU hash table over (b,x,y,z) voxel coordinates and the submanifold-conv
// neighbour map built from it.
//
// Table layout (private to this file; it never leaves the library):
//   32-bit keys: one 64-bit word per slot, (key << 32) | row, empty = ~0.
//                One CAS inserts key and value together and one 8-byte load
//                answers a probe.
//   64-bit keys: uint64 keys[slots] followed by uint32 rows[slots].
// Open addressing with linear probing; the slot is the Murmur3 finaliser of
// the key mapped to [0, slots) by a multiply-high.
//
// The lookup kernel flattens (voxel, offset) pairs in the order the map is
// stored, so consecutive threads write consecutive map words and no staging or
// pre-fill of the map is needed.  While the row is in flight the kernel also
// derives everything the later passes need from it: the per-voxel validity
// mask (gray code), its Gray-to-binary decode, and per-(offset, block) valid
// counts that a small scan turns into the offsets of the wgrad pair lists.
//
// Sorted input (the common case: coordinates in lexicographic (b, x, y, z)
// order, which is ascending flat-index order) needs no hash table at all: a
// row's position in the input IS its rank among the keys, and the voxels of one
// (b, x, y) column are consecutive rows.  One kernel checks the order and, while
// it has neighbouring rows in hand, writes the first and one-past-last row of
// every column into a direct-address table (8 bytes per column, kept in the
// memory the caller provided for the hash table); the lookup kernel then finds a
// neighbour by reading the column entry of (x + dx, y + dy) and searching the
// few rows of that column for z + dz.  The decision is taken on the device --
// the kernels of the other path return at once -- so no host round trip is
// added; both paths produce the same map.
#include <algorithm>
#include <type_traits>

#include "fgb_common.cuh"
#include "fgb_device.cuh"
#include "fgb_hash.cuh"

namespace fgb {

struct Stencil {
  int Kw, Kh, Kd, Dw, Dh, Dd, V;
  int Sw = 1, Sh = 1, Sd = 1;     // generic sparse conv only: stride
  int Pw = 0, Ph = 0, Pd = 0;     // generic sparse conv only: padding
};

// One CTA per 256 voxels; thread t handles the flattened (voxel, offset) items
// t, t+256, ... of the CTA, i.e. exactly the words t, t+256, ... of the CTA's
// slice of the map.
//
// kGeneral = false: submanifold conv.  The rows are the table's own voxels, the
// probed coordinate is coords[i] + (k - K/2) * dilation and the centre offset
// is the row itself.
// kGeneral = true: generic sparse conv.  The rows are output voxels, the table
// holds the input voxels, the probed coordinate is coords[i] * stride - padding
// + k * dilation, and every hit is also scattered into the backward map
// nbr_bwd[input row, v] = output row (when nbr_bwd is non-null).
template <int kKeyBits, bool kGeneral>
__global__ void __launch_bounds__(kMapBlock)
    subm_lookup_kernel(const int4* __restrict__ coords, uint32_t n, Grid3 g, Stencil st, void* table_mem, uint32_t slots,
                       uint32_t* __restrict__ nbr, uint32_t* __restrict__ nbr_bwd, int32_t* __restrict__ gray_out,
                       int32_t* __restrict__ binary_out, uint32_t* __restrict__ block_counts, uint32_t nblk,
                       const uint32_t* __restrict__ unsorted) {
  chain_release();
  chain_wait();
  if (unsorted != nullptr && *unsorted == 0u) return;  // the sorted-input kernel builds the map
  __shared__ int4 s_coord[kMapBlock];
  __shared__ uint32_t s_gray[kMapBlock];
  __shared__ uint32_t s_count[32];
  __shared__ int4 s_delta[32];  // (dx, dy, dz) of each offset: no divisions in the item loop
  const uint32_t n0 = blockIdx.x * kMapBlock;
  const uint32_t nv = min(static_cast<uint32_t>(kMapBlock), n - n0);
  const int t = threadIdx.x;
  const int V = st.V;
  if (t < nv) {
    int4 c = __ldg(&coords[n0 + t]);
    if constexpr (kGeneral) c.y *= st.Sw, c.z *= st.Sh, c.w *= st.Sd;
    s_coord[t] = c;
  }
  s_gray[t] = 0;
  if (t < 32) {
    s_count[t] = 0;
    const int KhKd = st.Kh * st.Kd;
    const int kx = t / KhKd, ky = (t / st.Kd) % st.Kh, kz = t % st.Kd;
    if constexpr (kGeneral) s_delta[t] = make_int4(kx * st.Dw - st.Pw, ky * st.Dh - st.Ph, kz * st.Dd - st.Pd, 0);
    else s_delta[t] = make_int4((kx - st.Kw / 2) * st.Dw, (ky - st.Kh / 2) * st.Dh, (kz - st.Kd / 2) * st.Dd, 0);
  }
  __syncthreads();

  const auto table = make_table<kKeyBits>(table_mem, slots);
  const int centre = V >> 1;  // all kernel extents are odd
  const uint32_t items = nv * V;
  uint32_t* out = nbr + static_cast<size_t>(n0) * V;
  // item = lv * V + v walks t, t + 256, ...: (lv, v) advance by (256 / V, 256 % V) with a carry
  const uint32_t step_lv = kMapBlock / V;
  const int step_v = kMapBlock % V;
  uint32_t lv = t / V;
  int v = t - lv * V;
  for (uint32_t item = t; item < items; item += kMapBlock) {
    uint32_t val;
    if (!kGeneral && v == centre) {
      val = n0 + lv;
    } else {
      const int4 c = s_coord[lv];
      const int4 d = s_delta[v];
      const int x = c.y + d.x, y = c.z + d.y, z = c.w + d.z;
      val = kInvalid;
      if (x >= 0 && x < g.W && y >= 0 && y < g.H && z >= 0 && z < g.D) val = table.find(g.template key<kKeyBits>(c.x, x, y, z));
    }
    out[item] = val;
    if (val != kInvalid) {
      if constexpr (kGeneral) {
        if (nbr_bwd) nbr_bwd[static_cast<size_t>(val) * V + v] = n0 + lv;
      }
      atomicOr(&s_gray[lv], 1u << v);
      atomicAdd(&s_count[v], 1u);
    }
    lv += step_lv;
    v += step_v;
    if (v >= V) {
      v -= V;
      ++lv;
    }
  }
  __syncthreads();
  if (t < nv) {
    const uint32_t gray = s_gray[t];
    uint32_t binary = gray;  // Gray -> binary: prefix xor from the top bit down
    binary ^= binary >> 1;
    binary ^= binary >> 2;
    binary ^= binary >> 4;
    binary ^= binary >> 8;
    binary ^= binary >> 16;
    gray_out[n0 + t] = static_cast<int32_t>(gray);
    binary_out[n0 + t] = static_cast<int32_t>(binary);
  }
  if (t < V) block_counts[static_cast<size_t>(t) * nblk + blockIdx.x] = s_count[t];
}

// CTA v turns block_counts[v, :] into exclusive offsets in place and leaves the
// total of offset v in seg[v + 1].  With `finish` the CTA that ends last also turns the totals into the segment table
// (what seg_prefix_kernel does as a launch of its own); seg[0] counts the finished CTAs and must be 0 on entry.
__global__ void __launch_bounds__(1024) block_scan_kernel(uint32_t* __restrict__ block_counts, uint32_t nblk, uint32_t* __restrict__ seg,
                                                          bool finish) {
  chain_release();
  chain_wait();
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  uint32_t* row = block_counts + static_cast<size_t>(blockIdx.x) * nblk;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  if (t == 0) s_carry = 0;
  __syncthreads();
  for (uint32_t base = 0; base < nblk; base += 1024) {
    const uint32_t i = base + t;
    const uint32_t x = i < nblk ? row[i] : 0u;
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
      s_warp[lane] = ws;  // inclusive over warps
    }
    __syncthreads();
    const uint32_t carry = s_carry;
    const uint32_t warp_excl = w == 0 ? 0u : s_warp[w - 1];
    if (i < nblk) row[i] = carry + warp_excl + inc - x;
    __syncthreads();
    if (t == 1023) s_carry = carry + s_warp[31];
    __syncthreads();
  }
  if (t == 0) {
    seg[blockIdx.x + 1] = s_carry;
    if (finish) {
      __threadfence();
      if (atomicAdd(&seg[0], 1u) == gridDim.x - 1) {  // every total is written
        __threadfence();
        uint32_t acc = 0;
        for (uint32_t v = 1; v <= gridDim.x; ++v) {
          acc += *reinterpret_cast<volatile uint32_t*>(&seg[v]);
          seg[v] = acc;
        }
        seg[0] = 0;
      }
    }
  }
}

__global__ void seg_prefix_kernel(uint32_t* seg, int V) {
  chain_release();
  chain_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    uint32_t acc = 0;
    seg[0] = 0;
    for (int v = 1; v <= V; ++v) {
      acc += seg[v];
      seg[v] = acc;
    }
  }
}

// ------------------------------------------------------------------ sorted-input path
// Column table entry: (first row, one past the last row) of the voxels of one (b, x, y) column; first == kInvalid for
// an empty column.
//
// *unsorted = 1 when some key is not greater than its predecessor or a coordinate lies outside the grid / batch (the
// word must be 0 on entry); otherwise every non-empty column's entry is written (the table must be filled with
// 0xff bytes on entry).
template <int kKeyBits>
__global__ void __launch_bounds__(256) column_index_kernel(const int4* __restrict__ coords, uint32_t n, Grid3 g, uint64_t columns,
                                                          uint2* __restrict__ col_table, uint32_t* unsorted) {
  chain_release();
  chain_wait();
  const uint32_t i = blockIdx.x * 256u + threadIdx.x;
  // an earlier CTA found the rows out of order: the table will not be used.  (Lane 0's reading decides for the warp:
  // the word may change between the lanes' loads, and the vote below needs the whole warp.)
  if (__shfl_sync(0xffffffffu, *reinterpret_cast<volatile uint32_t*>(unsorted), 0) != 0u) return;
  bool bad = false;
  if (i < n) {
    const int4 b = __ldg(&coords[i]);
    const bool inside = b.x >= 0 && b.y >= 0 && b.y < g.W && b.z >= 0 && b.z < g.H && b.w >= 0 && b.w < g.D;
    const uint64_t col = (static_cast<uint64_t>(static_cast<uint32_t>(b.x)) * g.W + static_cast<uint32_t>(b.y)) * g.H + static_cast<uint32_t>(b.z);
    bad = !inside || col >= columns;
    uint64_t col_prev = ~uint64_t(0);
    if (i > 0) {
      const int4 a = __ldg(&coords[i - 1]);
      bad = bad || g.template key<kKeyBits>(a.x, a.y, a.z, a.w) >= g.template key<kKeyBits>(b.x, b.y, b.z, b.w);
      col_prev = (static_cast<uint64_t>(static_cast<uint32_t>(a.x)) * g.W + static_cast<uint32_t>(a.y)) * g.H + static_cast<uint32_t>(a.z);
    }
    if (!bad) {
      if (col != col_prev) {
        col_table[col].x = i;
        if (i > 0 && col_prev < columns) col_table[col_prev].y = i;
      }
      if (i == n - 1) col_table[col].y = n;
    }
  }
  // one store per warp at most, and none once the word is set (with shuffled input every thread would store otherwise)
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0 && *reinterpret_cast<volatile uint32_t*>(unsorted) == 0u) *unsorted = 1u;
}

// fills the table with the empty pattern unless the sorted-input path runs
__global__ void __launch_bounds__(256) table_clear_kernel(uint32_t* __restrict__ words, size_t count, const uint32_t* __restrict__ unsorted) {
  chain_release();
  chain_wait();
  if (unsorted != nullptr && *unsorted == 0u) return;
  for (size_t i = blockIdx.x * size_t(256) + threadIdx.x; i < count; i += size_t(gridDim.x) * 256) words[i] = 0xFFFFFFFFu;
}

// One CTA per 256 voxels (the blocking of the hash lookup, so the side products are the same).  Work items are
// (voxel, (kx, ky)) pairs, dealt to the threads round-robin: an item reads the entry of the neighbouring column and
// walks the column's rows (ascending z) once for the Kd targets z + (kz - Kd/2) * Dd, which ascend with kz.  Hits go
// into the CTA's map tile in shared memory, which leaves as 16-byte stores.
//
// The kernel is bound by instruction issue, not by memory, so the common stencil (3x3x3, dilation 1: kUnit) gets an
// instance whose extents are compile-time constants (divisions by 9 and 3 become multiplies, the target loop unrolls),
// and column indices are 32-bit (the table has fewer than 2^32 entries by construction).
template <int kKeyBits, bool kUnit>
__global__ void __launch_bounds__(kMapBlock)
    subm_column_lookup_kernel(const int4* __restrict__ coords, uint32_t n, Grid3 g, Stencil st, const uint2* __restrict__ col_table,
                              uint32_t* __restrict__ nbr, int32_t* __restrict__ gray_out, int32_t* __restrict__ binary_out,
                              uint32_t* __restrict__ block_counts, uint32_t nblk, const uint32_t* __restrict__ unsorted) {
  chain_release();
  chain_wait();
  if (*unsorted != 0u) return;  // the hash kernels build the map
  extern __shared__ __align__(16) uint32_t s_nbr[];  // [kMapBlock * V]
  __shared__ int4 s_coord[kMapBlock];                // (column index, x, y, z)
  __shared__ uint32_t s_count[32];
  const int Kw = kUnit ? 3 : st.Kw, Kh = kUnit ? 3 : st.Kh, Kd = kUnit ? 3 : st.Kd;
  const int Dw = kUnit ? 1 : st.Dw, Dh = kUnit ? 1 : st.Dh, Dd = kUnit ? 1 : st.Dd;
  const int V = kUnit ? 27 : st.V;
  const uint32_t n0 = blockIdx.x * kMapBlock;
  const uint32_t nv = min(static_cast<uint32_t>(kMapBlock), n - n0);
  const int t = threadIdx.x, lane = t & 31;
  {
    const uint4 inv = make_uint4(kInvalid, kInvalid, kInvalid, kInvalid);
    for (int i = t; i < kMapBlock * V / 4; i += kMapBlock) reinterpret_cast<uint4*>(s_nbr)[i] = inv;  // kMapBlock * V is a multiple of 4
  }
  if (t < 32) s_count[t] = 0;
  if (t < nv) {
    const int4 c = __ldg(&coords[n0 + t]);
    const uint32_t col = (static_cast<uint32_t>(c.x) * static_cast<uint32_t>(g.W) + static_cast<uint32_t>(c.y)) * static_cast<uint32_t>(g.H) +
                         static_cast<uint32_t>(c.z);
    s_coord[t] = make_int4(static_cast<int>(col), c.y, c.z, c.w);
  }
  __syncthreads();

  const int combos = Kw * Kh;
  const int back = (Kd / 2) * Dd;  // smallest target z = own z - back
  const uint32_t items = nv * combos;
  for (uint32_t item = t; item < items; item += kMapBlock) {
    const uint32_t lv = item / combos;
    const int c = static_cast<int>(item - lv * combos);
    const int kx = c / Kh, ky = c - kx * Kh;
    const int dx = (kx - Kw / 2) * Dw, dy = (ky - Kh / 2) * Dh;
    const int4 me = s_coord[lv];
    const int x = me.y + dx, y = me.z + dy;
    if (x < 0 || x >= g.W || y < 0 || y >= g.H) continue;
    const uint2 e = __ldg(&col_table[static_cast<uint32_t>(me.x) + static_cast<uint32_t>(dx * g.H + dy)]);
    if (e.x == kInvalid) continue;
    uint32_t* out = s_nbr + lv * V + c * Kd;
    const int z_first = me.w - back;
    uint32_t lo = e.x;
    if (dx == 0 && dy == 0 && back <= 8) {
      // the voxel's own column: z strictly increases along its rows, so z - back lies at most `back` rows before it
      const uint32_t self = n0 + lv;
      lo = self - e.x > static_cast<uint32_t>(back) ? self - back : e.x;
    } else if (e.y - e.x > 4u) {  // short columns (a surface crosses a column a few times) are walked from their start
      uint32_t hi = e.y;
      while (hi - lo > 4u) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (__ldg(&coords[mid].w) < z_first) lo = mid + 1;
        else hi = mid;
      }
    }
    uint32_t row = lo;
    int zr = __ldg(&coords[row].w);  // lo < e.y: a non-empty column, and bisection keeps lo below its end or at a row that exists
#pragma unroll
    for (int kz = 0; kz < Kd; ++kz) {  // three iterations, unrolled, in the kUnit instance
      const int z = z_first + kz * Dd;
      while (zr < z) {
        ++row;
        zr = row < e.y ? __ldg(&coords[row].w) : 0x7FFFFFFF;
      }
      if (zr == z && z >= 0 && z < g.D) out[kz] = row;
    }
  }
  __syncthreads();

  uint32_t gray = 0;
  if (t < nv) {
    for (int k = 0; k < V; ++k) {
      if (s_nbr[t * V + k] != kInvalid) gray |= 1u << k;
    }
  }
  // per-offset valid counts of the CTA (for the pair-list offsets): lane v of each warp keeps the warp's count of offset v
  {
    uint32_t mine = 0;
    for (int v = 0; v < V; ++v) {
      const uint32_t b = __ballot_sync(0xffffffffu, (gray >> v) & 1u);
      if (lane == v) mine = static_cast<uint32_t>(__popc(b));
    }
    if (lane < V && mine != 0u) atomicAdd(&s_count[lane], mine);
  }
  __syncthreads();
  {
    // the CTA's map rows leave as 16-byte pieces (a block starts 256 * V * 4 bytes after the previous one)
    uint32_t* out = nbr + static_cast<size_t>(n0) * V;
    const uint32_t words = nv * V;
    const uint32_t vecs = (reinterpret_cast<uintptr_t>(out) & 15) == 0 ? words >> 2 : 0u;  // a map that is only 4-byte aligned goes word by word
    for (uint32_t i = t; i < vecs; i += kMapBlock) reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(s_nbr)[i];
    for (uint32_t i = vecs * 4 + t; i < words; i += kMapBlock) out[i] = s_nbr[i];
  }
  if (t < nv) {
    uint32_t binary = gray;
    binary ^= binary >> 1;
    binary ^= binary >> 2;
    binary ^= binary >> 4;
    binary ^= binary >> 8;
    binary ^= binary >> 16;
    gray_out[n0 + t] = static_cast<int32_t>(gray);
    binary_out[n0 + t] = static_cast<int32_t>(binary);
  }
  if (t < V) block_counts[static_cast<size_t>(t) * nblk + blockIdx.x] = s_count[t];
}

template <int kKeyBits>
static int build_impl(const int32_t* coords, uint32_t n, int B, Grid3 g, Stencil st, void* table, uint32_t slots, uint32_t* nbr,
                      int32_t* gray, int32_t* binary, uint32_t* block_counts, uint32_t* seg, int32_t* status, cudaStream_t s) {
  const uint32_t nblk = static_cast<uint32_t>(ceil_div(n, kMapBlock));
  const int4* c4 = reinterpret_cast<const int4*>(coords);
  const size_t table_bytes = static_cast<size_t>(fgb_hash_table_bytes(slots, kKeyBits));
  const size_t table_words = table_bytes / 4;
  const unsigned clear_grid = static_cast<unsigned>(std::min<size_t>(ceil_div(static_cast<int64_t>(table_words), 256 * 8), 148 * 16));
  // The sorted-input path needs one 8-byte entry per (b, x, y) column and keeps them in the caller's table memory; the
  // map tile of a CTA must fit shared memory.  seg[V + 1] carries the device-side decision between the two paths (0 =
  // rows in key order, the table-free path built the map) and stays there for the pair-list kernel.
  const uint64_t columns = static_cast<uint64_t>(B > 0 ? B : 0) * g.W * g.H;
  const bool try_sorted = columns > 0 && columns * sizeof(uint2) <= table_bytes;
  uint32_t* unsorted = try_sorted ? seg + st.V + 1 : nullptr;
  {
    // seg[0] = 0: the scan's count of finished CTAs; seg[V + 1]: the key-order word
    cudaError_t e = cudaMemsetAsync(seg, 0, (st.V + 2) * sizeof(uint32_t), s);
    if (e == cudaSuccess && !try_sorted) e = cudaMemsetAsync(seg + st.V + 1, 1, sizeof(uint32_t), s);
    if (e != cudaSuccess) return cuda_status(e);
  }
  if (try_sorted) {
    cudaError_t e = cudaMemsetAsync(table, 0xFF, columns * sizeof(uint2), s);
    if (e != cudaSuccess) return cuda_status(e);
    column_index_kernel<kKeyBits><<<static_cast<unsigned>(ceil_div(n, 256)), 256, 0, s>>>(c4, n, g, columns, static_cast<uint2*>(table), unsorted);
  }
  // from here on every kernel is chained to the one before it (fgb_device.cuh): the launches overlap the kernels' tails
  LaunchErrors chain;
  chain.add(launch_chained(table_clear_kernel, dim3(clear_grid > 0 ? clear_grid : 1), dim3(256), 0, s, static_cast<uint32_t*>(table),
                           table_words, unsorted));
  chain.add(launch_chained(hash_insert_kernel<kKeyBits>, dim3(nblk), dim3(kMapBlock), 0, s, c4, n, g, table, slots, status, unsorted));
  chain.add(launch_chained(subm_lookup_kernel<kKeyBits, false>, dim3(nblk), dim3(kMapBlock), 0, s, c4, n, g, st, table, slots, nbr,
                           static_cast<uint32_t*>(nullptr), gray, binary, block_counts, nblk, unsorted));
  if (try_sorted) {
    const size_t smem = size_t(kMapBlock) * st.V * sizeof(uint32_t);
    const bool unit = st.Kw == 3 && st.Kh == 3 && st.Kd == 3 && st.Dw == 1 && st.Dh == 1 && st.Dd == 1;
    if (unit)
      chain.add(launch_chained(subm_column_lookup_kernel<kKeyBits, true>, dim3(nblk), dim3(kMapBlock), smem, s, c4, n, g, st,
                               static_cast<const uint2*>(table), nbr, gray, binary, block_counts, nblk, unsorted));
    else
      chain.add(launch_chained(subm_column_lookup_kernel<kKeyBits, false>, dim3(nblk), dim3(kMapBlock), smem, s, c4, n, g, st,
                               static_cast<const uint2*>(table), nbr, gray, binary, block_counts, nblk, unsorted));
  }
  chain.add(launch_chained(block_scan_kernel, dim3(st.V), dim3(1024), 0, s, block_counts, nblk, seg, true));
  return chain.first != cudaSuccess ? cuda_status(chain.first) : launch_status();
}

// generic sparse conv: table over the input voxels, rows = output voxels
template <int kKeyBits>
static int build_general_impl(const int32_t* in_coords, uint32_t n_in, const int32_t* out_coords, uint32_t n_out, Grid3 g, Stencil st,
                              void* table, uint32_t slots, uint32_t* nbr, uint32_t* nbr_bwd, int32_t* gray, int32_t* binary,
                              uint32_t* block_counts, uint32_t* seg, int32_t* status, cudaStream_t s) {
  if (n_in > 0)
    hash_insert_kernel<kKeyBits><<<static_cast<unsigned>(ceil_div(n_in, kMapBlock)), kMapBlock, 0, s>>>(
        reinterpret_cast<const int4*>(in_coords), n_in, g, table, slots, status, nullptr);
  const uint32_t nblk = static_cast<uint32_t>(ceil_div(n_out, kMapBlock));
  subm_lookup_kernel<kKeyBits, true><<<nblk, kMapBlock, 0, s>>>(reinterpret_cast<const int4*>(out_coords), n_out, g, st, table, slots,
                                                               nbr, nbr_bwd, gray, binary, block_counts, nblk, nullptr);
  block_scan_kernel<<<st.V, 1024, 0, s>>>(block_counts, nblk, seg, false);
  seg_prefix_kernel<<<1, 32, 0, s>>>(seg, st.V);
  return launch_status();
}

// gray[i] = mask of the valid offsets of map row i, binary[i] = its Gray-to-binary decode
__global__ void __launch_bounds__(256) gray_from_map_kernel(const uint32_t* __restrict__ nbr, uint32_t n, int V,
                                                            int32_t* __restrict__ gray_out, int32_t* __restrict__ binary_out) {
  // a warp covers 32 consecutive map words at a time; lanes vote the validity bits of each row
  __shared__ uint32_t s_gray[256];
  const uint32_t n0 = blockIdx.x * 256u;
  const uint32_t nv = min(256u, n - n0);
  const int t = threadIdx.x;
  s_gray[t] = 0;
  __syncthreads();
  const uint32_t items = nv * V;
  const uint32_t* in = nbr + static_cast<size_t>(n0) * V;
  for (uint32_t item = t; item < items; item += 256) {
    if (__ldg(&in[item]) != kInvalid) {
      const uint32_t lv = item / V;
      atomicOr(&s_gray[lv], 1u << (item - lv * V));
    }
  }
  __syncthreads();
  if (t < nv) {
    const uint32_t gray = s_gray[t];
    uint32_t binary = gray;
    binary ^= binary >> 1;
    binary ^= binary >> 2;
    binary ^= binary >> 4;
    binary ^= binary >> 8;
    binary ^= binary >> 16;
    gray_out[n0 + t] = static_cast<int32_t>(gray);
    binary_out[n0 + t] = static_cast<int32_t>(binary);
  }
}

}  // namespace fgb

extern "C" int64_t fgb_hash_table_bytes(int64_t slots, int key_bits) {
  if (slots < 0 || slots >= (int64_t(1) << 31)) return FGB_E_SIZE;
  if (key_bits == 32) return slots * 8;
  if (key_bits == 64) return slots * 12;
  return FGB_E_DTYPE;
}

extern "C" int64_t fgb_map_num_blocks(int64_t n) { return n < 0 ? FGB_E_SIZE : fgb::ceil_div(n, fgb::kMapBlock); }

extern "C" int fgb_subm_build_neighbor_map(const int32_t* coords, int64_t n, int B, int W, int H, int D, int Kw, int Kh, int Kd, int Dw,
                                           int Dh, int Dd, void* table, int64_t slots, int key_bits, uint32_t* neighbor_map,
                                           int32_t* gray_code, int32_t* binary_code, uint32_t* block_counts,
                                           uint32_t* valid_signal_seg, int32_t* status, void* stream) {
  using namespace fgb;
  if (n < 0 || n >= (int64_t(1) << 32) - 1) return FGB_E_SIZE;
  if (B < 0 || W <= 0 || H <= 0 || D <= 0) return FGB_E_SIZE;
  if (Kw <= 0 || Kh <= 0 || Kd <= 0 || !(Kw & 1) || !(Kh & 1) || !(Kd & 1)) return FGB_E_SIZE;
  if (Dw <= 0 || Dh <= 0 || Dd <= 0) return FGB_E_SIZE;
  const int64_t V = int64_t(Kw) * Kh * Kd;
  if (V > 32) return FGB_E_SIZE;
  if (key_bits != 32 && key_bits != 64) return FGB_E_DTYPE;
  if (slots < n || slots >= (int64_t(1) << 31)) return FGB_E_SIZE;
  if (valid_signal_seg == nullptr) return FGB_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0) return cuda_status(cudaMemsetAsync(valid_signal_seg, 0, (V + 1) * sizeof(uint32_t), s));
  if (!coords || !table || !neighbor_map || !gray_code || !binary_code || !block_counts) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(coords) & 15) return FGB_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(table) & 7) return FGB_E_ALIGN;
  const Grid3 g{W, H, D};
  const Stencil st{Kw, Kh, Kd, Dw, Dh, Dd, static_cast<int>(V)};
  if (key_bits == 32)
    return build_impl<32>(coords, static_cast<uint32_t>(n), B, g, st, table, static_cast<uint32_t>(slots), neighbor_map, gray_code,
                          binary_code, block_counts, valid_signal_seg, status, s);
  return build_impl<64>(coords, static_cast<uint32_t>(n), B, g, st, table, static_cast<uint32_t>(slots), neighbor_map, gray_code,
                        binary_code, block_counts, valid_signal_seg, status, s);
}

extern "C" int fgb_sparse_build_neighbor_map(const int32_t* in_coords, int64_t n_in, const int32_t* out_coords, int64_t n_out, int W,
                                             int H, int D, int Kw, int Kh, int Kd, int Sw, int Sh, int Sd, int Pw, int Ph, int Pd,
                                             int Dw, int Dh, int Dd, void* table, int64_t slots, int key_bits, uint32_t* neighbor_map,
                                             uint32_t* neighbor_map_bwd, int32_t* gray_code, int32_t* binary_code,
                                             uint32_t* block_counts, uint32_t* valid_signal_seg, int32_t* status, void* stream) {
  using namespace fgb;
  const int64_t lim = (int64_t(1) << 32) - 1;
  if (n_in < 0 || n_in >= lim || n_out < 0 || n_out >= lim) return FGB_E_SIZE;
  if (W <= 0 || H <= 0 || D <= 0) return FGB_E_SIZE;
  if (Kw <= 0 || Kh <= 0 || Kd <= 0 || Sw <= 0 || Sh <= 0 || Sd <= 0 || Dw <= 0 || Dh <= 0 || Dd <= 0) return FGB_E_SIZE;
  if (Pw < 0 || Ph < 0 || Pd < 0) return FGB_E_SIZE;
  const int64_t V = int64_t(Kw) * Kh * Kd;
  if (V > 32) return FGB_E_SIZE;
  if (key_bits != 32 && key_bits != 64) return FGB_E_DTYPE;
  if (slots < n_in || slots < 1 || slots >= (int64_t(1) << 31)) return FGB_E_SIZE;
  if (valid_signal_seg == nullptr) return FGB_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc;
  if (neighbor_map_bwd && n_in > 0) {
    rc = cuda_status(cudaMemsetAsync(neighbor_map_bwd, 0xFF, static_cast<size_t>(n_in) * V * sizeof(uint32_t), s));
    if (rc != FGB_OK) return rc;
  }
  if (n_out == 0) return cuda_status(cudaMemsetAsync(valid_signal_seg, 0, (V + 1) * sizeof(uint32_t), s));
  if (!out_coords || !table || !neighbor_map || !gray_code || !binary_code || !block_counts) return FGB_E_NULL;
  if (n_in > 0 && !in_coords) return FGB_E_NULL;
  if ((reinterpret_cast<uintptr_t>(in_coords) | reinterpret_cast<uintptr_t>(out_coords)) & 15) return FGB_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(table) & 7) return FGB_E_ALIGN;
  rc = cuda_status(cudaMemsetAsync(table, 0xFF, static_cast<size_t>(fgb_hash_table_bytes(slots, key_bits)), s));
  if (rc != FGB_OK) return rc;
  const Grid3 g{W, H, D};
  Stencil st{Kw, Kh, Kd, Dw, Dh, Dd, static_cast<int>(V)};
  st.Sw = Sw, st.Sh = Sh, st.Sd = Sd, st.Pw = Pw, st.Ph = Ph, st.Pd = Pd;
  if (key_bits == 32)
    return build_general_impl<32>(in_coords, static_cast<uint32_t>(n_in), out_coords, static_cast<uint32_t>(n_out), g, st, table,
                                  static_cast<uint32_t>(slots), neighbor_map, neighbor_map_bwd, gray_code, binary_code, block_counts,
                                  valid_signal_seg, status, s);
  return build_general_impl<64>(in_coords, static_cast<uint32_t>(n_in), out_coords, static_cast<uint32_t>(n_out), g, st, table,
                                static_cast<uint32_t>(slots), neighbor_map, neighbor_map_bwd, gray_code, binary_code, block_counts,
                                valid_signal_seg, status, s);
}

extern "C" int fgb_pp_gray_code(const uint32_t* neighbor_map, int64_t n, int V, int32_t* gray_code, int32_t* binary_code, void* stream) {
  using namespace fgb;
  if (n < 0 || n >= (int64_t(1) << 32) - 1 || V < 1 || V > 32) return FGB_E_SIZE;
  if (n == 0) return FGB_OK;
  if (!neighbor_map || !gray_code || !binary_code) return FGB_E_NULL;
  gray_from_map_kernel<<<static_cast<unsigned>(ceil_div(n, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      neighbor_map, static_cast<uint32_t>(n), V, gray_code, binary_code);
  return launch_status();
}
