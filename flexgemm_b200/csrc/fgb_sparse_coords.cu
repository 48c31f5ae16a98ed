// Output coordinates of a generic (strided / padded / dilated) sparse
// convolution: the set of output voxels that at least one input voxel
// contributes to, in the order of a serialisation key.
//
// Two calls with one host read between them (the caller needs the count to
// allocate the result):
//   collect  -- every (input voxel, kernel offset) pair proposes the output
//               voxel it feeds; a hash set over the flat (b, x, y, z) index of
//               the output grid keeps the first proposal of each voxel and the
//               winner appends the index to a compact list;
//   finalize -- sorts the list by the serialisation key (flat index, Morton
//               code or Hilbert index, batch in the top bits) and decodes it
//               to int32 (b, x, y, z) rows.
#include <cub/device/device_radix_sort.cuh>

#include "fgb_common.cuh"

namespace fgb {

struct OutGrid {
  int Wo, Ho, Do;
  __device__ __forceinline__ uint64_t flat(int b, int x, int y, int z) const {
    return ((static_cast<uint64_t>(b) * Wo + x) * Ho + y) * static_cast<uint64_t>(Do) + z;
  }
  __device__ __forceinline__ int4 coords(uint64_t key) const {
    const int z = static_cast<int>(key % Do);
    key /= Do;
    const int y = static_cast<int>(key % Ho);
    key /= Ho;
    return make_int4(static_cast<int>(key / Wo), static_cast<int>(key % Wo), y, z);
  }
};

struct ConvGeom {
  int Kw, Kh, Kd, Sw, Sh, Sd, Pw, Ph, Pd, Dw, Dh, Dd;
};

template <typename K>
__device__ __forceinline__ uint32_t set_home(K key, uint32_t slots);
template <>
__device__ __forceinline__ uint32_t set_home<uint32_t>(uint32_t key, uint32_t slots) { return __umulhi(fmix32(key), slots); }
template <>
__device__ __forceinline__ uint32_t set_home<unsigned long long>(unsigned long long key, uint32_t slots) {
  return __umulhi(fmix64_hi(key), slots);
}

// One thread per (input voxel, offset).  K = uint32_t or unsigned long long.
template <typename K>
__global__ void __launch_bounds__(256) collect_out_keys_kernel(const int4* __restrict__ coords, uint32_t n, ConvGeom cg, OutGrid og,
                                                               K* __restrict__ set, uint32_t slots, K* __restrict__ keys,
                                                               uint32_t* __restrict__ count, int32_t* status) {
  const int V = cg.Kw * cg.Kh * cg.Kd;
  const uint64_t tid = blockIdx.x * uint64_t(256) + threadIdx.x;
  const uint32_t i = static_cast<uint32_t>(tid / V);
  if (i >= n) return;
  const int v = static_cast<int>(tid - uint64_t(i) * V);
  const int kx = v / (cg.Kh * cg.Kd), ky = (v / cg.Kd) % cg.Kh, kz = v % cg.Kd;
  const int4 c = __ldg(&coords[i]);
  int x = c.y + cg.Pw - kx * cg.Dw, y = c.z + cg.Ph - ky * cg.Dh, z = c.w + cg.Pd - kz * cg.Dd;
  if (x < 0 || y < 0 || z < 0) return;
  if (x % cg.Sw != 0 || y % cg.Sh != 0 || z % cg.Sd != 0) return;
  x /= cg.Sw, y /= cg.Sh, z /= cg.Sd;
  if (x >= og.Wo || y >= og.Ho || z >= og.Do) return;
  const K key = static_cast<K>(og.flat(c.x, x, y, z));
  const K empty = ~K(0);
  uint32_t s = set_home<K>(key, slots);
  for (uint32_t probe = 0; probe < slots; ++probe) {
    const K prev = atomicCAS(&set[s], empty, key);
    if (prev == empty) {
      keys[atomicAdd(count, 1u)] = key;  // at most `slots` winners: the list has that capacity
      return;
    }
    if (prev == key) return;
    if (++s >= slots) s = 0;
  }
  report(status, FGB_S_TABLE_FULL);
}

__device__ __forceinline__ uint64_t spread3(uint64_t v) {  // 21 bits -> every third bit
  v = (v | (v << 32)) & 0x001F00000000FFFFull;
  v = (v | (v << 16)) & 0x001F0000FF0000FFull;
  v = (v | (v << 8)) & 0x100F00F00F00F00Full;
  v = (v | (v << 4)) & 0x10C30C30C30C30C3ull;
  v = (v | (v << 2)) & 0x1249249249249249ull;
  return v;
}
__device__ __forceinline__ uint64_t morton3(uint32_t x, uint32_t y, uint32_t z) {  // x owns the top bit of every triple
  return (spread3(x) << 2) | (spread3(y) << 1) | spread3(z);
}

// Hilbert index of (x, y, z) on a 2^bits cube: Skilling's axes-to-transpose
// transform ("Programming the Hilbert curve", 2004) followed by bit interleaving.
__device__ __forceinline__ uint64_t hilbert3(uint32_t x, uint32_t y, uint32_t z, int bits) {
  uint32_t a[3] = {x, y, z};
  const uint32_t top = 1u << (bits - 1);
  for (uint32_t q = top; q > 1; q >>= 1) {
    const uint32_t low = q - 1;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      if (a[i] & q) {
        a[0] ^= low;
      } else {
        const uint32_t swap = (a[0] ^ a[i]) & low;
        a[0] ^= swap;
        a[i] ^= swap;
      }
    }
  }
  a[1] ^= a[0];
  a[2] ^= a[1];
  uint32_t fold = 0;
  for (uint32_t q = top; q > 1; q >>= 1)
    if (a[2] & q) fold ^= q - 1;
  return morton3(a[0] ^ fold, a[1] ^ fold, a[2] ^ fold);
}

// sort key of a flat output index under serialisation mode 1 (Morton) or 2 (Hilbert)
template <typename K>
__global__ void __launch_bounds__(256) serial_key_kernel(const K* __restrict__ keys, uint32_t count, OutGrid og, int mode, int bits,
                                                         uint64_t* __restrict__ sort_keys) {
  const uint32_t i = blockIdx.x * 256u + threadIdx.x;
  if (i >= count) return;
  const int4 c = og.coords(keys[i]);
  const uint64_t code = mode == 1 ? morton3(c.y, c.z, c.w) : hilbert3(c.y, c.z, c.w, bits);
  const uint64_t mask = bits >= 21 ? ~0ull >> 1 : ((1ull << (3 * bits)) - 1);
  sort_keys[i] = (code & mask) | (static_cast<uint64_t>(c.x) << (3 * bits));
}

template <typename K>
__global__ void __launch_bounds__(256) decode_out_keys_kernel(const K* __restrict__ keys, uint32_t count, OutGrid og,
                                                              int4* __restrict__ out) {
  const uint32_t i = blockIdx.x * 256u + threadIdx.x;
  if (i < count) out[i] = og.coords(keys[i]);
}

static int bit_length(uint64_t v) {
  int b = 0;
  while (v) ++b, v >>= 1;
  return b;
}

struct CoordsPlan {
  size_t sorted_off, skey_in_off, skey_out_off, temp_off, temp_bytes, total;
};

template <typename K>
static int coords_plan(int64_t count, int mode, CoordsPlan* p) {
  auto align = [](size_t x) { return (x + 255) & ~size_t(255); };
  p->sorted_off = 0;
  p->skey_in_off = align(size_t(count) * sizeof(K));
  p->skey_out_off = p->skey_in_off + (mode ? align(size_t(count) * 8) : 0);
  p->temp_off = p->skey_out_off + (mode ? align(size_t(count) * 8) : 0);
  p->temp_bytes = 0;
  cudaError_t e;
  if (mode == 0)
    e = cub::DeviceRadixSort::SortKeys(nullptr, p->temp_bytes, static_cast<const K*>(nullptr), static_cast<K*>(nullptr), count, 0,
                                       int(sizeof(K) * 8), nullptr);
  else
    e = cub::DeviceRadixSort::SortPairs(nullptr, p->temp_bytes, static_cast<const uint64_t*>(nullptr), static_cast<uint64_t*>(nullptr),
                                        static_cast<const K*>(nullptr), static_cast<K*>(nullptr), count, 0, 64, nullptr);
  if (e != cudaSuccess) return cuda_status(e);
  p->total = p->temp_off + align(p->temp_bytes);
  return FGB_OK;
}

template <typename K>
static int finalize_impl(const K* keys, int64_t count, int B, OutGrid og, int mode, int bits, char* ws, int64_t ws_bytes, int32_t* out,
                         cudaStream_t s) {
  CoordsPlan p;
  int rc = coords_plan<K>(count, mode, &p);
  if (rc != FGB_OK) return rc;
  if (ws_bytes < static_cast<int64_t>(p.total)) return FGB_E_WORKSPACE;
  K* sorted = reinterpret_cast<K*>(ws + p.sorted_off);
  const unsigned grid = static_cast<unsigned>(ceil_div(count, 256));
  cudaError_t e;
  if (mode == 0) {
    const uint64_t vol = uint64_t(B) * og.Wo * og.Ho * og.Do;
    int end_bit = bit_length(vol ? vol - 1 : 0);
    if (end_bit < 1) end_bit = 1;
    if (end_bit > int(sizeof(K) * 8)) end_bit = int(sizeof(K) * 8);
    e = cub::DeviceRadixSort::SortKeys(ws + p.temp_off, p.temp_bytes, keys, sorted, count, 0, end_bit, s);
  } else {
    uint64_t* skey_in = reinterpret_cast<uint64_t*>(ws + p.skey_in_off);
    uint64_t* skey_out = reinterpret_cast<uint64_t*>(ws + p.skey_out_off);
    serial_key_kernel<K><<<grid, 256, 0, s>>>(keys, static_cast<uint32_t>(count), og, mode, bits, skey_in);
    rc = launch_status();
    if (rc != FGB_OK) return rc;
    int end_bit = 3 * bits + bit_length(B > 0 ? uint64_t(B - 1) : 0);
    if (end_bit < 1) end_bit = 1;
    if (end_bit > 64) end_bit = 64;
    e = cub::DeviceRadixSort::SortPairs(ws + p.temp_off, p.temp_bytes, skey_in, skey_out, keys, sorted, count, 0, end_bit, s);
  }
  if (e != cudaSuccess) return cuda_status(e);
  decode_out_keys_kernel<K><<<grid, 256, 0, s>>>(sorted, static_cast<uint32_t>(count), og, reinterpret_cast<int4*>(out));
  return launch_status();
}

static bool out_grid(int W, int H, int D, const ConvGeom& cg, OutGrid* og) {
  og->Wo = (W + 2 * cg.Pw - cg.Dw * (cg.Kw - 1) - 1) / cg.Sw + 1;
  og->Ho = (H + 2 * cg.Ph - cg.Dh * (cg.Kh - 1) - 1) / cg.Sh + 1;
  og->Do = (D + 2 * cg.Pd - cg.Dd * (cg.Kd - 1) - 1) / cg.Sd + 1;
  return og->Wo > 0 && og->Ho > 0 && og->Do > 0;
}

static bool geom_ok(const ConvGeom& cg) {
  return cg.Kw > 0 && cg.Kh > 0 && cg.Kd > 0 && cg.Sw > 0 && cg.Sh > 0 && cg.Sd > 0 && cg.Pw >= 0 && cg.Ph >= 0 && cg.Pd >= 0 &&
         cg.Dw > 0 && cg.Dh > 0 && cg.Dd > 0 && int64_t(cg.Kw) * cg.Kh * cg.Kd <= 32;
}

}  // namespace fgb

extern "C" int fgb_sparse_out_grid(int W, int H, int D, int Kw, int Kh, int Kd, int Sw, int Sh, int Sd, int Pw, int Ph, int Pd, int Dw,
                                   int Dh, int Dd, int* Wo, int* Ho, int* Do) {
  using namespace fgb;
  const ConvGeom cg{Kw, Kh, Kd, Sw, Sh, Sd, Pw, Ph, Pd, Dw, Dh, Dd};
  if (!Wo || !Ho || !Do) return FGB_E_NULL;
  if (W <= 0 || H <= 0 || D <= 0 || !geom_ok(cg)) return FGB_E_SIZE;
  OutGrid og;
  out_grid(W, H, D, cg, &og);
  *Wo = og.Wo, *Ho = og.Ho, *Do = og.Do;
  return FGB_OK;
}

extern "C" int fgb_sparse_out_coords_collect(const int32_t* in_coords, int64_t n_in, int W, int H, int D, int Kw, int Kh, int Kd, int Sw,
                                             int Sh, int Sd, int Pw, int Ph, int Pd, int Dw, int Dh, int Dd, void* set, int64_t slots,
                                             int key_bits, void* keys, uint32_t* count, int32_t* status, void* stream) {
  using namespace fgb;
  const ConvGeom cg{Kw, Kh, Kd, Sw, Sh, Sd, Pw, Ph, Pd, Dw, Dh, Dd};
  if (n_in < 0 || n_in >= (int64_t(1) << 32) - 1) return FGB_E_SIZE;
  if (W <= 0 || H <= 0 || D <= 0 || !geom_ok(cg)) return FGB_E_SIZE;
  if (key_bits != 32 && key_bits != 64) return FGB_E_DTYPE;
  if (slots < 1 || slots >= (int64_t(1) << 31)) return FGB_E_SIZE;
  if (!count) return FGB_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = cuda_status(cudaMemsetAsync(count, 0, sizeof(uint32_t), s));
  if (rc != FGB_OK) return rc;
  OutGrid og;
  if (n_in == 0 || !out_grid(W, H, D, cg, &og)) return FGB_OK;  // nothing can be produced
  if (!in_coords || !set || !keys) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(in_coords) & 15) return FGB_E_ALIGN;
  if ((reinterpret_cast<uintptr_t>(set) | reinterpret_cast<uintptr_t>(keys)) & 7) return FGB_E_ALIGN;
  rc = cuda_status(cudaMemsetAsync(set, 0xFF, static_cast<size_t>(slots) * (key_bits / 8), s));
  if (rc != FGB_OK) return rc;
  const int V = Kw * Kh * Kd;
  const int64_t grid = ceil_div(n_in * V, 256);
  if (grid > 0x7FFFFFFF) return FGB_E_SIZE;
  if (key_bits == 32)
    collect_out_keys_kernel<uint32_t><<<static_cast<unsigned>(grid), 256, 0, s>>>(
        reinterpret_cast<const int4*>(in_coords), static_cast<uint32_t>(n_in), cg, og, static_cast<uint32_t*>(set),
        static_cast<uint32_t>(slots), static_cast<uint32_t*>(keys), count, status);
  else
    collect_out_keys_kernel<unsigned long long><<<static_cast<unsigned>(grid), 256, 0, s>>>(
        reinterpret_cast<const int4*>(in_coords), static_cast<uint32_t>(n_in), cg, og, static_cast<unsigned long long*>(set),
        static_cast<uint32_t>(slots), static_cast<unsigned long long*>(keys), count, status);
  return launch_status();
}

extern "C" int64_t fgb_sparse_out_coords_workspace_bytes(int64_t count, int key_bits, int mode) {
  using namespace fgb;
  if (count < 0 || count >= (int64_t(1) << 32) - 1 || mode < 0 || mode > 2) return FGB_E_SIZE;
  if (key_bits != 32 && key_bits != 64) return FGB_E_DTYPE;
  if (count == 0) return 0;
  CoordsPlan p;
  const int rc = key_bits == 32 ? coords_plan<uint32_t>(count, mode, &p) : coords_plan<unsigned long long>(count, mode, &p);
  return rc == FGB_OK ? static_cast<int64_t>(p.total) : rc;
}

extern "C" int fgb_sparse_out_coords_finalize(const void* keys, int64_t count, int key_bits, int mode, int coord_bits, int B, int W, int H,
                                              int D, int Kw, int Kh, int Kd, int Sw, int Sh, int Sd, int Pw, int Ph, int Pd, int Dw,
                                              int Dh, int Dd, void* workspace, int64_t workspace_bytes, int32_t* out_coords,
                                              void* stream) {
  using namespace fgb;
  const ConvGeom cg{Kw, Kh, Kd, Sw, Sh, Sd, Pw, Ph, Pd, Dw, Dh, Dd};
  if (count < 0 || count >= (int64_t(1) << 32) - 1 || mode < 0 || mode > 2 || B < 1) return FGB_E_SIZE;
  if (W <= 0 || H <= 0 || D <= 0 || !geom_ok(cg)) return FGB_E_SIZE;
  if (key_bits != 32 && key_bits != 64) return FGB_E_DTYPE;
  if (mode != 0 && (coord_bits < 1 || coord_bits > 21)) return FGB_E_SIZE;
  if (count == 0) return FGB_OK;
  OutGrid og;
  if (!out_grid(W, H, D, cg, &og)) return FGB_E_SIZE;
  if (!keys || !workspace || !out_coords) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FGB_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(out_coords) & 15) return FGB_E_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (key_bits == 32)
    return finalize_impl<uint32_t>(static_cast<const uint32_t*>(keys), count, B, og, mode, coord_bits, static_cast<char*>(workspace),
                                   workspace_bytes, out_coords, s);
  return finalize_impl<unsigned long long>(static_cast<const unsigned long long*>(keys), count, B, og, mode, coord_bits,
                                           static_cast<char*>(workspace), workspace_bytes, out_coords, s);
}
