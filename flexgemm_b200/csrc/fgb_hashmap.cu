// Generic hash map with caller-chosen values, in the caller-visible layout
// of the reference's table calls: a key array (uint32 or uint64, empty slot =
// all ones) and a value array (uint32 or uint64) of `slots` entries each, both
// owned and initialised by the caller.  Open addressing, linear probing; the
// home slot is the Murmur3 finaliser of the key mapped to [0, slots) by a
// multiply-high.  Which slot a key lands in is not observable through these
// calls -- only insert followed by lookup is -- so the slot choice differs from
// the reference's (hash % slots) without changing any result.
//
// (The neighbour-map builder keeps its own packed 64-bit-slot table, see
// fgb_hash.cuh: its table never leaves the library.)
//
// Duplicate keys in one insert call: one of their values survives, as in the
// reference.  A table without a free slot records FGB_S_TABLE_FULL in the
// status word instead of probing forever.
#include "fgb_common.cuh"

namespace fgb {

template <typename K>
__device__ __forceinline__ uint32_t open_home(K key, uint32_t slots) {
  if constexpr (sizeof(K) == 4) return __umulhi(fmix32(static_cast<uint32_t>(key)), slots);
  else return __umulhi(fmix64_hi(static_cast<uint64_t>(key)), slots);
}

template <typename K>
__device__ __forceinline__ K open_cas(K* addr, K expect, K desired) {
  if constexpr (sizeof(K) == 4) return atomicCAS(reinterpret_cast<unsigned int*>(addr), expect, desired);
  else return atomicCAS(reinterpret_cast<unsigned long long*>(addr), static_cast<unsigned long long>(expect),
                        static_cast<unsigned long long>(desired));
}

template <typename K, typename V>
__device__ __forceinline__ bool open_insert(K* keys, V* vals, uint32_t slots, K key, V value) {
  constexpr K kEmpty = ~K(0);
  uint32_t s = open_home<K>(key, slots);
  for (uint32_t i = 0; i < slots; ++i) {
    const K prev = open_cas<K>(&keys[s], kEmpty, key);
    if (prev == kEmpty || prev == key) {
      vals[s] = value;
      return true;
    }
    if (++s >= slots) s = 0;
  }
  return false;
}

template <typename K, typename V>
__device__ __forceinline__ V open_lookup(const K* __restrict__ keys, const V* __restrict__ vals, uint32_t slots, K key) {
  constexpr K kEmpty = ~K(0);
  uint32_t s = open_home<K>(key, slots);
  for (uint32_t i = 0; i < slots; ++i) {
    const K k = __ldg(&keys[s]);
    if (k == kEmpty) return ~V(0);
    if (k == key) return __ldg(&vals[s]);
    if (++s >= slots) s = 0;
  }
  return ~V(0);
}

// flat (b, x, y, z) index in 64 bits, truncated to the key type as the reference does
template <typename K>
__device__ __forceinline__ K flat_key(const int4 c, int W, int H, int D) {
  const uint64_t f = ((static_cast<uint64_t>(static_cast<uint32_t>(c.x)) * W + static_cast<uint32_t>(c.y)) * H + static_cast<uint32_t>(c.z)) *
                         static_cast<uint64_t>(D) + static_cast<uint32_t>(c.w);
  return static_cast<K>(f);
}

enum { kByKey = 0, kByCoord = 1, kByCoordRowValue = 2 };

// kMode: keys given directly / keys = flat index of coordinate rows / the same with value = row number
template <typename K, typename V, int kMode>
__global__ void __launch_bounds__(256) open_insert_kernel(K* __restrict__ keys, V* __restrict__ vals, uint32_t slots, const void* __restrict__ in,
                                                         const V* __restrict__ in_vals, int64_t m, int W, int H, int D, int32_t* status) {
  const int64_t i = blockIdx.x * int64_t(256) + threadIdx.x;
  if (i >= m) return;
  K key;
  if constexpr (kMode == kByKey) key = __ldg(static_cast<const K*>(in) + i);
  else key = flat_key<K>(__ldg(static_cast<const int4*>(in) + i), W, H, D);
  V value;
  if constexpr (kMode == kByCoordRowValue) value = static_cast<V>(i);
  else value = __ldg(&in_vals[i]);
  if (!open_insert<K, V>(keys, vals, slots, key, value)) report(status, FGB_S_TABLE_FULL);
}

template <typename K, typename V, int kMode>
__global__ void __launch_bounds__(256) open_lookup_kernel(const K* __restrict__ keys, const V* __restrict__ vals, uint32_t slots,
                                                         const void* __restrict__ in, int64_t m, int W, int H, int D, V* __restrict__ out) {
  const int64_t i = blockIdx.x * int64_t(256) + threadIdx.x;
  if (i >= m) return;
  if constexpr (kMode == kByKey) {
    out[i] = open_lookup<K, V>(keys, vals, slots, __ldg(static_cast<const K*>(in) + i));
  } else {
    const int4 c = __ldg(static_cast<const int4*>(in) + i);
    // coordinates outside the grid are absent (the reference does not test the batch index; a negative one cannot be stored)
    if (c.y < 0 || c.y >= W || c.z < 0 || c.z >= H || c.w < 0 || c.w >= D) out[i] = ~V(0);
    else out[i] = open_lookup<K, V>(keys, vals, slots, flat_key<K>(c, W, H, D));
  }
}

template <int kMode, bool kInsert>
static int dispatch_open(void* keys, void* vals, int64_t slots, int key_bits, int val_bits, const void* in, const void* in_vals, int64_t m,
                         int W, int H, int D, void* out, int32_t* status, cudaStream_t s) {
  if ((key_bits != 32 && key_bits != 64) || (val_bits != 32 && val_bits != 64)) return FGB_E_DTYPE;
  if (slots < 1 || slots >= (int64_t(1) << 31) || m < 0) return FGB_E_SIZE;
  if (kMode != kByKey && (W <= 0 || H <= 0 || D <= 0)) return FGB_E_SIZE;
  if (m == 0) return FGB_OK;
  if (!keys || !vals || !in) return FGB_E_NULL;
  if (kInsert && kMode != kByCoordRowValue && !in_vals) return FGB_E_NULL;
  if (!kInsert && !out) return FGB_E_NULL;
  if (kMode != kByKey && (reinterpret_cast<uintptr_t>(in) & 15)) return FGB_E_ALIGN;
  const unsigned grid = static_cast<unsigned>(ceil_div(m, 256));
  const uint32_t n = static_cast<uint32_t>(slots);
  auto run = [&](auto k0, auto v0) {
    using K = decltype(k0);
    using V = decltype(v0);
    if constexpr (kInsert)
      open_insert_kernel<K, V, kMode><<<grid, 256, 0, s>>>(static_cast<K*>(keys), static_cast<V*>(vals), n, in, static_cast<const V*>(in_vals), m,
                                                          W, H, D, status);
    else
      open_lookup_kernel<K, V, kMode><<<grid, 256, 0, s>>>(static_cast<const K*>(keys), static_cast<const V*>(vals), n, in, m, W, H, D,
                                                          static_cast<V*>(out));
  };
  if (key_bits == 32 && val_bits == 32) run(uint32_t(0), uint32_t(0));
  else if (key_bits == 32) run(uint32_t(0), uint64_t(0));
  else if (val_bits == 32) run(uint64_t(0), uint32_t(0));
  else run(uint64_t(0), uint64_t(0));
  return launch_status();
}

}  // namespace fgb

extern "C" int fgb_hashmap_insert(void* hashmap_keys, void* hashmap_vals, int64_t slots, int key_bits, int val_bits, const void* keys,
                                  const void* values, int64_t m, int32_t* status, void* stream) {
  return fgb::dispatch_open<fgb::kByKey, true>(hashmap_keys, hashmap_vals, slots, key_bits, val_bits, keys, values, m, 1, 1, 1, nullptr, status,
                                               static_cast<cudaStream_t>(stream));
}

extern "C" int fgb_hashmap_lookup(const void* hashmap_keys, const void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                                  const void* keys, int64_t m, void* out_values, void* stream) {
  return fgb::dispatch_open<fgb::kByKey, false>(const_cast<void*>(hashmap_keys), const_cast<void*>(hashmap_vals), slots, key_bits, val_bits, keys,
                                                nullptr, m, 1, 1, 1, out_values, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int fgb_hashmap_insert_3d(void* hashmap_keys, void* hashmap_vals, int64_t slots, int key_bits, int val_bits, const int32_t* coords,
                                     const void* values, int64_t m, int W, int H, int D, int32_t* status, void* stream) {
  return fgb::dispatch_open<fgb::kByCoord, true>(hashmap_keys, hashmap_vals, slots, key_bits, val_bits, coords, values, m, W, H, D, nullptr,
                                                 status, static_cast<cudaStream_t>(stream));
}

extern "C" int fgb_hashmap_insert_3d_idx_as_val(void* hashmap_keys, void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                                                const int32_t* coords, int64_t m, int W, int H, int D, int32_t* status, void* stream) {
  return fgb::dispatch_open<fgb::kByCoordRowValue, true>(hashmap_keys, hashmap_vals, slots, key_bits, val_bits, coords, nullptr, m, W, H, D,
                                                         nullptr, status, static_cast<cudaStream_t>(stream));
}

extern "C" int fgb_hashmap_lookup_3d(const void* hashmap_keys, const void* hashmap_vals, int64_t slots, int key_bits, int val_bits,
                                     const int32_t* coords, int64_t m, int W, int H, int D, void* out_values, void* stream) {
  return fgb::dispatch_open<fgb::kByCoord, false>(const_cast<void*>(hashmap_keys), const_cast<void*>(hashmap_vals), slots, key_bits, val_bits,
                                                  coords, nullptr, m, W, H, D, out_values, nullptr, static_cast<cudaStream_t>(stream));
}
