// GPU hash table over (b, x, y, z) voxel coordinates, shared by the neighbour-map
// and grid-sample kernels.
//
// Table layout (private to the library; it never leaves it):
//   32-bit keys: one 64-bit word per slot, (key << 32) | row, empty = ~0.
//                One CAS inserts key and value together and one 8-byte load
//                answers a probe.
//   64-bit keys: uint64 keys[slots] followed by uint32 rows[slots].
// Open addressing with linear probing; the slot is the Murmur3 finaliser of
// the key mapped to [0, slots) by a multiply-high.  Probes are bounded by the
// slot count.
#pragma once

#include "fgb_common.cuh"
#include "fgb_device.cuh"

namespace fgb {

template <int kKeyBits>
struct Table;

template <>
struct Table<32> {
  unsigned long long* slots_;
  uint32_t n_;
  __device__ __forceinline__ uint32_t home(uint64_t key) const { return __umulhi(fmix32(static_cast<uint32_t>(key)), n_); }
  // returns false when every slot was visited without finding room
  __device__ __forceinline__ bool insert(uint64_t key, uint32_t row) const {
    const unsigned long long word = (static_cast<unsigned long long>(static_cast<uint32_t>(key)) << 32) | row;
    uint32_t s = home(key);
    for (uint32_t i = 0; i < n_; ++i) {
      unsigned long long prev = atomicCAS(&slots_[s], ~0ULL, word);
      if (prev == ~0ULL || static_cast<uint32_t>(prev >> 32) == static_cast<uint32_t>(key)) return true;
      if (++s >= n_) s = 0;
    }
    return false;
  }
  __device__ __forceinline__ uint32_t find(uint64_t key) const {
    uint32_t s = home(key);
    for (uint32_t i = 0; i < n_; ++i) {
      unsigned long long w = __ldg(&slots_[s]);
      if (w == ~0ULL) return kInvalid;
      if (static_cast<uint32_t>(w >> 32) == static_cast<uint32_t>(key)) return static_cast<uint32_t>(w);
      if (++s >= n_) s = 0;
    }
    return kInvalid;
  }
};

template <>
struct Table<64> {
  unsigned long long* keys_;
  uint32_t* rows_;
  uint32_t n_;
  __device__ __forceinline__ uint32_t home(uint64_t key) const { return __umulhi(fmix64_hi(key), n_); }
  __device__ __forceinline__ bool insert(uint64_t key, uint32_t row) const {
    uint32_t s = home(key);
    for (uint32_t i = 0; i < n_; ++i) {
      unsigned long long prev = atomicCAS(&keys_[s], ~0ULL, static_cast<unsigned long long>(key));
      if (prev == ~0ULL) {
        rows_[s] = row;
        return true;
      }
      if (prev == key) return true;
      if (++s >= n_) s = 0;
    }
    return false;
  }
  __device__ __forceinline__ uint32_t find(uint64_t key) const {
    uint32_t s = home(key);
    for (uint32_t i = 0; i < n_; ++i) {
      unsigned long long k = __ldg(&keys_[s]);
      if (k == ~0ULL) return kInvalid;
      if (k == key) return __ldg(&rows_[s]);
      if (++s >= n_) s = 0;
    }
    return kInvalid;
  }
};

template <int kKeyBits>
__device__ __forceinline__ Table<kKeyBits> make_table(void* mem, uint32_t slots);
template <>
__device__ __forceinline__ Table<32> make_table<32>(void* mem, uint32_t slots) {
  return Table<32>{static_cast<unsigned long long*>(mem), slots};
}
template <>
__device__ __forceinline__ Table<64> make_table<64>(void* mem, uint32_t slots) {
  auto* keys = static_cast<unsigned long long*>(mem);
  return Table<64>{keys, reinterpret_cast<uint32_t*>(keys + slots), slots};
}

struct Grid3 {
  int W, H, D;
  // flat index b*W*H*D + x*H*D + y*D + z; 32-bit arithmetic is exact whenever the 32-bit table is in use
  template <int kKeyBits>
  __device__ __forceinline__ uint64_t key(int b, int x, int y, int z) const {
    if constexpr (kKeyBits == 32) {
      return ((static_cast<uint32_t>(b) * W + x) * H + y) * static_cast<uint32_t>(D) + z;
    } else {
      return ((static_cast<uint64_t>(b) * W + x) * H + y) * static_cast<uint64_t>(D) + z;
    }
  }
};

// one thread per voxel, 16-byte coordinate loads
// `unsorted` (may be null): device word, 0 when the sorted-input path builds the map instead -- then the table is not needed
template <int kKeyBits>
__global__ void __launch_bounds__(kMapBlock) hash_insert_kernel(const int4* __restrict__ coords, uint32_t n, Grid3 g,
                                                                void* table_mem, uint32_t slots, int32_t* status,
                                                                const uint32_t* __restrict__ unsorted) {
  chain_release();
  chain_wait();
  if (unsorted != nullptr && *unsorted == 0u) return;
  const uint32_t i = blockIdx.x * kMapBlock + threadIdx.x;
  if (i >= n) return;
  const int4 c = __ldg(&coords[i]);
  const auto table = make_table<kKeyBits>(table_mem, slots);
  if (!table.insert(g.template key<kKeyBits>(c.x, c.y, c.z, c.w), i)) report(status, FGB_S_TABLE_FULL);
}

}  // namespace fgb
