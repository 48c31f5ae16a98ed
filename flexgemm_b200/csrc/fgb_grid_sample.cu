// Generic use of the coordinate hash table and the sparse grid sample built on it:
// insert / lookup of (b, x, y, z) rows, the nearest and trilinear neighbour maps of
// arbitrary query points, and the gather (forward) / scatter-add (backward) of
// features through such a map.  All of it is HBM-bound byte and index work.
#include <algorithm>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fgb_common.cuh"
#include "fgb_hash.cuh"

namespace fgb {

__global__ void __launch_bounds__(256) fill_words_kernel(uint32_t* __restrict__ words, size_t count, uint32_t value) {
  for (size_t i = blockIdx.x * size_t(256) + threadIdx.x; i < count; i += size_t(gridDim.x) * 256) words[i] = value;
}

template <int kKeyBits>
__global__ void __launch_bounds__(256) hash_lookup_3d_kernel(const int4* __restrict__ query, uint32_t m, Grid3 g, void* table_mem,
                                                            uint32_t slots, uint32_t* __restrict__ out) {
  const uint32_t i = blockIdx.x * 256u + threadIdx.x;
  if (i >= m) return;
  const int4 c = __ldg(&query[i]);
  uint32_t val = kInvalid;
  if (c.x >= 0 && c.y >= 0 && c.y < g.W && c.z >= 0 && c.z < g.H && c.w >= 0 && c.w < g.D)
    val = make_table<kKeyBits>(table_mem, slots).find(g.template key<kKeyBits>(c.x, c.y, c.z, c.w));
  out[i] = val;
}

// neighbor[q] = row of the voxel that contains query point q (coordinates truncated towards zero), or 0xffffffff
template <int kKeyBits>
__global__ void __launch_bounds__(256) nearest_map_kernel(const float* __restrict__ query, uint32_t B, uint32_t L, Grid3 g,
                                                         void* table_mem, uint32_t slots, uint32_t* __restrict__ neighbor) {
  const uint32_t i = blockIdx.x * 256u + threadIdx.x;
  if (i >= B * L) return;
  const int b = static_cast<int>(i / L);
  const int x = static_cast<int>(__ldg(&query[3 * size_t(i)])), y = static_cast<int>(__ldg(&query[3 * size_t(i) + 1])),
            z = static_cast<int>(__ldg(&query[3 * size_t(i) + 2]));
  uint32_t val = kInvalid;
  if (x >= 0 && x < g.W && y >= 0 && y < g.H && z >= 0 && z < g.D)
    val = make_table<kKeyBits>(table_mem, slots).find(g.template key<kKeyBits>(b, x, y, z));
  neighbor[i] = val;
}

// The eight voxels around query point q (corner i: x + (i & 1), y + ((i >> 1) & 1), z + ((i >> 2) & 1) from the
// base floor(q - 0.5)) and their trilinear weights, normalised over the voxels that exist.
template <int kKeyBits>
__global__ void __launch_bounds__(256) trilinear_map_kernel(const float* __restrict__ query, uint32_t B, uint32_t L, Grid3 g,
                                                           void* table_mem, uint32_t slots, uint32_t* __restrict__ neighbor,
                                                           float* __restrict__ weight) {
  const uint32_t i = blockIdx.x * 256u + threadIdx.x;
  if (i >= B * L) return;
  const int b = static_cast<int>(i / L);
  const float qx = __ldg(&query[3 * size_t(i)]), qy = __ldg(&query[3 * size_t(i) + 1]), qz = __ldg(&query[3 * size_t(i) + 2]);
  const int bx = static_cast<int>(floorf(qx - 0.5f)), by = static_cast<int>(floorf(qy - 0.5f)), bz = static_cast<int>(floorf(qz - 0.5f));
  const auto table = make_table<kKeyBits>(table_mem, slots);
  uint32_t nb[8];
  float w[8];
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int x = bx + (k & 1), y = by + ((k >> 1) & 1), z = bz + ((k >> 2) & 1);
    nb[k] = kInvalid;
    w[k] = 0.f;
    if (x >= 0 && x < g.W && y >= 0 && y < g.H && z >= 0 && z < g.D) {
      const uint32_t row = table.find(g.template key<kKeyBits>(b, x, y, z));
      if (row != kInvalid) {
        nb[k] = row;
        w[k] = (1.f - fabsf(qx - x - 0.5f)) * (1.f - fabsf(qy - y - 0.5f)) * (1.f - fabsf(qz - z - 0.5f));
        sum += w[k];
      }
    }
  }
  const float inv = 1.f / fmaxf(sum, 1e-12f);
  uint4* no = reinterpret_cast<uint4*>(neighbor + 8 * size_t(i));
  float4* wo = reinterpret_cast<float4*>(weight + 8 * size_t(i));
  no[0] = make_uint4(nb[0], nb[1], nb[2], nb[3]);
  no[1] = make_uint4(nb[4], nb[5], nb[6], nb[7]);
  wo[0] = make_float4(w[0] * inv, w[1] * inv, w[2] * inv, w[3] * inv);
  wo[1] = make_float4(w[4] * inv, w[5] * inv, w[6] * inv, w[7] * inv);
}

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 t = __ldg(reinterpret_cast<const float4*>(p));
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
  const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x)),
               b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, const float (&v)[4]) {
  const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// out[m, :] = sum_k weight[m, k] * feats[indices[m, k], :] over the valid entries (weight == null: every weight 1).
// A thread owns four consecutive channels of one output row; the rows of a warp are consecutive, so the index and
// weight loads coalesce and every feature load is 8 or 16 bytes of a gathered row.
template <typename T>
__global__ void __launch_bounds__(256) weighted_gather_kernel(const T* __restrict__ feats, const uint32_t* __restrict__ indices,
                                                             const float* __restrict__ weight, T* __restrict__ out, int64_t M, int C,
                                                             int V) {
  const int c4 = C / 4;
  const int64_t e = blockIdx.x * int64_t(256) + threadIdx.x;
  if (e >= M * c4) return;
  const int64_t m = e / c4;
  const int c = static_cast<int>(e - m * c4) * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < V; ++k) {
    const uint32_t row = __ldg(&indices[m * V + k]);
    if (row == kInvalid) continue;
    const float w = weight != nullptr ? __ldg(&weight[m * V + k]) : 1.f;
    float v[4];
    load4<T>(feats + size_t(row) * C + c, v);
    acc[0] += w * v[0], acc[1] += w * v[1], acc[2] += w * v[2], acc[3] += w * v[3];
  }
  store4<T>(out + m * C + c, acc);
}

// grad_feats_f32[indices[m, k], :] += weight[m, k] * grad_out[m, :]   (fp32 atomics; the caller zeroes the buffer)
template <typename T>
__global__ void __launch_bounds__(256) weighted_scatter_kernel(const T* __restrict__ grad_out, const uint32_t* __restrict__ indices,
                                                              const float* __restrict__ weight, float* __restrict__ grad_feats, int64_t M,
                                                              int C, int V) {
  const int c4 = C / 4;
  const int64_t e = blockIdx.x * int64_t(256) + threadIdx.x;
  if (e >= M * c4) return;
  const int64_t m = e / c4;
  const int c = static_cast<int>(e - m * c4) * 4;
  float g[4];
  load4<T>(grad_out + m * C + c, g);
  for (int k = 0; k < V; ++k) {
    const uint32_t row = __ldg(&indices[m * V + k]);
    if (row == kInvalid) continue;
    const float w = weight != nullptr ? __ldg(&weight[m * V + k]) : 1.f;
    float* dst = grad_feats + size_t(row) * C + c;
    atomicAdd(dst + 0, w * g[0]);
    atomicAdd(dst + 1, w * g[1]);
    atomicAdd(dst + 2, w * g[2]);
    atomicAdd(dst + 3, w * g[3]);
  }
}

static int check_table(const void* table, int64_t slots, int key_bits) {
  if (key_bits != 32 && key_bits != 64) return FGB_E_DTYPE;
  if (slots < 1 || slots >= (int64_t(1) << 31)) return FGB_E_SIZE;
  if (!table) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(table) & 7) return FGB_E_ALIGN;
  return FGB_OK;
}

static int elem_code_ok(int dtype) { return dtype == FGB_F16 || dtype == FGB_BF16 || dtype == FGB_F32_TF32 || dtype == FGB_F32_IEEE; }

}  // namespace fgb

extern "C" int fgb_hash_insert_3d_idx_as_val(const int32_t* coords, int64_t n, int W, int H, int D, void* table, int64_t slots,
                                             int key_bits, int32_t* status, void* stream) {
  using namespace fgb;
  if (n < 0 || n >= (int64_t(1) << 32) - 1 || W <= 0 || H <= 0 || D <= 0) return FGB_E_SIZE;
  int rc = check_table(table, slots, key_bits);
  if (rc != FGB_OK) return rc;
  if (slots < n) return FGB_E_SIZE;
  if (n > 0 && !coords) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(coords) & 15) return FGB_E_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t words = static_cast<size_t>(fgb_hash_table_bytes(slots, key_bits)) / 4;
  const unsigned grid = static_cast<unsigned>(std::min<size_t>((words + 2047) / 2048, 148 * 16));
  fill_words_kernel<<<grid > 0 ? grid : 1, 256, 0, s>>>(static_cast<uint32_t*>(table), words, 0xFFFFFFFFu);
  if (n == 0) return launch_status();
  const Grid3 g{W, H, D};
  const unsigned blocks = static_cast<unsigned>(ceil_div(n, kMapBlock));
  if (key_bits == 32)
    hash_insert_kernel<32><<<blocks, kMapBlock, 0, s>>>(reinterpret_cast<const int4*>(coords), static_cast<uint32_t>(n), g, table,
                                                       static_cast<uint32_t>(slots), status, nullptr);
  else
    hash_insert_kernel<64><<<blocks, kMapBlock, 0, s>>>(reinterpret_cast<const int4*>(coords), static_cast<uint32_t>(n), g, table,
                                                       static_cast<uint32_t>(slots), status, nullptr);
  return launch_status();
}

extern "C" int fgb_hash_lookup_3d(const int32_t* query_coords, int64_t m, int W, int H, int D, void* table, int64_t slots, int key_bits,
                                  uint32_t* out_rows, void* stream) {
  using namespace fgb;
  if (m < 0 || m >= (int64_t(1) << 32) - 1 || W <= 0 || H <= 0 || D <= 0) return FGB_E_SIZE;
  int rc = check_table(table, slots, key_bits);
  if (rc != FGB_OK) return rc;
  if (m == 0) return FGB_OK;
  if (!query_coords || !out_rows) return FGB_E_NULL;
  if (reinterpret_cast<uintptr_t>(query_coords) & 15) return FGB_E_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Grid3 g{W, H, D};
  const unsigned blocks = static_cast<unsigned>(ceil_div(m, 256));
  if (key_bits == 32)
    hash_lookup_3d_kernel<32><<<blocks, 256, 0, s>>>(reinterpret_cast<const int4*>(query_coords), static_cast<uint32_t>(m), g, table,
                                                    static_cast<uint32_t>(slots), out_rows);
  else
    hash_lookup_3d_kernel<64><<<blocks, 256, 0, s>>>(reinterpret_cast<const int4*>(query_coords), static_cast<uint32_t>(m), g, table,
                                                    static_cast<uint32_t>(slots), out_rows);
  return launch_status();
}

extern "C" int fgb_grid_sample_neighbor_map(const float* query, int64_t B, int64_t L, int W, int H, int D, void* table, int64_t slots,
                                            int key_bits, int trilinear, uint32_t* neighbor, float* weight, void* stream) {
  using namespace fgb;
  if (B < 0 || L < 0 || B * L >= (int64_t(1) << 28) || W <= 0 || H <= 0 || D <= 0) return FGB_E_SIZE;
  int rc = check_table(table, slots, key_bits);
  if (rc != FGB_OK) return rc;
  if (B * L == 0) return FGB_OK;
  if (!query || !neighbor || (trilinear && !weight)) return FGB_E_NULL;
  if (trilinear && ((reinterpret_cast<uintptr_t>(neighbor) | reinterpret_cast<uintptr_t>(weight)) & 15)) return FGB_E_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Grid3 g{W, H, D};
  const unsigned blocks = static_cast<unsigned>(ceil_div(B * L, 256));
  const uint32_t b = static_cast<uint32_t>(B), l = static_cast<uint32_t>(L), sl = static_cast<uint32_t>(slots);
  if (trilinear) {
    if (key_bits == 32) trilinear_map_kernel<32><<<blocks, 256, 0, s>>>(query, b, l, g, table, sl, neighbor, weight);
    else trilinear_map_kernel<64><<<blocks, 256, 0, s>>>(query, b, l, g, table, sl, neighbor, weight);
  } else {
    if (key_bits == 32) nearest_map_kernel<32><<<blocks, 256, 0, s>>>(query, b, l, g, table, sl, neighbor);
    else nearest_map_kernel<64><<<blocks, 256, 0, s>>>(query, b, l, g, table, sl, neighbor);
  }
  return launch_status();
}

extern "C" int fgb_indice_weighted_sum_fwd(const void* feats, const uint32_t* indices, const float* weight, void* out, int64_t M,
                                           int C, int V, int dtype, void* stream) {
  using namespace fgb;
  if (!elem_code_ok(dtype)) return FGB_E_DTYPE;
  if (M < 0 || C <= 0 || V < 1 || V > 64) return FGB_E_SIZE;
  if (C % 4) return FGB_E_ALIGN;
  if (M == 0) return FGB_OK;
  if (!feats || !indices || !out) return FGB_E_NULL;
  if ((reinterpret_cast<uintptr_t>(feats) | reinterpret_cast<uintptr_t>(out)) & 15) return FGB_E_ALIGN;
  const int64_t blocks = ceil_div(M * (C / 4), 256);
  if (blocks > 0x7FFFFFFF) return FGB_E_SIZE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned g = static_cast<unsigned>(blocks);
  if (dtype == FGB_F16)
    weighted_gather_kernel<__half><<<g, 256, 0, s>>>(static_cast<const __half*>(feats), indices, weight, static_cast<__half*>(out), M, C, V);
  else if (dtype == FGB_BF16)
    weighted_gather_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(feats), indices, weight,
                                                            static_cast<__nv_bfloat16*>(out), M, C, V);
  else
    weighted_gather_kernel<float><<<g, 256, 0, s>>>(static_cast<const float*>(feats), indices, weight, static_cast<float*>(out), M, C, V);
  return launch_status();
}

extern "C" int fgb_indice_weighted_sum_bwd(const void* grad_out, const uint32_t* indices, const float* weight, float* grad_feats_f32,
                                           int64_t M, int64_t N, int C, int V, int dtype, void* stream) {
  using namespace fgb;
  if (!elem_code_ok(dtype)) return FGB_E_DTYPE;
  if (M < 0 || N < 0 || C <= 0 || V < 1 || V > 64) return FGB_E_SIZE;
  if (C % 4) return FGB_E_ALIGN;
  if (N > 0 && !grad_feats_f32) return FGB_E_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N > 0) {
    int rc = cuda_status(cudaMemsetAsync(grad_feats_f32, 0, static_cast<size_t>(N) * C * sizeof(float), s));
    if (rc != FGB_OK) return rc;
  }
  if (M == 0 || N == 0) return FGB_OK;
  if (!grad_out || !indices) return FGB_E_NULL;
  if ((reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(grad_feats_f32)) & 15) return FGB_E_ALIGN;
  const int64_t blocks = ceil_div(M * (C / 4), 256);
  if (blocks > 0x7FFFFFFF) return FGB_E_SIZE;
  const unsigned g = static_cast<unsigned>(blocks);
  if (dtype == FGB_F16)
    weighted_scatter_kernel<__half><<<g, 256, 0, s>>>(static_cast<const __half*>(grad_out), indices, weight, grad_feats_f32, M, C, V);
  else if (dtype == FGB_BF16)
    weighted_scatter_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(grad_out), indices, weight, grad_feats_f32, M,
                                                             C, V);
  else
    weighted_scatter_kernel<float><<<g, 256, 0, s>>>(static_cast<const float*>(grad_out), indices, weight, grad_feats_f32, M, C, V);
  return launch_status();
}
