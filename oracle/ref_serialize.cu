// Host driver around the reference's own serialisation headers
// (flex_gemm/kernels/cuda/serialize/z_order.h, hilbert.h), used once to produce
// golden Morton / Hilbert keys for the oracle.  TEST INFRASTRUCTURE ONLY.
//
// Build (the include path points into the FlexGEMM tree; nothing is copied):
//   nvcc -O1 -I<FlexGEMM>/flex_gemm/kernels/cuda -o oracle/_ref/ref_serialize oracle/ref_serialize.cu
// Input on stdin: "<bits> <n>" then n lines "b x y z"; output: n lines
// "<morton64> <hilbert64> <morton32> <hilbert32>" (the 32-bit pair is 0 0 when
// the key does not fit 32 bits, i.e. when batch bits + 3 * bits >= 32).
#include <cstdint>
#include <cstdio>
#include <limits>

#include "serialize/z_order.h"
#include "serialize/hilbert.h"

int main() {
  int bits = 0;
  long n = 0;
  if (scanf("%d %ld", &bits, &n) != 2) return 1;
  for (long i = 0; i < n; ++i) {
    unsigned b, x, y, z;
    if (scanf("%u %u %u %u", &b, &x, &y, &z) != 4) return 1;
    uint64_t m64 = 0, h64 = 0;
    uint32_t m32 = 0, h32 = 0;
    flex_gemm::serialize::z_order_encode<uint64_t>(b, x, y, z, static_cast<size_t>(bits), m64);
    flex_gemm::serialize::hilbert_encode<uint64_t>(b, x, y, z, static_cast<size_t>(bits), h64);
    int bb = 0;
    for (unsigned t = b; t; t >>= 1) ++bb;
    if (bb + 3 * bits < 32) {
      flex_gemm::serialize::z_order_encode<uint32_t>(b, x, y, z, static_cast<size_t>(bits), m32);
      flex_gemm::serialize::hilbert_encode<uint32_t>(b, x, y, z, static_cast<size_t>(bits), h32);
    }
    printf("%llu %llu %u %u\n", (unsigned long long)m64, (unsigned long long)h64, m32, h32);
  }
  return 0;
}
