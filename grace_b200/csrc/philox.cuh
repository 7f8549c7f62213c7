// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
// Convention used by every stochastic kernel here, and restated in
// grace_b200/utils/philox.py for the CPU oracle:
//   key     = (seed_lo, seed_hi)
//   counter = (group_lo, group_hi, step, stream)
// where `group` indexes four consecutive flat elements; element 4*group+j uses
// output word j.  uniform = (word >> 8) * 2^-24, exact in fp32, in [0,1).
#pragma once
#include <cstdint>

namespace grace {

struct Philox4 {
  unsigned x, y, z, w;
};

__host__ __device__ __forceinline__ Philox4 philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3,
                                                          unsigned k0, unsigned k1) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const unsigned n0 = (unsigned)(p1 >> 32) ^ c1 ^ k0;
    const unsigned n1 = (unsigned)p1;
    const unsigned n2 = (unsigned)(p0 >> 32) ^ c3 ^ k1;
    const unsigned n3 = (unsigned)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}

__host__ __device__ __forceinline__ Philox4 philox_group(uint64_t group, unsigned step, unsigned stream, uint64_t seed) {
  return philox4x32_10((unsigned)group, (unsigned)(group >> 32), step, stream, (unsigned)seed, (unsigned)(seed >> 32));
}

__host__ __device__ __forceinline__ float u01(unsigned word) { return (float)(word >> 8) * 5.9604644775390625e-08f; }

}  // namespace grace
