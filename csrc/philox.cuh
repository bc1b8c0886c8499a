// Counter-based random numbers (Philox-4x32 with ten rounds, Salmon et al. 2011) for the
// kernels that draw inside the kernel: dropout masks and Gumbel noise for sampling. A draw is
// a pure function of (seed, stream, index), so the backward pass of a dropout regenerates the
// mask of its forward pass from three integers, and ranks that hold copies of the same
// activation rows draw the same mask without exchanging anything.
#pragma once
#include <stdint.h>

namespace t5x {

struct Philox4 {
  uint32_t x, y, z, w;
};

__host__ __device__ __forceinline__ void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi,
                                                        uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * static_cast<uint64_t>(b);
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}

// Four 32-bit words for counter (index_lo, index_hi, stream, 0) under key (seed_lo, seed_hi).
__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint64_t seed, uint32_t stream,
                                                          uint64_t index) {
  uint32_t c0 = static_cast<uint32_t>(index), c1 = static_cast<uint32_t>(index >> 32), c2 = stream,
           c3 = 0u;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c0, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0;
    c1 = n1;
    c2 = n2;
    c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}

// Uniform in (0, 1): never 0 or 1, so that log(u) and log(-log(u)) are finite.
__host__ __device__ __forceinline__ float philox_uniform(uint32_t bits) {
  return (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

}  // namespace t5x
