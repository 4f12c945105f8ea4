// Philox-4x32-10 counter-based generator, identical on the host (C++), in CUDA and in the NumPy oracle.
// Element i of a stream is a pure function of (seed, i), so any split of the index space over workers or
// GPUs produces the same values.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200 {

struct Philox4 { uint32_t v[4]; };

B200_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * b;
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}

B200_HD Philox4 philox4x32_10(uint64_t counter, uint64_t seed) {
  uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c0, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// uniform in [-1, 1) with 24 bits of resolution
B200_HD float u32_to_uniform_pm1(uint32_t x) { return static_cast<float>(x >> 8) * (2.0f / 16777216.0f) - 1.0f; }

// element `i` of the uniform[-1,1) stream of `seed`
B200_HD float philox_uniform_pm1(uint64_t i, uint64_t seed) {
  const Philox4 r = philox4x32_10(i >> 2, seed);
  return u32_to_uniform_pm1(r.v[i & 3]);
}

}  // namespace b200
