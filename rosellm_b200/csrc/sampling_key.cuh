// What the sampling kernels and the head product that samples in its epilogue share: the order-
// preserving bit pattern of a logit, the Gumbel noise of a vocabulary entry, and the choice
// between two candidates.  One definition, so that both give the same token bit for bit.
#pragma once

#include <math_constants.h>

#include "common.cuh"

namespace rl {

__device__ __forceinline__ uint32_t ordered_bits(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t philox_first(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
  uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

// Gumbel noise of vocabulary entry `index` for the `counter`-th generated token of a request.
__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint32_t counter, uint32_t index) {
  const uint32_t x = philox_first(index, counter, (uint32_t)seed, (uint32_t)(seed >> 32));
  const float u = ((float)(x >> 8) + 0.5f) * 5.9604644775390625e-08f;  // (0, 1), 2^-24 steps
  return -logf(-logf(u));
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// The score a sampled row maximises: logit / temperature + noise, in one rounding.
__device__ __forceinline__ float sample_key(float logit, float inv_t, uint64_t seed, uint32_t counter, uint32_t index) {
  return __fmaf_rn(logit, inv_t, gumbel_noise(seed, counter, index));
}

}  // namespace rl
