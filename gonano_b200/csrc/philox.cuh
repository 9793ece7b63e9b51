// Philox-4x32-10 counter-based generator (Salmon et al., SC'11), the generator
// behind the sampler's uniforms when the caller passes none.  The reference
// draws from Go's math/rand/v2 PCG (tensors/random.go:16-21); this library
// documents its own counter layout instead, so that every uniform is addressed
// by (seed, step, row, column) and rows can be sampled in parallel.
#pragma once
#include <cstdint>

namespace gn {

__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                                       uint32_t (&out)[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)M0 * c0, p1 = (uint64_t)M1 * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// 24 random bits -> [0,1).
__host__ __device__ __forceinline__ float philox_u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }

// Uniform of (seed, decode step, row within the group, vocabulary column).
__host__ __device__ __forceinline__ float sampler_uniform(uint64_t seed, uint32_t step, uint32_t row, uint32_t column) {
  uint32_t r[4];
  philox4x32_10(column >> 2, row, step, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
  return philox_u01(r[column & 3u]);
}

}  // namespace gn
