// TEST INFRASTRUCTURE (CPU oracle). Not part of the shipped library.
//
// Philox-4x32-10 counter-based generator (Salmon et al., "Parallel random
// numbers: as easy as 1, 2, 3", SC'11), restated from the published
// algorithm.  The reference draws its sampler uniforms from Go's
// math/rand/v2 PCG (tensors/random.go:16-21), whose source is not available
// to this build; the reference's tests pin no draw value, so the CUDA library
// and this oracle share this documented generator instead.  The same routine
// is restated in gonano_b200/csrc/philox.cuh; tests compare the two.
#pragma once
#include <cstdint>

namespace gnrng {

struct U4 { uint32_t v[4]; };

static inline void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  uint64_t p = (uint64_t)a * (uint64_t)b;
  hi = (uint32_t)(p >> 32);
  lo = (uint32_t)p;
}

static inline U4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                               uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int round = 0; round < 10; ++round) {
    uint32_t hi0, lo0, hi1, lo1;
    mulhilo(M0, c0, hi0, lo0);
    mulhilo(M1, c2, hi1, lo1);
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  U4 out; out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// Uniform float32 in [0,1) with 24 random bits.
static inline float u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }

// The sampler's uniform for (seed, step, row, vocab column): one uniform per
// vocabulary entry per row per decode step, as the reference consumes them
// (tensors/random.go:60-80), addressed by counter instead of by order.
static inline float sampler_uniform(uint64_t seed, uint32_t step, uint32_t row, uint32_t column) {
  U4 r = philox4x32_10(column >> 2, row, step, 0u, (uint32_t)seed, (uint32_t)(seed >> 32));
  return u01(r.v[column & 3u]);
}

// Stream 1: per-rollout synthetic rewards.
static inline float reward_uniform(uint64_t seed, uint32_t rollout) {
  U4 r = philox4x32_10(rollout, 0u, 0u, 1u, (uint32_t)seed, (uint32_t)(seed >> 32));
  return u01(r.v[0]);
}

}  // namespace gnrng
