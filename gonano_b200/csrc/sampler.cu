// Next-token sampler: logit top-k mask + Gumbel-max (inference/sampler.go:16-77,
// tensors/random.go:60-80), one CTA per row.
//
// The reference walks each row sequentially: it keeps the k largest values in a
// sorted array to find the k-th largest, masks everything below it to -inf
// (values EQUAL to the threshold survive, so ties can keep more than k), draws
// one uniform per vocabulary entry, and keeps the first maximum of
// value/temperature - log(-log(u)).  Here the row is read from HBM once into
// registers, the k-th largest value is found exactly by an 8-bit radix select
// on the order-preserving integer image of the floats, and only the survivors
// pay for the uniform and the float64 logarithms.  Uniforms are addressed by
// counter, so skipping the masked entries changes nothing.
#include "kernels.cuh"
#include "philox.cuh"

namespace gn {

constexpr int ST = 1024;  // threads per row

__device__ __forceinline__ uint32_t order_bits(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unorder_bits(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

struct Best { float score; int index; };
__device__ __forceinline__ void best_merge(Best& a, float s, int i) {
  if (s > a.score || (s == a.score && i < a.index)) { a.score = s; a.index = i; }
}
__device__ __forceinline__ Best block_best(Best b, float* shs, int* shi) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float os = __shfl_xor_sync(0xffffffffu, b.score, o);
    int oi = __shfl_xor_sync(0xffffffffu, b.index, o);
    best_merge(b, os, oi);
  }
  __syncthreads();
  if (lane == 0) { shs[warp] = b.score; shi[warp] = b.index; }
  __syncthreads();
  if (warp == 0) {
    int nw = blockDim.x >> 5;
    b.score = lane < nw ? shs[lane] : -INFINITY; b.index = lane < nw ? shi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float os = __shfl_xor_sync(0xffffffffu, b.score, o);
      int oi = __shfl_xor_sync(0xffffffffu, b.index, o);
      best_merge(b, os, oi);
    }
    if (lane == 0) { shs[0] = b.score; shi[0] = b.index; }
  }
  __syncthreads();
  b.score = shs[0]; b.index = shi[0];
  return b;
}

// IPT = vocabulary entries held per thread (vocab <= IPT * 1024).
template <int IPT>
__global__ void __launch_bounds__(ST) sample_kernel(const float* __restrict__ logits, int vocab, int row_div, const float* __restrict__ uniforms,
                                                    const uint64_t* __restrict__ seeds, int group, const uint32_t* step_dev, uint32_t step_host,
                                                    float temperature, int top_k, int32_t* __restrict__ out) {
  __shared__ unsigned int hist[32][256];  // one histogram per warp
  __shared__ unsigned int total[256];
  __shared__ unsigned int sel_prefix, sel_remaining;
  __shared__ float shs[32];
  __shared__ int shi[32];

  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5;
  const float* src = logits + (int64_t)(row / row_div) * vocab;
  float x[IPT];
#pragma unroll
  for (int it = 0; it < IPT; ++it) {
    int c = it * ST + tid;
    x[it] = c < vocab ? src[c] : -INFINITY;
  }

  if (temperature <= 0.0f) {  // plain argmax, first maximum (inference/sampler.go:37-45)
    Best b{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int it = 0; it < IPT; ++it) { int c = it * ST + tid; if (c < vocab) best_merge(b, x[it], c); }
    b = block_best(b, shs, shi);
    if (tid == 0) out[row] = b.index == 0x7fffffff ? 0 : b.index;
    return;
  }

  float threshold = -INFINITY;
  const bool mask = top_k > 0 && top_k < vocab;
  if (mask) {
    if (tid == 0) { sel_prefix = 0u; sel_remaining = (unsigned)top_k; }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = tid; i < 32 * 256; i += ST) (&hist[0][0])[i] = 0u;
      __syncthreads();
      const unsigned prefix = sel_prefix;
      const unsigned pmask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
#pragma unroll
      for (int it = 0; it < IPT; ++it) {
        int c = it * ST + tid;
        if (c < vocab) {
          unsigned u = order_bits(x[it]);
          if ((u & pmask) == prefix) atomicAdd(&hist[warp][(u >> shift) & 255u], 1u);
        }
      }
      __syncthreads();
      if (tid < 256) {
        unsigned t = 0;
#pragma unroll
        for (int w = 0; w < 32; ++w) t += hist[w][tid];
        total[tid] = t;
      }
      __syncthreads();
      if (warp == 0) {
        // Walk from the largest digit down until the k-th largest falls inside
        // a bin: lane l owns bins [8l, 8l+8); a suffix sum over lanes finds the
        // lane whose bins contain the crossing.
        const int lane = tid & 31;
        unsigned cnt[8], lsum = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) { cnt[e] = total[lane * 8 + e]; lsum += cnt[e]; }
        unsigned incl = lsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          unsigned t = __shfl_down_sync(0xffffffffu, incl, o);
          if (lane + o < 32) incl += t;
        }
        const unsigned above = incl - lsum;
        const unsigned remaining = sel_remaining;
        __syncwarp();
        if (above < remaining && remaining <= above + lsum) {
          unsigned rem = remaining - above, digit = (unsigned)(lane * 8);
          for (int e = 7; e >= 0; --e) {
            if (cnt[e] >= rem) { digit = (unsigned)(lane * 8 + e); break; }
            rem -= cnt[e];
          }
          sel_remaining = rem;
          sel_prefix = prefix | (digit << shift);
        }
      }
      __syncthreads();
    }
    threshold = unorder_bits(sel_prefix);
  }

  const uint64_t seed = seeds ? seeds[row / group] : 0ull;
  const uint32_t grow = (uint32_t)(row % group);
  const uint32_t step = step_dev ? *step_dev : step_host;
  Best b{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int it = 0; it < IPT; ++it) {
    int c = it * ST + tid;
    if (c >= vocab) continue;
    float value = x[it];
    if (mask && !(value >= threshold)) continue;  // masked to -inf: can never beat a survivor
    float u = uniforms ? uniforms[(int64_t)row * vocab + c] : sampler_uniform(seed, step, grow, (uint32_t)c);
    if (u <= 0.0f) u = 1e-12f;
    float gumbel = -(float)log(-log((double)u));
    float score = __fadd_rn(__fdiv_rn(value, temperature), gumbel);
    best_merge(b, score, c);
  }
  b = block_best(b, shs, shi);
  if (tid == 0) out[row] = b.index == 0x7fffffff ? 0 : b.index;
}

int sample_launch(const float* logits, int rows, int vocab, int logits_row_div, const float* uniforms, const uint64_t* seeds_dev, int group,
                  const uint32_t* step_dev, uint32_t step_host, float temperature, int top_k, int32_t* out, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  GN_REQUIRE(vocab > 0 && vocab <= 64 * ST, "sampler: vocabulary %d outside (0, %d]", vocab, 64 * ST);
  if (logits_row_div < 1) logits_row_div = 1;
  if (group < 1) group = 1;
#define GN_SAMPLE(IPT) sample_kernel<IPT><<<rows, ST, 0, s>>>(logits, vocab, logits_row_div, uniforms, seeds_dev, group, step_dev, step_host, temperature, top_k, out)
  if (vocab <= 8 * ST) GN_SAMPLE(8);
  else if (vocab <= 16 * ST) GN_SAMPLE(16);
  else if (vocab <= 32 * ST) GN_SAMPLE(32);
  else GN_SAMPLE(64);
#undef GN_SAMPLE
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
