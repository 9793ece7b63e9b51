// Next-token sampler: logit top-k mask + Gumbel-max (inference/sampler.go:16-77,
// tensors/random.go:60-80), one CTA per row.
//
// The reference walks each row sequentially: it keeps the k largest values in a
// sorted array to find the k-th largest, masks everything below it to -inf
// (values EQUAL to the threshold survive, so ties can keep more than k), draws
// one uniform per vocabulary entry, and keeps the first maximum of
// value/temperature - log(-log(u)).  Here the row is read from HBM once into
// registers, the k-th largest value is found exactly by an 8-bit radix select
// on the order-preserving integer image of the floats (for small k a candidate
// filter finds it without the histograms), and only the survivors
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
// The rollout engine's per-row bookkeeping after a sampling step (inference/engine.go:260-319, 349-367), done by the
// row's own CTA: the row's position advances past the token that was just forwarded, its context length for the next
// step follows, a queued forced token replaces the sampled one, the thinking budget is enforced, and the token is
// either kept or ends the row (<|bos|>, <|assistant_end|>).  Returns the token the row forwards next.
__device__ __forceinline__ int32_t sample_tail(const SampleTail& t, int row, int32_t token) {
  int32_t mask = 1;
  if (t.forced_len && t.forced_len[row] > 0) {   // a queued token overrides the sampled one (the draw is still consumed)
    const int head = t.forced_head[row];
    token = t.forced_buf[(int64_t)row * t.forced_cap + head];
    t.forced_head[row] = (head + 1) % t.forced_cap; t.forced_len[row] -= 1;
    mask = 0;
  }
  if (t.step_mask) t.step_mask[row] = mask;
  if (t.pos) { const int32_t pn = t.pos[row] + t.advance; t.pos[row] = pn; if (t.ctxlen) t.ctxlen[row] = pn + 1; }
  if (t.thinking && t.in_think) {
    if (token == t.think_start) { t.in_think[row] = 1; t.think_count[row] = 0; }
    else if (token == t.think_end && t.in_think[row]) t.in_think[row] = 0;
    else if (t.in_think[row]) {
      const int n = t.think_count[row] + 1;
      t.think_count[row] = n;
      if (t.thinking_budget > 0 && n >= t.thinking_budget && t.forced_len && t.forced_len[row] < t.forced_cap) {
        t.forced_buf[(int64_t)row * t.forced_cap + (t.forced_head[row] + t.forced_len[row]) % t.forced_cap] = t.think_end;
        t.forced_len[row] += 1;
      }
    }
  }
  if (t.done && !t.done[row]) {
    if (token == t.aend || token == t.bos) { t.done[row] = 1; atomicAdd(t.n_done, 1); }
    else {
      const int n = t.out_lengths[row];
      if (n < t.max_tokens) {
        t.out_tokens[(int64_t)row * t.max_tokens + n] = token;
        if (t.out_masks) t.out_masks[(int64_t)row * t.max_tokens + n] = mask;
        t.out_lengths[row] = n + 1;
      }
    }
  }
  return token;
}

template <int IPT>
__global__ void __launch_bounds__(ST) sample_kernel(const float* __restrict__ logits, int vocab, int row_div, const float* __restrict__ uniforms,
                                                    const uint64_t* __restrict__ seeds, int group, const uint32_t* step_dev, uint32_t step_host,
                                                    float temperature, int top_k, int32_t* __restrict__ out, SampleTail tail) {
  __shared__ unsigned int hist[32][256];  // one histogram per warp
  __shared__ unsigned int total[256];
  __shared__ unsigned int sel_prefix, sel_remaining, warp_count[32];
  __shared__ float sel_threshold;
  __shared__ float shs[32];
  __shared__ int shi[32];

  pdl_trigger();
  pdl_wait();
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
    if (tid == 0) { const int32_t t = b.index == 0x7fffffff ? 0 : b.index; out[row] = sample_tail(tail, row, t); }
    return;
  }

  float threshold = -INFINITY;
  const bool mask = top_k > 0 && top_k < vocab;
  bool found = false;
  unsigned n_cand = 0;
  // Fast path for small k.  Take, per warp, the m = ceil(k/32) largest of its threads' maxima: these are 32m >= k
  // distinct entries, so the k-th largest of the row is at least t0 = the smallest of them, and every entry >= t0 is
  // a candidate (a few hundred for ordinary logits).  The exact k-th largest is then found among the candidates by
  // counting ranks.  Rows with more candidates than fit (many equal values) take the radix select below.
  constexpr unsigned kWarpCand = 64, kCand = 32 * kWarpCand;  // 4 * kCand words = the histogram storage
  const int m_per_warp = (top_k + 31) / 32;
  if (mask && m_per_warp <= 4) {
    float* warp_val = reinterpret_cast<float*>(&hist[0][0]);            // [32 warps][kWarpCand]
    int* warp_idx = reinterpret_cast<int*>(&hist[0][0]) + kCand;         // [32 warps][kWarpCand]
    float* cand = reinterpret_cast<float*>(&hist[0][0]) + 2 * kCand;     // packed [kCand]
    int* cand_index = reinterpret_cast<int*>(&hist[0][0]) + 3 * kCand;   // packed [kCand]
    const int lane = tid & 31;
    float tmax = -INFINITY;
#pragma unroll
    for (int it = 0; it < IPT; ++it) tmax = fmaxf(tmax, x[it]);
    float v = tmax, tw = -INFINITY;
    for (int r = 0; r < m_per_warp; ++r) {
      float w = v;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, o));
      tw = w;
      const unsigned holders = __ballot_sync(0xffffffffu, v == w);
      if (lane == __ffs(holders) - 1) v = -INFINITY;  // one holder leaves; ties stay for the next round
    }
    if (lane == 0) shs[warp] = tw;
    __syncthreads();
    float t0 = shs[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t0 = fminf(t0, __shfl_xor_sync(0xffffffffu, t0, o));
    // Each warp lists its own candidates (positions from ballots, no atomics), then the lists are packed.
    unsigned mine_count = 0;
    const unsigned below = (1u << lane) - 1u;
#pragma unroll
    for (int it = 0; it < IPT; ++it) {
      const bool pred = it * ST + tid < vocab && x[it] >= t0;
      const unsigned votes = __ballot_sync(0xffffffffu, pred);
      if (votes) {
        const unsigned pos = mine_count + __popc(votes & below);
        if (pred && pos < kWarpCand) { warp_val[warp * kWarpCand + pos] = x[it]; warp_idx[warp * kWarpCand + pos] = it * ST + tid; }
        mine_count += __popc(votes);
      }
    }
    if (lane == 0) warp_count[warp] = mine_count;
    __syncthreads();
    const unsigned cnt_l = warp_count[lane];
    const bool overflow = __any_sync(0xffffffffu, cnt_l > kWarpCand);
    unsigned incl = cnt_l;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const unsigned t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
    const unsigned C = __shfl_sync(0xffffffffu, incl, 31);
    const unsigned offset = __shfl_sync(0xffffffffu, incl - cnt_l, warp);
    if (!overflow)
      for (unsigned j = lane; j < mine_count; j += 32) { cand[offset + j] = warp_val[warp * kWarpCand + j]; cand_index[offset + j] = warp_idx[warp * kWarpCand + j]; }
    __syncthreads();
    if (!overflow) {
      for (unsigned i = tid; i < C; i += ST) {
        const float mine = cand[i];
        int greater = 0, not_less = 0;
#pragma unroll 4
        for (unsigned j = 0; j < C; ++j) { const float other = cand[j]; greater += other > mine; not_less += other >= mine; }
        if (greater < top_k && not_less >= top_k) sel_threshold = mine;  // every writer holds the same value
      }
      found = true;
    }
    __syncthreads();
    if (found) threshold = sel_threshold;
    n_cand = found ? C : 0u;
  }
  if (mask && !found) {
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
  // with the engine tail the step is the number of tokens this row has sampled so far: its position past the prompt
  const uint32_t step = tail.pos ? (uint32_t)(tail.pos[row] - tail.pos_base + tail.advance) : (step_dev ? *step_dev : step_host);
  Best b{-INFINITY, 0x7fffffff};
  auto consider = [&](float value, int c) {
    float u = uniforms ? uniforms[(int64_t)row * vocab + c] : sampler_uniform(seed, step, grow, (uint32_t)c);
    if (u <= 0.0f) u = 1e-12f;
    float gumbel = -(float)log(-log((double)u));
    float score = __fadd_rn(__fdiv_rn(value, temperature), gumbel);
    best_merge(b, score, c);
  };
  if (found) {
    // The survivors are among the candidates: one thread per survivor, so the float64 logarithms of the whole row
    // run side by side instead of once per warp that happens to hold a survivor.
    const float* cand = reinterpret_cast<const float*>(&hist[0][0]) + 2 * kCand;
    const int* cand_index = reinterpret_cast<const int*>(&hist[0][0]) + 3 * kCand;
    for (unsigned i = tid; i < n_cand; i += ST)
      if (cand[i] >= threshold) consider(cand[i], cand_index[i]);
  } else {
#pragma unroll
    for (int it = 0; it < IPT; ++it) {
      int c = it * ST + tid;
      if (c >= vocab) continue;
      float value = x[it];
      if (mask && !(value >= threshold)) continue;  // masked to -inf: can never beat a survivor
      consider(value, c);
    }
  }
  b = block_best(b, shs, shi);
  if (tid == 0) { const int32_t t = b.index == 0x7fffffff ? 0 : b.index; out[row] = sample_tail(tail, row, t); }
}

int sample_launch(const float* logits, int rows, int vocab, int logits_row_div, const float* uniforms, const uint64_t* seeds_dev, int group,
                  const uint32_t* step_dev, uint32_t step_host, float temperature, int top_k, int32_t* out, cudaStream_t s, const SampleTail* tail_in) {
  SampleTail tail{};
  if (tail_in) tail = *tail_in;
  if (rows <= 0) return GN_OK;
  GN_REQUIRE(vocab > 0 && vocab <= 64 * ST, "sampler: vocabulary %d outside (0, %d]", vocab, 64 * ST);
  if (logits_row_div < 1) logits_row_div = 1;
  if (group < 1) group = 1;
#define GN_SAMPLE(IPT) GN_CUDA(launch_pdl(sample_kernel<IPT>, dim3(rows), dim3(ST), 0, s, logits, vocab, logits_row_div, uniforms, seeds_dev, group, step_dev, step_host, temperature, top_k, out, tail))
  if (vocab <= 8 * ST) { GN_SAMPLE(8); }
  else if (vocab <= 16 * ST) { GN_SAMPLE(16); }
  else if (vocab <= 32 * ST) { GN_SAMPLE(32); }
  else { GN_SAMPLE(64); }
#undef GN_SAMPLE
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
