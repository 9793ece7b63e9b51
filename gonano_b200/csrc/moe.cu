// Router top-k, gate, grouped expert GEMM and the lightning-indexer scores
// (kernels/backend.go:103-141; scalar statement kernels/scalar/moe.go:8-73,
// kernels/scalar/indexer.go:11-61).  Routing runs one warp per token row with
// the row's scores held in shared memory; indices are exact: descending score,
// ties toward the smaller index.
#include "kernels.cuh"

namespace gn {

// Each warp owns one row.  Scores are staged to shared memory (count <= 1024
// per warp slot) or read from global for wider rows.
constexpr int TOPK_WARPS = 4;
constexpr int TOPK_SMEM_COLS = 1024;

__device__ __forceinline__ void warp_argmax_first(float& best, int& bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
}

// scores = logits (+ bias when bias != null).  If probs != null, also writes the
// row softmax of logits and, per selected slot, its probability.
__global__ void __launch_bounds__(TOPK_WARPS * 32) topk_kernel(int32_t* dst, const float* logits, const float* bias, float* probs, float* weights,
                                                                int rows, int count, int k, float* spill) {
  __shared__ float sh[TOPK_WARPS][TOPK_SMEM_COLS];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int row = blockIdx.x * TOPK_WARPS + warp;
  if (row >= rows) return;
  const float* src = logits + (int64_t)row * count;
  float* work = (count <= TOPK_SMEM_COLS) ? sh[warp] : spill + (int64_t)row * count;
  if (probs) {
    // kernels/scalar/norm.go:7-24 softmax of the raw logits.
    float m = -INFINITY;
    for (int c = lane; c < count; c += 32) m = fmaxf(m, src[c]);
    m = warp_max(m);
    float sum = 0;
    for (int c = lane; c < count; c += 32) sum += expf(src[c] - m);
    sum = warp_sum(sum);
    float inv = 1.0f / sum;
    for (int c = lane; c < count; c += 32) probs[(int64_t)row * count + c] = expf(src[c] - m) * inv;
  }
  for (int c = lane; c < count; c += 32) work[c] = bias ? src[c] + bias[c] : src[c];
  __syncwarp();
  int limit = k < count ? k : count;
  for (int slot = 0; slot < limit; ++slot) {
    // The scalar statement starts from index 0 and replaces on strict '>' only:
    // the first maximum wins, and when every value is -inf index 0 is returned.
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int c = lane; c < count; c += 32) {
      float v = work[c];
      if (v > best || (v == best && c < bi)) { best = v; bi = c; }
    }
    warp_argmax_first(best, bi);
    if (bi == 0x7fffffff) bi = 0;
    if (lane == 0) {
      dst[(int64_t)row * k + slot] = bi;
      work[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (probs && weights) {
    __syncwarp();
    for (int slot = lane; slot < limit; slot += 32)
      weights[(int64_t)row * k + slot] = probs[(int64_t)row * count + dst[(int64_t)row * k + slot]];
  }
}

static float* g_spill = nullptr;
static size_t g_spill_bytes = 0;

static int topk_go(int32_t* dst, const float* logits, const float* bias, float* probs, float* w, int rows, int count, int k, cudaStream_t s) {
  if (rows <= 0 || count <= 0 || k <= 0) return GN_OK;
  float* spill = nullptr;
  if (count > TOPK_SMEM_COLS) {
    size_t need = (size_t)rows * count * sizeof(float);
    if (need > g_spill_bytes) {
      if (g_spill) cudaFree(g_spill);
      GN_CUDA(cudaMalloc(&g_spill, need));
      g_spill_bytes = need;
    }
    spill = g_spill;
  }
  topk_kernel<<<ceil_div(rows, TOPK_WARPS), TOPK_WARPS * 32, 0, s>>>(dst, logits, bias, probs, w, rows, count, k, spill);
  GN_LAUNCH_CHECK();
  return GN_OK;
}
int topk_indices_launch(int32_t* dst, const float* scores, int rows, int count, int k, cudaStream_t s) {
  return topk_go(dst, scores, nullptr, nullptr, nullptr, rows, count, k, s);
}
int moe_gate_topk_launch(const float* logits, const float* bias, float* probs, int32_t* sel, float* w, int rows, int experts, int k, cudaStream_t s) {
  return topk_go(sel, logits, bias, probs, w, rows, experts, k, s);
}

// Grouped expert GEMM: rows are expert-major; a prefix scan of the counts maps
// each 16-row tile to its expert.  One warp per output row segment; float32
// accumulation like the scalar statement (kernels/scalar/moe.go:52-73).
__global__ void __launch_bounds__(256) grouped_gemm_kernel(float* dst, const float* input, const float* weight, const int32_t* counts, int experts,
                                                            int cols, int inner, int64_t total_rows) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.y * 8 + warp;
  if (row >= total_rows) return;
  int e = 0; int64_t off = 0;
  while (e < experts && row >= off + counts[e]) { off += counts[e]; ++e; }
  if (e >= experts) return;
  const float* in = input + row * inner;
  const float* wb = weight + (int64_t)e * cols * inner;
  for (int c = blockIdx.x; c < cols; c += gridDim.x) {
    const float* wr = wb + (int64_t)c * inner;
    float acc = 0;
    for (int i = lane; i < inner; i += 32) acc = fmaf(in[i], wr[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) dst[row * cols + c] = acc;
  }
}
int grouped_matmul_t_launch(float* dst, const float* input, const float* weight, const int32_t* counts_dev, int experts, int cols, int inner,
                            int64_t total_rows, cudaStream_t s) {
  if (total_rows <= 0 || cols <= 0) return GN_OK;
  dim3 grid(std::min(cols, 64), ceil_div(total_rows, 8));
  grouped_gemm_kernel<<<grid, 256, 0, s>>>(dst, input, weight, counts_dev, experts, cols, inner, total_rows);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// destination[row, block] = sum_h weight[h] * max(0, q[row,h] . k[block,h])
__global__ void __launch_bounds__(256) indexer_scores_kernel(float* dst, const float* q, const float* key, const float* w, int rows, int blocks, int heads, int dim) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)rows * blocks) return;
  int row = (int)(idx / blocks), b = (int)(idx % blocks);
  float total = 0;
  for (int h = 0; h < heads; ++h) {
    const float* qh = q + ((int64_t)row * heads + h) * dim;
    const float* kh = key + ((int64_t)b * heads + h) * dim;
    float d = 0;
    for (int e = lane; e < dim; e += 32) d = fmaf(qh[e], kh[e], d);
    d = warp_sum(d);
    if (d > 0) total += w[h] * d;
  }
  if (lane == 0) dst[idx] = total;
}
// The same for many rows and blocks: a 64 x 64 tile of scores per CTA, 4 x 4 per thread; per head the query and key tiles pass
// through shared memory 32 dimensions at a time (rows padded to 33 words: no bank conflicts), relu and the head weight are
// applied when the head's dot products are complete.
template <bool GATE>
__global__ void __launch_bounds__(256) indexer_scores_tiled_kernel(float* __restrict__ dst, const float* __restrict__ q, const float* __restrict__ key,
                                                                   const float* __restrict__ w, int rows, int blocks, int heads, int dim) {
  __shared__ float qs[64][33], ks[64][33];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int r0 = blockIdx.y * 64, b0 = blockIdx.x * 64;
  float total[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) total[i][j] = 0.0f;
  for (int h = 0; h < heads; ++h) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int d0 = 0; d0 < dim; d0 += 32) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < 64 * 32; idx += 256) {
        const int rr = idx >> 5, dd = idx & 31;
        const bool dok = d0 + dd < dim;
        qs[rr][dd] = (dok && r0 + rr < rows) ? q[((int64_t)(r0 + rr) * heads + h) * dim + d0 + dd] : 0.0f;
        ks[rr][dd] = (dok && b0 + rr < blocks) ? key[((int64_t)(b0 + rr) * heads + h) * dim + d0 + dd] : 0.0f;
      }
      __syncthreads();
#pragma unroll 8
      for (int dd = 0; dd < 32; ++dd) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { a[i] = qs[ty + 16 * i][dd]; b[i] = ks[tx + 16 * i][dd]; }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    }
    const float wh = w[h];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) if (!GATE || acc[i][j] > 0.0f) total[i][j] += wh * acc[i][j];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + ty + 16 * i, b = b0 + tx + 16 * j;
      if (r < rows && b < blocks) dst[(int64_t)r * blocks + b] = total[i][j];
    }
}
int indexer_scores_launch(float* dst, const float* q, const float* k, const float* w, int rows, int blocks, int heads, int dim, cudaStream_t s) {
  int64_t n = (int64_t)rows * blocks;
  if (n <= 0) return GN_OK;
  if (rows >= 64 && blocks >= 64) {
    indexer_scores_tiled_kernel<true><<<dim3(ceil_div(blocks, 64), ceil_div(rows, 64)), 256, 0, s>>>(dst, q, k, w, rows, blocks, heads, dim);
    GN_LAUNCH_CHECK();
    return GN_OK;
  }
  indexer_scores_kernel<<<ceil_div(n, 8), 256, 0, s>>>(dst, q, k, w, rows, blocks, heads, dim);
  GN_LAUNCH_CHECK();
  return GN_OK;
}
// dst[row, block] = scale[0] * (q[row] . key[block]): the tiled kernel above without the gate, one head
int dot_scores_launch(float* dst, const float* q, const float* k, const float* scale, int rows, int blocks, int dim, cudaStream_t s) {
  if ((int64_t)rows * blocks <= 0) return GN_OK;
  indexer_scores_tiled_kernel<false><<<dim3(ceil_div(blocks, 64), ceil_div(rows, 64)), 256, 0, s>>>(dst, q, k, scale, rows, blocks, 1, dim);
  GN_LAUNCH_CHECK();
  return GN_OK;
}
__global__ void __launch_bounds__(256) indexer_block_max_kernel(float* dst, const float* scores, int rows, int blocks, int group, int groups) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * groups) return;
  int row = (int)(idx / groups), g = (int)(idx % groups);
  int s0 = g * group, e0 = min(s0 + group, blocks);
  float m = -INFINITY;
  for (int i = s0; i < e0; ++i) m = fmaxf(m, scores[(int64_t)row * blocks + i]);
  dst[idx] = m;
}
int indexer_block_max_launch(float* dst, const float* scores, int rows, int blocks, int group, cudaStream_t s) {
  if (group < 1) group = 1;
  int groups = (blocks + group - 1) / group;
  int64_t n = (int64_t)rows * groups;
  if (n <= 0) return GN_OK;
  indexer_block_max_kernel<<<ceil_div(n, 256), 256, 0, s>>>(dst, scores, rows, blocks, group, groups);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
