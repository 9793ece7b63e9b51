// Building blocks of the reference's compressed attention layers (the "flash" preset), inference forward:
//   channel compressor            model/compress.go:93-177 (logits = hidden W^T + positional bias, softmax over the rows
//                                 of a block per channel, weighted sum of the block's value rows)
//   attention over the compressed blocks that strictly precede the query's block
//                                 model/compress_attention.go:624-673
//   merge of two softmax branches that share one normalisation (compressed + sliding window)
//                                 model/compress_attention.go:440-484
//   block selection of the sparse indexer: the top-k allowed blocks per token, descending score, ties toward the
//   smaller index                 model/indexer.go:160-262
// All HBM-bound row kernels; the compressor's logits come from the ordinary product.
#include "kernels.cuh"

namespace gn {

namespace {

// one thread per (batch, block, channel); logits [B*T, C] already hold hidden W^T
__global__ void __launch_bounds__(256) compressor_pool_kernel(const float* __restrict__ logits, const float* __restrict__ bias, const float* __restrict__ value,
                                                              int B, int T, int C, int ratio, int blocks, float* __restrict__ compressed,
                                                              float* __restrict__ probabilities) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * blocks * C) return;
  const int c = (int)(idx % C); const int64_t bb = idx / C; const int blk = (int)(bb % blocks); const int b = (int)(bb / blocks);
  const int t0 = blk * ratio, rows = min(ratio, T - t0);
  const float* lg = logits + ((int64_t)b * T + t0) * C + c;
  float mx = -INFINITY;
  for (int r = 0; r < rows; ++r) mx = fmaxf(mx, lg[(int64_t)r * C] + bias[(int64_t)r * C + c]);
  double total = 0.0;
  for (int r = 0; r < rows; ++r) total += (double)(float)exp((double)(lg[(int64_t)r * C] + bias[(int64_t)r * C + c] - mx));
  float acc = 0.0f;
  const float inv = total > 0.0 ? (float)(1.0 / total) : 0.0f;
  const float* vp = value + ((int64_t)b * T + t0) * C + c;
  float* pp = probabilities ? probabilities + (((int64_t)b * blocks + blk) * ratio) * C + c : nullptr;
  for (int r = 0; r < ratio; ++r) {
    float p = 0.0f;
    if (r < rows && total > 0.0) {
      p = (float)exp((double)(lg[(int64_t)r * C] + bias[(int64_t)r * C + c] - mx)) * inv;
      acc = __fadd_rn(acc, __fmul_rn(p, vp[(int64_t)r * C]));
    }
    if (pp) pp[(int64_t)r * C] = p;
  }
  compressed[idx] = acc;
}

// compressForward for every kv head at once (model/compress_attention.go:562-622): the block softmax depends on the hidden state
// alone, so a thread computes the weights of its (batch, block, channel) once -- the same arithmetic as compressor_pool_kernel --
// and applies them to the keys and the values of every kv head.  probabilities [B, blocks, ratio, C] is written (it is also the
// scratch between the two steps).
__global__ void __launch_bounds__(256) compress_heads_kernel(const float* __restrict__ logits, const float* __restrict__ bias, const float* __restrict__ key,
                                                             const float* __restrict__ value, int B, int H, int T, int C, int ratio, int blocks,
                                                             float* __restrict__ key_c, float* __restrict__ value_c, float* __restrict__ probabilities) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * blocks * C) return;
  const int c = (int)(idx % C); const int64_t bb = idx / C; const int blk = (int)(bb % blocks); const int b = (int)(bb / blocks);
  const int t0 = blk * ratio, rows = min(ratio, T - t0);
  const float* lg = logits + ((int64_t)b * T + t0) * C + c;
  float mx = -INFINITY;
  for (int r = 0; r < rows; ++r) mx = fmaxf(mx, lg[(int64_t)r * C] + bias[(int64_t)r * C + c]);
  double total = 0.0;
  for (int r = 0; r < rows; ++r) total += (double)(float)exp((double)(lg[(int64_t)r * C] + bias[(int64_t)r * C + c] - mx));
  const float inv = total > 0.0 ? (float)(1.0 / total) : 0.0f;
  float* pp = probabilities + (((int64_t)b * blocks + blk) * ratio) * C + c;
  for (int r = 0; r < ratio; ++r) pp[(int64_t)r * C] = (r < rows && total > 0.0) ? (float)exp((double)(lg[(int64_t)r * C] + bias[(int64_t)r * C + c] - mx)) * inv : 0.0f;
  for (int h = 0; h < H; ++h) {
    const int64_t head = (int64_t)b * H + h;
    const float* kp = key + (head * T + t0) * C + c; const float* vp = value + (head * T + t0) * C + c;
    float ak = 0.0f, av = 0.0f;
    for (int r = 0; r < rows; ++r) {
      const float p = pp[(int64_t)r * C];
      ak = __fadd_rn(ak, __fmul_rn(p, kp[(int64_t)r * C])); av = __fadd_rn(av, __fmul_rn(p, vp[(int64_t)r * C]));
    }
    key_c[(head * blocks + blk) * C + c] = ak; value_c[(head * blocks + blk) * C + c] = av;
  }
}
// compressBackward for every kv head at once (model/compress_attention.go:1182-1209): grad_key / grad_value [B, H, T, C] of the rows,
// and the logit gradient summed over the heads and over keys and values (the hidden-state and weight gradients follow from it).
__global__ void __launch_bounds__(256) compress_heads_bwd_kernel(const float* __restrict__ key, const float* __restrict__ value,
                                                                 const float* __restrict__ probabilities, const float* __restrict__ key_c,
                                                                 const float* __restrict__ value_c, const float* __restrict__ grad_key_c,
                                                                 const float* __restrict__ grad_value_c, int B, int H, int T, int C, int ratio, int blocks,
                                                                 float* __restrict__ grad_logits, float* __restrict__ grad_key, float* __restrict__ grad_value) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * blocks * C) return;
  const int c = (int)(idx % C); const int64_t bb = idx / C; const int blk = (int)(bb % blocks); const int b = (int)(bb / blocks);
  const int t0 = blk * ratio, rows = min(ratio, T - t0);
  const float* pp = probabilities + (((int64_t)b * blocks + blk) * ratio) * C + c;
  for (int r = 0; r < rows; ++r) {
    const float p = pp[(int64_t)r * C];
    float gl = 0.0f;
    for (int h = 0; h < H; ++h) {
      const int64_t head = (int64_t)b * H + h, ci = (head * blocks + blk) * C + c, o = (head * T + t0 + r) * C + c;
      const float pk = __fmul_rn(p, grad_key_c[ci]), pv = __fmul_rn(p, grad_value_c[ci]);
      grad_key[o] = pk; grad_value[o] = pv;
      gl = __fadd_rn(gl, __fmul_rn(pk, __fsub_rn(key[o], key_c[ci])));
      gl = __fadd_rn(gl, __fmul_rn(pv, __fsub_rn(value[o], value_c[ci])));
    }
    grad_logits[((int64_t)b * T + t0 + r) * C + c] = gl;
  }
}

// backward of the block softmax: one thread per (batch, block, channel) writes dlogits and dvalue of its rows
__global__ void __launch_bounds__(256) compressor_pool_bwd_kernel(const float* __restrict__ value, const float* __restrict__ probabilities,
                                                                  const float* __restrict__ compressed, const float* __restrict__ grad_compressed, int B, int T, int C,
                                                                  int ratio, int blocks, float* __restrict__ grad_logits, float* __restrict__ grad_value) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * blocks * C) return;
  const int c = (int)(idx % C); const int64_t bb = idx / C; const int blk = (int)(bb % blocks); const int b = (int)(bb / blocks);
  const int t0 = blk * ratio, rows = min(ratio, T - t0);
  const float g = grad_compressed[idx], cv = compressed[idx];
  for (int r = 0; r < rows; ++r) {
    const float p = probabilities[(((int64_t)b * blocks + blk) * ratio + r) * C + c];
    const int64_t o = ((int64_t)b * T + t0 + r) * C + c;
    grad_logits[o] = __fmul_rn(__fmul_rn(p, g), __fsub_rn(value[o], cv));
    grad_value[o] = __fmul_rn(p, g);
  }
}
// bias gradient: one thread per (block position, channel), the rows added in (batch, position) order
__global__ void __launch_bounds__(256) compressor_bias_bwd_kernel(const float* __restrict__ grad_logits, int B, int T, int C, int ratio, float* __restrict__ grad_bias) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= ratio * C) return;
  const int c = idx % C, r = idx / C;
  float acc = grad_bias[idx];
  for (int b = 0; b < B; ++b)
    for (int t = r; t < T; t += ratio) acc = __fadd_rn(acc, grad_logits[((int64_t)b * T + t) * C + c]);
  grad_bias[idx] = acc;
}

// One warp per (batch, kv head, token) and HR query heads of the group: keys = compressed blocks 0 .. (offset + t) / ratio - 1, or
// the token's selected blocks.  The K and V rows are read once for the HR heads (the heads of a group see the same keys; with one
// row read per head the kernel sat on the L2 -> SM bandwidth).  32 keys at a time: lane j keeps the scores of key j of the chunk,
// a chunk shares one rescale per head, rows are requested four at a time so that their latencies overlap.  An index outside the
// blocks is ignored, never dereferenced.
template <int DP, int HR>
__global__ void __launch_bounds__(256) compressed_attention_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc, int B,
                                                                   int Hq, int Hkv, int T, int D, int blocks, int ratio, float* __restrict__ out,
                                                                   float* __restrict__ lse, const int32_t* __restrict__ selection,
                                                                   const int32_t* __restrict__ counts, int topk, int offset) {
  constexpr int PER = DP / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hr = Hq / Hkv, parts = hr / HR;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)B * Hkv * parts * T) return;
  const int t = (int)(idx % T); const int64_t rest = idx / T; const int part = (int)(rest % parts); const int64_t kvh = rest / parts;
  const int hk = (int)(kvh % Hkv); const int b = (int)(kvh / Hkv);
  const int64_t row0 = ((int64_t)b * Hq + hk * hr + part * HR) * T + t;     // head g of this warp: row0 + g * T
  const int32_t* sel = selection ? selection + (kvh * T + t) * topk : nullptr;
  const int nk = selection ? max(0, min(counts[kvh * T + t], topk)) : min((offset + t) / ratio, blocks);
  const int64_t kbase = kvh * blocks * D;
  float qv[HR][PER], acc[HR][PER], m[HR], l[HR];
#pragma unroll
  for (int g = 0; g < HR; ++g) {
    m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; qv[g][i] = c < D ? q[(row0 + (int64_t)g * T) * D + c] : 0.0f; acc[g][i] = 0.0f; }
  }
  for (int j0 = 0; j0 < nk; j0 += 32) {
    const int cn = min(32, nk - j0);
    int myblk = -1;
    if (lane < cn) { myblk = sel ? sel[j0 + lane] : j0 + lane; if ((unsigned)myblk >= (unsigned)blocks) myblk = -1; }
    float mys[HR];
#pragma unroll
    for (int g = 0; g < HR; ++g) mys[g] = -INFINITY;
    for (int u0 = 0; u0 < cn; u0 += 4) {
      float kv[4][PER]; int bl[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { bl[u] = __shfl_sync(0xffffffffu, myblk, (u0 + u) & 31); if (u0 + u >= cn) bl[u] = -1; }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float* kr = kc + kbase + (int64_t)max(bl[u], 0) * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; kv[u][i] = (bl[u] >= 0 && c < D) ? kr[c] : 0.0f; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (bl[u] < 0) continue;
#pragma unroll
        for (int g = 0; g < HR; ++g) {
          float sc = 0.0f;
#pragma unroll
          for (int i = 0; i < PER; ++i) sc = fmaf(qv[g][i], kv[u][i], sc);
          sc = warp_sum(sc);
          if (lane == u0 + u) mys[g] = sc;
        }
      }
    }
    float e[HR];
#pragma unroll
    for (int g = 0; g < HR; ++g) {
      float cm = mys[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
      e[g] = 0.0f;
      if (cm == -INFINITY) continue;                       // no usable key in this chunk (the same for every lane)
      const float mn = fmaxf(m[g], cm);
      const float f = __expf(m[g] - mn);
      e[g] = mys[g] == -INFINITY ? 0.0f : __expf(mys[g] - mn);
      l[g] = l[g] * f + warp_sum(e[g]);
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[g][i] *= f;
      m[g] = mn;
    }
    for (int u0 = 0; u0 < cn; u0 += 4) {
      float vv[4][PER]; int bl[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { bl[u] = __shfl_sync(0xffffffffu, myblk, (u0 + u) & 31); if (u0 + u >= cn) bl[u] = -1; }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float* vr = vc + kbase + (int64_t)max(bl[u], 0) * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; vv[u][i] = (bl[u] >= 0 && c < D) ? vr[c] : 0.0f; }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int g = 0; g < HR; ++g) {
          const float pw = __shfl_sync(0xffffffffu, e[g], (u0 + u) & 31);     // 0 for a key that is not there
#pragma unroll
          for (int i = 0; i < PER; ++i) acc[g][i] = fmaf(pw, vv[u][i], acc[g][i]);
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < HR; ++g) {
    const float inv = l[g] > 0.0f ? 1.0f / l[g] : 0.0f;
    const int64_t row = row0 + (int64_t)g * T;
#pragma unroll
    for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; if (c < D) out[row * D + c] = acc[g][i] * inv; }
    if (lse && lane == 0) lse[row] = l[g] > 0.0f ? m[g] + logf(l[g]) : -INFINITY;
  }
}

// Backward over the preceding blocks (model/compress_attention.go:735-781), deterministic, no atomics.
// dq: one warp per (batch, query head, token): p_j = exp(q.k_j - lse), dp_j = dO.v_j, ds_j = p_j (dp_j - delta), dq += sum_j ds_j k_j,
// delta = row_correction[t] when given, else sum_j p_j dp_j (its own pass).  With a selection the keys are the token's selected blocks.
template <int DP>
__global__ void __launch_bounds__(256) compressed_attention_dq_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc,
                                                                      const float* __restrict__ dout, const float* __restrict__ lse,
                                                                      const float* __restrict__ delta, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio,
                                                                      float* __restrict__ dq, const int32_t* __restrict__ selection,
                                                                      const int32_t* __restrict__ counts, int topk) {
  constexpr int PER = DP / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)B * Hq * T) return;
  const int t = (int)(idx % T); const int64_t bh = idx / T; const int h = (int)(bh % Hq); const int b = (int)(bh / Hq);
  const int64_t kvh = (int64_t)b * Hkv + h / (Hq / Hkv);
  const int32_t* sel = selection ? selection + (kvh * T + t) * topk : nullptr;
  const int nk = selection ? max(0, min(counts[kvh * T + t], topk)) : min(t / ratio, blocks);
  if (nk <= 0) return;
  const int64_t kbase = kvh * blocks * D;
  float qv[PER], gv[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; qv[i] = c < D ? q[idx * D + c] : 0.0f; gv[i] = c < D ? dout[idx * D + c] : 0.0f; acc[i] = 0.0f; }
  const float L = lse[idx], dl = delta[idx];
  for (int j = 0; j < nk; ++j) {
    const int blk = sel ? sel[j] : j;
    if ((unsigned)blk >= (unsigned)blocks) continue;
    const int64_t kr = kbase + (int64_t)blk * D;
    float s = 0.0f, dp = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; if (c < D) { s = fmaf(qv[i], kc[kr + c], s); dp = fmaf(gv[i], vc[kr + c], dp); } }
    s = warp_sum(s); dp = warp_sum(dp);
    const float ds = __expf(s - L) * (dp - dl);
#pragma unroll
    for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; if (c < D) acc[i] = fmaf(ds, kc[kr + c], acc[i]); }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; if (c < D) dq[idx * D + c] += acc[i]; }
}
// bits[(kvh * words + j / 32) * T + t] bit j % 32 = token t of (batch, kv head) kvh selected block j (zeroed before; an OR of bits
// gives the same word in any order)
__global__ void __launch_bounds__(256) select_bits_kernel(const int32_t* __restrict__ selection, const int32_t* __restrict__ counts, int64_t tokens, int T, int topk,
                                                          int blocks, uint32_t* __restrict__ bits) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tokens * topk) return;
  const int slot = (int)(idx % topk); const int64_t tr = idx / topk;      // tr = kvh * T + t
  if (slot >= min(counts[tr], topk)) return;
  const int j = selection[idx];
  if ((unsigned)j >= (unsigned)blocks) return;
  const int64_t kvh = tr / T; const int t = (int)(tr % T);
  atomicOr(bits + (kvh * ((blocks + 31) / 32) + (j >> 5)) * T + t, 1u << (j & 31));
}
// dkc / dvc: one CTA per (batch, kv head, block j) walks the tokens that attend to block j (dense: those of the later blocks;
// selected blocks: a scan of each token's selection list) and, per token, the query heads of the group.  Warp w takes the tokens
// t0 + w, t0 + w + 8, ... in ascending order (a block early in a long sequence is attended by thousands of (token, head) rows,
// and one warp's chain of dependent row reads set the kernel's time); the eight partial sums are added in warp order.
template <int DP>
__global__ void __launch_bounds__(256) compressed_attention_dkv_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc,
                                                                       const float* __restrict__ dout, const float* __restrict__ lse,
                                                                       const float* __restrict__ delta, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio,
                                                                       float* __restrict__ dkc, float* __restrict__ dvc, const int32_t* __restrict__ selection,
                                                                       const int32_t* __restrict__ counts, int topk, const uint32_t* __restrict__ bits) {
  constexpr int PER = DP / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ float part[8][2][DP];
  const int64_t idx = blockIdx.x;   // grid = B * Hkv * blocks
  const int j = (int)(idx % blocks); const int64_t kvh = idx / blocks; const int hk = (int)(kvh % Hkv); const int b = (int)(kvh / Hkv);
  const int hr = Hq / Hkv;
  float kv[PER], vv[PER], ak[PER], av[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; kv[i] = c < D ? kc[idx * D + c] : 0.0f; vv[i] = c < D ? vc[idx * D + c] : 0.0f; ak[i] = av[i] = 0.0f; }
  const int t0 = selection ? 0 : (int)min((int64_t)(j + 1) * ratio, (int64_t)T);
  // With the selection turned into bits[(kvh, j / 32), t] (select_bits_kernel) a warp learns with one coalesced read which of
  // 32 tokens attend to block j; warp w takes the token groups w, w + 8, ...  Without the bits it reads every token's list.
  const int words = (blocks + 31) / 32;
  const int step = bits ? 256 : 8;
  for (int tb = t0 + (bits ? warp * 32 : warp); tb < T; tb += step) {
    unsigned pending = 1u;                        // one token per iteration unless the bits name up to 32
    if (bits) {
      const uint32_t wd = tb + lane < T ? bits[(kvh * words + (j >> 5)) * T + tb + lane] : 0u;
      pending = __ballot_sync(0xffffffffu, (wd >> (j & 31)) & 1u);
    } else if (selection) {
      const int n = max(0, min(counts[kvh * T + tb], topk));
      const int32_t* sel = selection + (kvh * T + tb) * topk;
      bool mine = false;
      for (int i = lane; i < n; i += 32) mine |= sel[i] == j;
      if (!__any_sync(0xffffffffu, mine)) continue;
    }
    while (pending) {
    const int t = tb + __ffs(pending) - 1;
    pending &= pending - 1;
    for (int hh = 0; hh < hr; ++hh) {
      const int64_t row = ((int64_t)b * Hq + hk * hr + hh) * T + t;
      const float* qr = q + row * D; const float* gr = dout + row * D;
      float qx[PER], gx[PER];
      float s = 0.0f, dp = 0.0f;
#pragma unroll
      for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; qx[i] = c < D ? qr[c] : 0.0f; gx[i] = c < D ? gr[c] : 0.0f; s = fmaf(qx[i], kv[i], s); dp = fmaf(gx[i], vv[i], dp); }
      s = warp_sum(s); dp = warp_sum(dp);
      const float p = __expf(s - lse[row]);
      const float ds = p * (dp - delta[row]);
#pragma unroll
      for (int i = 0; i < PER; ++i) { av[i] = fmaf(p, gx[i], av[i]); ak[i] = fmaf(ds, qx[i], ak[i]); }
    }
    }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) { part[warp][0][lane + 32 * i] = ak[i]; part[warp][1][lane + 32 * i] = av[i]; }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * D; c += 256) {
    const int which = c / D, cc = c % D;
    float acc = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) acc += part[w][which][cc];
    float* dst = which == 0 ? dkc : dvc;
    dst[idx * D + cc] += acc;
  }
}
// delta[t] = sum_j p_j dp_j over the keys of the row, for the rows that have no row correction
template <int DP>
__global__ void __launch_bounds__(256) compressed_attention_delta_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc,
                                                                         const float* __restrict__ dout, const float* __restrict__ lse, int B, int Hq, int Hkv, int T,
                                                                         int D, int blocks, int ratio, float* __restrict__ delta,
                                                                         const int32_t* __restrict__ selection, const int32_t* __restrict__ counts, int topk) {
  constexpr int PER = DP / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)B * Hq * T) return;
  const int t = (int)(idx % T); const int64_t bh = idx / T; const int h = (int)(bh % Hq); const int b = (int)(bh / Hq);
  const int64_t kvh = (int64_t)b * Hkv + h / (Hq / Hkv);
  const int32_t* sel = selection ? selection + (kvh * T + t) * topk : nullptr;
  const int nk = selection ? max(0, min(counts[kvh * T + t], topk)) : min(t / ratio, blocks);
  const int64_t kbase = kvh * blocks * D;
  float qv[PER], gv[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; qv[i] = c < D ? q[idx * D + c] : 0.0f; gv[i] = c < D ? dout[idx * D + c] : 0.0f; }
  const float L = nk > 0 ? lse[idx] : 0.0f;
  float d = 0.0f;
  for (int j = 0; j < nk; ++j) {
    const int blk = sel ? sel[j] : j;
    if ((unsigned)blk >= (unsigned)blocks) continue;
    const int64_t kr = kbase + (int64_t)blk * D;
    float s = 0.0f, dp = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) { const int c = lane + 32 * i; if (c < D) { s = fmaf(qv[i], kc[kr + c], s); dp = fmaf(gv[i], vc[kr + c], dp); } }
    s = warp_sum(s); dp = warp_sum(dp);
    d = fmaf(__expf(s - L), dp, d);
  }
  if (lane == 0) delta[idx] = d;
}

// one warp per row
__global__ void __launch_bounds__(256) attention_merge_kernel(const float* __restrict__ oa, const float* __restrict__ la, const float* __restrict__ ob,
                                                              const float* __restrict__ lb, int64_t rows, int D, float* __restrict__ out, float* __restrict__ lse) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + warp;
  if (r >= rows) return;
  const float a = la[r], b = lb[r];
  const float mx = fmaxf(a, b);
  if (mx == -INFINITY) {
    for (int c = lane; c < D; c += 32) out[r * D + c] = 0.0f;
    if (lse && lane == 0) lse[r] = mx;
    return;
  }
  const float wa = (float)exp((double)(a - mx)), wb = (float)exp((double)(b - mx));
  const float total = wa + wb;
  const float inv = (float)(1.0 / (double)total);
  for (int c = lane; c < D; c += 32) out[r * D + c] = (wa * oa[r * D + c] + wb * ob[r * D + c]) * inv;
  if (lse && lane == 0) lse[r] = mx + (float)log((double)total);
}

// one warp per token: the rank of an allowed block is the number of blocks that beat it (larger score, or equal score and
// smaller index); blocks of rank < count are the selection, in rank order.  Exact, no sort.
__global__ void __launch_bounds__(256) select_blocks_kernel(const float* __restrict__ scores, int tokens, int blocks, int offset, int ratio, int topk,
                                                            int32_t* __restrict__ selection, int32_t* __restrict__ counts) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= tokens) return;
  const int allowed = min((offset + t) / ratio, blocks);
  const int count = allowed > 0 ? min(topk, allowed) : 0;
  int32_t* sel = selection + (int64_t)t * topk;
  for (int i = lane; i < topk; i += 32) sel[i] = -1;
  if (lane == 0) counts[t] = count;
  __syncwarp();
  const float* v = scores + (int64_t)t * blocks;
  for (int i = lane; i < allowed; i += 32) {
    const float vi = v[i];
    int rank = 0;
    for (int j = 0; j < allowed; ++j) { const float vj = v[j]; rank += (vj > vi || (vj == vi && j < i)) ? 1 : 0; }
    if (rank < count) sel[rank] = i;
  }
}

// Score part of SparseIndexer.Backward (model/indexer.go:107-151), no atomics.  gate = dot(q[row, h], k[block, h]) > 0.
// grad_query: one warp per (row, head) over the blocks; it also leaves sum_b g * dot in wpart [rows, heads].
__global__ void __launch_bounds__(256) indexer_bwd_query_kernel(const float* __restrict__ gs, const float* __restrict__ q, const float* __restrict__ key,
                                                                const float* __restrict__ w, int rows, int blocks, int heads, int dim,
                                                                float* __restrict__ gq, float* __restrict__ wpart) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)rows * heads) return;
  const int h = (int)(idx % heads); const int64_t row = idx / heads;
  float qv[4], acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < 4; ++i) { const int c = lane + 32 * i; qv[i] = c < dim ? q[idx * dim + c] : 0.0f; }
  const float wh = w[h];
  float wsum = 0.0f;
  for (int b = 0; b < blocks; ++b) {
    const float* kr = key + ((int64_t)b * heads + h) * dim;
    float kv[4], d = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const int c = lane + 32 * i; kv[i] = c < dim ? kr[c] : 0.0f; d = fmaf(qv[i], kv[i], d); }
    d = warp_sum(d);
    if (d <= 0.0f) continue;
    const float g = gs[row * blocks + b];
    wsum = fmaf(g, d, wsum);
    const float wg = g * wh;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(wg, kv[i], acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) { const int c = lane + 32 * i; if (c < dim) gq[idx * dim + c] = acc[i]; }
  if (lane == 0) wpart[idx] = wsum;
}
// grad_key: one warp per (block, head) over the rows
__global__ void __launch_bounds__(256) indexer_bwd_key_kernel(const float* __restrict__ gs, const float* __restrict__ q, const float* __restrict__ key,
                                                              const float* __restrict__ w, int rows, int blocks, int heads, int dim, float* __restrict__ gk) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)blocks * heads) return;
  const int h = (int)(idx % heads); const int64_t b = idx / heads;
  float kv[4], acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < 4; ++i) { const int c = lane + 32 * i; kv[i] = c < dim ? key[idx * dim + c] : 0.0f; }
  const float wh = w[h];
  for (int r = 0; r < rows; ++r) {
    const float* qr = q + ((int64_t)r * heads + h) * dim;
    float qv[4], d = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const int c = lane + 32 * i; qv[i] = c < dim ? qr[c] : 0.0f; d = fmaf(qv[i], kv[i], d); }
    d = warp_sum(d);
    if (d <= 0.0f) continue;
    const float wg = gs[(int64_t)r * blocks + b] * wh;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(wg, qv[i], acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) { const int c = lane + 32 * i; if (c < dim) gk[idx * dim + c] = acc[i]; }
}
// The same two gradients for many rows and blocks, in 64 x 64 tiles of scores (4 x 4 per thread, as indexer_scores_tiled_kernel):
// the tile of q . k is recomputed, G = grad_scores * w_h where the dot product is positive goes through shared memory, and a second
// small product adds G K (query side: a CTA owns 64 rows and walks the block tiles) or G^T Q (key side: a CTA owns 64 blocks and
// walks the row tiles) in a fixed order.  Shared memory: the two operand tiles at full dim (rows padded by one word) and G.
template <bool KEY_SIDE>
__global__ void __launch_bounds__(256) indexer_bwd_tiled_kernel(const float* __restrict__ gs, const float* __restrict__ q, const float* __restrict__ key,
                                                                const float* __restrict__ w, int rows, int blocks, int heads, int dim,
                                                                float* __restrict__ out, float* __restrict__ wpart, int tiles_per_split) {
  // blockIdx.z: a share of the tiles walked (key side with few block tiles: the shares' partial results, out + z * plane, are added
  // by a second pass)
  extern __shared__ float smem[];
  const int ld = dim + 1;
  float* Qs = smem; float* Ks = Qs + 64 * ld; float* Gs = Ks + 64 * ld;      // Gs [64 rows][65]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int h = blockIdx.y, own0 = blockIdx.x * 64;                          // the 64 rows (query side) or blocks (key side) of this CTA
  const float wh = w[h];
  const int ncol = (dim + 15) / 16;                                          // output columns per thread: tx, tx + 16, ... (at most 8)
  float acc_o[4][8], wsum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc_o[i][j] = 0.0f;
  auto load_tile = [&](float* dst, const float* src, int first, int limit) {
    for (int idx = threadIdx.x; idx < 64 * dim; idx += 256) {
      const int rr = idx / dim, dd = idx % dim;
      dst[rr * ld + dd] = first + rr < limit ? src[((int64_t)(first + rr) * heads + h) * dim + dd] : 0.0f;
    }
  };
  if (KEY_SIDE) load_tile(Ks, key, own0, blocks); else load_tile(Qs, q, own0, rows);
  const int other_n = KEY_SIDE ? rows : blocks;
  const int o_begin = blockIdx.z * tiles_per_split * 64, o_end = min(other_n, o_begin + tiles_per_split * 64);
  out += (int64_t)blockIdx.z * (KEY_SIDE ? blocks : rows) * heads * dim;
  for (int o0 = o_begin; o0 < o_end; o0 += 64) {
    __syncthreads();                                                         // the previous tile's second product is done
    if (KEY_SIDE) load_tile(Qs, q, o0, rows); else load_tile(Ks, key, o0, blocks);
    __syncthreads();
    const int r0 = KEY_SIDE ? o0 : own0, b0 = KEY_SIDE ? own0 : o0;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int d = 0; d < dim; ++d) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = Qs[(ty + 16 * i) * ld + d]; b[i] = Ks[(tx + 16 * i) * ld + d]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = r0 + ty + 16 * i, b = b0 + tx + 16 * j;
        float g = 0.0f;
        if (r < rows && b < blocks && acc[i][j] > 0.0f) {
          const float gsv = gs[(int64_t)r * blocks + b];
          if (!KEY_SIDE) wsum[i] = fmaf(gsv, acc[i][j], wsum[i]);
          g = gsv * wh;
        }
        Gs[(ty + 16 * i) * 65 + tx + 16 * j] = g;                            // [row of the tile][block of the tile]
      }
    __syncthreads();
    if (!KEY_SIDE) {
      // grad_query[row, c] += sum_b G[row][b] K[b][c]
      for (int bb = 0; bb < 64; ++bb) {
        float gv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) gv[i] = Gs[(ty + 16 * i) * 65 + bb];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j >= ncol) break;
          const int c = tx + 16 * j;
          const float kvv = c < dim ? Ks[bb * ld + c] : 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) acc_o[i][j] = fmaf(gv[i], kvv, acc_o[i][j]);
        }
      }
    } else {
      // grad_key[block, c] += sum_r G[r][block] Q[r][c]
      for (int rr = 0; rr < 64; ++rr) {
        float gv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) gv[i] = Gs[rr * 65 + ty + 16 * i];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j >= ncol) break;
          const int c = tx + 16 * j;
          const float qvv = c < dim ? Qs[rr * ld + c] : 0.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) acc_o[i][j] = fmaf(gv[i], qvv, acc_o[i][j]);
        }
      }
    }
  }
  const int own_n = KEY_SIDE ? blocks : rows;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int o = own0 + ty + 16 * i;
    if (o < own_n) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const int c = tx + 16 * j; if (j < ncol && c < dim) out[((int64_t)o * heads + h) * dim + c] = acc_o[i][j]; }
    }
    if (!KEY_SIDE) {
      float v = wsum[i];
#pragma unroll
      for (int m = 8; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);   // over the 16 threads that share the row
      if (tx == 0 && o < own_n) wpart[(int64_t)o * heads + h] = v;
    }
  }
}

// out[i] = sum of the planes part[z][i] in order
__global__ void __launch_bounds__(256) plane_sum_kernel(const float* __restrict__ part, int planes, int64_t n, float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.0f;
  for (int z = 0; z < planes; ++z) acc += part[(int64_t)z * n + i];
  out[i] = acc;
}
// grad_weight[h] += sum over rows of wpart[row, h]: one CTA per head, fixed order
__global__ void __launch_bounds__(256) indexer_bwd_weight_kernel(const float* __restrict__ wpart, int rows, int heads, float* __restrict__ gw) {
  __shared__ double part[256];
  const int h = blockIdx.x;
  double a = 0.0;
  for (int r = threadIdx.x; r < rows; r += 256) a += (double)wpart[(int64_t)r * heads + h];
  part[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) { if ((int)threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o]; __syncthreads(); }
  if (threadIdx.x == 0) gw[h] += (float)part[0];
}

// distillationTarget (model/compress_attention.go:155-196): one warp per (batch, kv head, token).  The averaged logits are left in
// the target row, then turned into the softmax over the allowed blocks; the rest of the row is zero.
__global__ void __launch_bounds__(256) distillation_target_kernel(const float* __restrict__ q, const float* __restrict__ kc, int B, int Hq, int Hkv, int T, int D,
                                                                  int blocks, int ratio, float* __restrict__ target) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= (int64_t)B * Hkv * T) return;
  const int t = (int)(idx % T); const int64_t kvh = idx / T; const int hk = (int)(kvh % Hkv); const int b = (int)(kvh / Hkv);
  const int hr = Hq / Hkv, allowed = min(t / ratio, blocks);
  float* row = target + idx * blocks;
  for (int j = allowed + lane; j < blocks; j += 32) row[j] = 0.0f;
  if (allowed == 0) return;
  float mx = -INFINITY;
  for (int j = 0; j < allowed; ++j) {
    const float* kr = kc + (kvh * blocks + j) * D;
    float sum = 0.0f;
    for (int hh = 0; hh < hr; ++hh) {
      const float* qr = q + (((int64_t)b * Hq + hk * hr + hh) * T + t) * D;
      float d = 0.0f;
      for (int c = lane; c < D; c += 32) d = fmaf(qr[c], kr[c], d);
      sum += warp_sum(d);
    }
    const float logit = sum / (float)hr;
    mx = fmaxf(mx, logit);
    if (lane == 0) row[j] = logit;
  }
  __syncwarp();
  double total = 0.0;
  for (int j = lane; j < allowed; j += 32) { const double v = exp((double)(row[j] - mx)); row[j] = (float)v; total += v; }
  total = warp_sum_d(total);
  const float ft = (float)total;
  for (int j = lane; j < allowed; j += 32) row[j] /= ft;
}
// The long-sequence form of the target: the logits are linear in the query, so the queries of a group are summed first
// (head_sum_kernel, heads in order), one tiled product per (batch, kv head) gives sum_h q_h . k / heads for every (token, block),
// and target_softmax_kernel turns each row into the softmax over its allowed blocks (float64 sum, as the reference) and zeroes the rest.
__global__ void __launch_bounds__(256) head_sum_kernel(const float* __restrict__ q, int B, int Hq, int Hkv, int T, int D, float* __restrict__ qsum) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)B * Hkv * T * D) return;
  const int c = (int)(idx % D); const int64_t r = idx / D; const int t = (int)(r % T); const int64_t kvh = r / T;
  const int hk = (int)(kvh % Hkv); const int b = (int)(kvh / Hkv); const int hr = Hq / Hkv;
  float acc = 0.0f;
  for (int h = 0; h < hr; ++h) acc += q[((((int64_t)b * Hq + hk * hr + h) * T + t) * D) + c];
  qsum[idx] = acc;
}
__global__ void __launch_bounds__(256) target_softmax_kernel(float* __restrict__ target, int64_t rows, int T, int blocks, int ratio) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + warp;
  if (r >= rows) return;
  const int allowed = min((int)(r % T) / ratio, blocks);
  float* row = target + r * blocks;
  float mx = -INFINITY;
  for (int j = lane; j < allowed; j += 32) mx = fmaxf(mx, row[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  double total = 0.0;
  for (int j = lane; j < allowed; j += 32) { const double v = exp((double)(row[j] - mx)); row[j] = (float)v; total += v; }
  total = warp_sum_d(total);
  const float ft = (float)total;
  for (int j = lane; j < blocks; j += 32) row[j] = j < allowed ? row[j] / ft : 0.0f;
}
__global__ void set_scalar_kernel(float* dst, float v) { *dst = v; }

// (softmax over the allowed blocks - target) * weight, optionally restricted to the row's candidate list
// (model/compress_attention.go:120-151, 203-231, 266-303): one warp per row; the gradient row doubles as the membership marker.
__global__ void __launch_bounds__(256) distillation_grad_kernel(const float* __restrict__ scores, const float* __restrict__ target,
                                                                const int32_t* __restrict__ candidates, const int32_t* __restrict__ candidate_counts, int cap,
                                                                int64_t rows, int blocks, int seq, int ratio, float weight, float* __restrict__ grad) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + warp;
  if (r >= rows) return;
  const float* sc = scores + r * blocks; const float* tg = target + r * blocks;
  float* g = grad + r * blocks;
  const int allowed = min((int)(r % seq) / ratio, blocks);
  const bool pooled = candidates != nullptr;
  double ttotal = 0.0;
  if (pooled) {
    for (int e = lane; e < blocks; e += 32) g[e] = 0.0f;
    __syncwarp();
    const int n = max(0, min(candidate_counts[r], cap));
    for (int i = lane; i < n; i += 32) { const int e = candidates[r * cap + i]; if (e >= 0 && e < blocks) g[e] = 1.0f; }
    __syncwarp();
    for (int e = lane; e < blocks; e += 32) if (g[e] != 0.0f) ttotal += (double)tg[e];
    ttotal = warp_sum_d(ttotal);
  }
  float mx = -INFINITY;
  for (int e = lane; e < allowed; e += 32) if (!pooled || g[e] != 0.0f) mx = fmaxf(mx, sc[e]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  double total = 0.0;
  if (mx != -INFINITY)
    for (int e = lane; e < allowed; e += 32) if (!pooled || g[e] != 0.0f) total += exp((double)(sc[e] - mx));
  total = warp_sum_d(total);
  const float ft = (float)total;
  for (int e = lane; e < blocks; e += 32) {
    const bool in = !pooled || g[e] != 0.0f;
    float t = in ? tg[e] : 0.0f;
    if (pooled && in && ttotal > 0.0) t = (float)((double)t / ttotal);
    float p = 0.0f;
    if (in && e < allowed && mx != -INFINITY) p = (float)exp((double)(sc[e] - mx)) / ft;
    g[e] = (p - t) * weight;
  }
}

// One warp per token, the two-level selection (model/indexer.go:442-513).  gmax [tokens, ceil(blocks / pool)] and chosen
// [tokens, per_token] are scratch.  Ranks are counted exactly as in select_blocks_kernel: super-blocks by their maximum over
// the allowed entries, then the candidate entries (super-blocks in rank order, entries ascending inside) by score with ties
// toward the earlier candidate.
__global__ void __launch_bounds__(256) select_hierarchical_kernel(const float* __restrict__ scores, int tokens, int blocks, int offset, int ratio, int topk,
                                                                  int pool, int per_token, float* __restrict__ gmax, int32_t* __restrict__ chosen,
                                                                  int32_t* __restrict__ selection, int32_t* __restrict__ counts,
                                                                  int32_t* __restrict__ candidates, int32_t* __restrict__ candidate_counts) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= tokens) return;
  const int cap = per_token * pool, all_groups = (blocks + pool - 1) / pool;
  const int allowed = topk > 0 ? min((offset + t) / ratio, blocks) : 0;
  int32_t* sel = selection + (int64_t)t * topk;
  int32_t* cand = candidates + (int64_t)t * cap;
  for (int i = lane; i < topk; i += 32) sel[i] = -1;
  for (int i = lane; i < cap; i += 32) cand[i] = -1;
  if (allowed <= 0) { if (lane == 0) { counts[t] = 0; candidate_counts[t] = 0; } return; }
  const float* v = scores + (int64_t)t * blocks;
  float* gm = gmax + (int64_t)t * all_groups;
  int32_t* ch = chosen + (int64_t)t * per_token;
  const int groups = (allowed + pool - 1) / pool, nch = min(per_token, groups);
  for (int g = lane; g < groups; g += 32) {
    float m = -INFINITY;
    for (int e = g * pool; e < min((g + 1) * pool, allowed); ++e) m = fmaxf(m, v[e]);
    gm[g] = m;
  }
  __syncwarp();
  for (int g = lane; g < groups; g += 32) {
    const float vi = gm[g];
    int rank = 0;
    for (int j = 0; j < groups; ++j) { const float vj = gm[j]; rank += (vj > vi || (vj == vi && j < g)) ? 1 : 0; }
    if (rank < nch) ch[rank] = g;
  }
  __syncwarp();
  // only the last allowed super-block can be short: find its rank among the chosen, if it is one of them
  const int tail = allowed - (groups - 1) * pool;          // entries of the last allowed super-block, 1..pool
  int short_rank = nch;
  if (tail < pool) { for (int r = 0; r < nch; ++r) if (ch[r] == groups - 1) short_rank = r; }
  const int ncand = nch * pool - (short_rank < nch ? pool - tail : 0);
  for (int c = lane; c < ncand; c += 32) {
    int r, e;
    if (c < short_rank * pool) { r = c / pool; e = c % pool; }
    else if (short_rank < nch && c < short_rank * pool + tail) { r = short_rank; e = c - short_rank * pool; }
    else { const int c2 = c - short_rank * pool - tail; r = short_rank + 1 + c2 / pool; e = c2 % pool; }
    cand[c] = ch[r] * pool + e;
  }
  __syncwarp();
  const int count = min(topk, ncand);
  if (lane == 0) { counts[t] = count; candidate_counts[t] = ncand; }
  for (int c = lane; c < ncand; c += 32) {
    const float vi = v[cand[c]];
    int rank = 0;
    for (int j = 0; j < ncand; ++j) { const float vj = v[cand[j]]; rank += (vj > vi || (vj == vi && j < c)) ? 1 : 0; }
    if (rank < count) sel[rank] = cand[c];
  }
}
// One warp per token: the top-k of a given candidate list (model/indexer.go:547-613); candidates outside [0, allowed) are dropped
__global__ void __launch_bounds__(256) select_within_pool_kernel(const float* __restrict__ scores, int tokens, int blocks, int offset, int ratio, int topk,
                                                                 const int32_t* __restrict__ candidates, const int32_t* __restrict__ candidate_counts, int cap,
                                                                 int32_t* __restrict__ selection, int32_t* __restrict__ counts) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= tokens) return;
  const int allowed = min((offset + t) / ratio, blocks);
  int32_t* sel = selection + (int64_t)t * topk;
  const int32_t* cand = candidates + (int64_t)t * cap;
  for (int i = lane; i < topk; i += 32) sel[i] = -1;
  const int n = topk > 0 ? max(0, min(candidate_counts[t], cap)) : 0;
  int kept = 0;
  for (int i = lane; i < n; i += 32) kept += (cand[i] >= 0 && cand[i] < allowed) ? 1 : 0;
  kept = (int)warp_sum((float)kept);                       // at most cap entries: exact in float below 2^24
  const int count = min(topk, kept);
  if (lane == 0) counts[t] = count;
  __syncwarp();
  const float* v = scores + (int64_t)t * blocks;
  for (int c = lane; c < n; c += 32) {
    const int e = cand[c];
    if (e < 0 || e >= allowed) continue;
    const float vi = v[e];
    int rank = 0;
    for (int j = 0; j < n; ++j) {
      const int ej = cand[j];
      if (ej < 0 || ej >= allowed) continue;
      const float vj = v[ej];
      rank += (vj > vi || (vj == vi && j < c)) ? 1 : 0;
    }
    if (rank < count) sel[rank] = e;
  }
}

}  // namespace

int compressor_pool_launch(const float* logits, const float* bias, const float* value, int B, int T, int C, int ratio, float* compressed, float* probabilities,
                           cudaStream_t s) {
  const int blocks = (T + ratio - 1) / ratio;
  const int64_t n = (int64_t)B * blocks * C;
  if (n <= 0) return GN_OK;
  compressor_pool_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, s>>>(logits, bias, value, B, T, C, ratio, blocks, compressed, probabilities);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int compressor_pool_backward_launch(const float* value, const float* probabilities, const float* compressed, const float* grad_compressed, int B, int T, int C,
                                    int ratio, float* grad_logits, float* grad_value, float* grad_bias, cudaStream_t s) {
  const int blocks = (T + ratio - 1) / ratio;
  const int64_t n = (int64_t)B * blocks * C;
  if (n <= 0) return GN_OK;
  compressor_pool_bwd_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, s>>>(value, probabilities, compressed, grad_compressed, B, T, C, ratio, blocks, grad_logits, grad_value);
  GN_LAUNCH_CHECK();
  compressor_bias_bwd_kernel<<<ceil_div((int64_t)ratio * C, 256), 256, 0, s>>>(grad_logits, B, T, C, ratio, grad_bias);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int compress_heads_launch(const float* logits, const float* bias, const float* key, const float* value, int B, int H, int T, int C, int ratio, float* key_c,
                          float* value_c, float* probabilities, cudaStream_t s) {
  const int blocks = (T + ratio - 1) / ratio;
  const int64_t n = (int64_t)B * blocks * C;
  if (n <= 0 || H <= 0) return GN_OK;
  compress_heads_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, s>>>(logits, bias, key, value, B, H, T, C, ratio, blocks, key_c, value_c, probabilities);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int compress_heads_backward_launch(const float* key, const float* value, const float* probabilities, const float* key_c, const float* value_c,
                                   const float* grad_key_c, const float* grad_value_c, int B, int H, int T, int C, int ratio, float* grad_logits, float* grad_key,
                                   float* grad_value, float* grad_bias, cudaStream_t s) {
  const int blocks = (T + ratio - 1) / ratio;
  const int64_t n = (int64_t)B * blocks * C;
  if (n <= 0 || H <= 0) return GN_OK;
  compress_heads_bwd_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, s>>>(key, value, probabilities, key_c, value_c, grad_key_c, grad_value_c, B, H, T, C, ratio, blocks,
                                                                       grad_logits, grad_key, grad_value);
  GN_LAUNCH_CHECK();
  compressor_bias_bwd_kernel<<<ceil_div((int64_t)ratio * C, 256), 256, 0, s>>>(grad_logits, B, T, C, ratio, grad_bias);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int compressed_attention_launch(const float* q, const float* kc, const float* vc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* out, float* lse,
                                const int32_t* selection, const int32_t* counts, int topk, int offset, cudaStream_t s) {
  GN_REQUIRE(D > 0 && D <= 128, "compressed attention: head_dim %d outside (0,128]", D);
  GN_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && ratio >= 1 && offset >= 0, "compressed attention: %d query heads, %d kv heads, ratio %d, offset %d", Hq, Hkv, ratio, offset);
  const int64_t n = (int64_t)B * Hq * T;
  if (n <= 0) return GN_OK;
#ifdef GN_HAVE_TCGEN05
  // head_dim 128, every block before the query's own: the tensor-core attention forward with keys counted in blocks.
  // Worth its fixed cost (operand split, 128-row query tiles) from a few thousand scores per head on.
  if (!selection && D == 128 && blocks >= 1 && (int64_t)T * blocks >= 4096) {
    AttnShape sh;
    sh.B = B; sh.Hq = Hq; sh.Hkv = Hkv; sh.D = D; sh.Tq = T; sh.Tk = blocks;
    sh.q_bstride = (int64_t)Hq * T * D; sh.q_tstride = D; sh.q_hstride = (int64_t)T * D;
    sh.kv_bstride = (int64_t)Hkv * blocks * D; sh.kv_tstride = D; sh.kv_hstride = (int64_t)blocks * D;
    sh.o_bstride = sh.q_bstride; sh.o_tstride = D; sh.o_hstride = sh.q_hstride;
    sh.window = -1; sh.offset0 = offset; sh.key_ratio = ratio; sh.tensor = 1;
    if (ratio > 1 && attention_tc_ok(sh, q, kc, vc, out)) return attention_tc_forward(sh, q, kc, vc, out, lse, s);
  }
#endif
  // the largest supported head count per warp that divides the group
  const int hr = Hq / Hkv;
  const int HR = hr % 8 == 0 ? 8 : hr % 4 == 0 ? 4 : hr % 3 == 0 ? 3 : hr % 2 == 0 ? 2 : 1;
  const unsigned grid = (unsigned)ceil_div(n / HR, 8);
#define GN_CA_FWD(DPV, HRV) compressed_attention_kernel<DPV, HRV><<<grid, 256, 0, s>>>(q, kc, vc, B, Hq, Hkv, T, D, blocks, ratio, out, lse, selection, counts, topk, offset)
#define GN_CA_FWD_D(HRV) do { if (D <= 32) GN_CA_FWD(32, HRV); else if (D <= 64) GN_CA_FWD(64, HRV); else GN_CA_FWD(128, HRV); } while (0)
  switch (HR) {
    case 8: GN_CA_FWD_D(8); break;
    case 4: GN_CA_FWD_D(4); break;
    case 3: GN_CA_FWD_D(3); break;
    case 2: GN_CA_FWD_D(2); break;
    default: GN_CA_FWD_D(1); break;
  }
#undef GN_CA_FWD_D
#undef GN_CA_FWD
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int compressed_attention_backward_launch(const float* q, const float* kc, const float* vc, const float* dout, const float* lse, const float* rowcorr,
                                         float* delta_scratch, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* dq, float* dkc, float* dvc,
                                         const int32_t* selection, const int32_t* counts, int topk, cudaStream_t s, uint32_t* select_bits) {
  GN_REQUIRE(D > 0 && D <= 128, "compressed attention: head_dim %d outside (0,128]", D);
  GN_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && ratio >= 1, "compressed attention: %d query heads, %d kv heads, ratio %d", Hq, Hkv, ratio);
  GN_REQUIRE(!selection || (counts && topk > 0), "compressed attention: a selection needs its counts and topk > 0");
  const uint32_t* bits = nullptr;
  if (selection && select_bits && (int64_t)B * Hq * T > 0 && blocks > 0) {
    const int64_t tokens = (int64_t)B * Hkv * T;
    GN_CUDA(cudaMemsetAsync(select_bits, 0, sizeof(uint32_t) * (size_t)tokens * ((blocks + 31) / 32), s));
    select_bits_kernel<<<(unsigned)ceil_div(tokens * topk, 256), 256, 0, s>>>(selection, counts, tokens, T, topk, blocks, select_bits);
    GN_LAUNCH_CHECK();
    bits = select_bits;
  }
  const int64_t nq = (int64_t)B * Hq * T, nkv = (int64_t)B * Hkv * blocks;
  if (nq <= 0 || nkv <= 0) return GN_OK;
  const unsigned gq = (unsigned)ceil_div(nq, 8);
  const float* delta = rowcorr;
  // head_dim 128, every block before the query's own: the mma.sync attention backward with keys counted in blocks (its dk / dv
  // kernel owns 128 blocks per CTA and walks the group's heads and the query tiles that see them; no atomics there either)
  if (!selection && D == 128 && ratio > 1 && (int64_t)T * blocks >= 4096) {
    AttnShape sh;
    sh.B = B; sh.Hq = Hq; sh.Hkv = Hkv; sh.D = D; sh.Tq = T; sh.Tk = blocks;
    sh.q_bstride = (int64_t)Hq * T * D; sh.q_tstride = D; sh.q_hstride = (int64_t)T * D;
    sh.kv_bstride = (int64_t)Hkv * blocks * D; sh.kv_tstride = D; sh.kv_hstride = (int64_t)blocks * D;
    sh.o_bstride = sh.q_bstride; sh.o_tstride = D; sh.o_hstride = sh.q_hstride;
    sh.window = -1; sh.offset0 = 0; sh.key_ratio = ratio; sh.tensor = 1;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (attention_mma_ok(sh, q, kc, vc, dout, dq) && al(dkc) && al(dvc)) {
      if (!delta) {
        compressed_attention_delta_kernel<128><<<gq, 256, 0, s>>>(q, kc, vc, dout, lse, B, Hq, Hkv, T, D, blocks, ratio, delta_scratch, nullptr, nullptr, 0);
        GN_LAUNCH_CHECK();
        delta = delta_scratch;
      }
      return attention_mma_backward(sh, q, kc, vc, dout, lse, delta, dq, dkc, dvc, 1, s);
    }
  }
#define GN_CA_BWD(DPV) do { \
    if (!delta) { compressed_attention_delta_kernel<DPV><<<gq, 256, 0, s>>>(q, kc, vc, dout, lse, B, Hq, Hkv, T, D, blocks, ratio, delta_scratch, selection, counts, topk); \
                  delta = delta_scratch; } \
    compressed_attention_dq_kernel<DPV><<<gq, 256, 0, s>>>(q, kc, vc, dout, lse, delta, B, Hq, Hkv, T, D, blocks, ratio, dq, selection, counts, topk); \
    compressed_attention_dkv_kernel<DPV><<<(unsigned)nkv, 256, 0, s>>>(q, kc, vc, dout, lse, delta, B, Hq, Hkv, T, D, blocks, ratio, dkc, dvc, selection, counts, topk, bits); } while (0)
  if (D <= 32) GN_CA_BWD(32); else if (D <= 64) GN_CA_BWD(64); else GN_CA_BWD(128);
#undef GN_CA_BWD
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int attention_merge_launch(const float* oa, const float* la, const float* ob, const float* lb, int64_t rows, int D, float* out, float* lse, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  attention_merge_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, s>>>(oa, la, ob, lb, rows, D, out, lse);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int select_blocks_launch(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int32_t* selection, int32_t* counts, cudaStream_t s) {
  if (tokens <= 0) return GN_OK;
  select_blocks_kernel<<<(unsigned)ceil_div(tokens, 8), 256, 0, s>>>(scores, tokens, blocks, offset, ratio, topk, selection, counts);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int indexer_scores_backward_launch(const float* gs, const float* q, const float* key, const float* w, int rows, int blocks, int heads, int dim, float* gq, float* gk,
                                   float* gw, float* wpart, cudaStream_t s, float* kpart, int kpart_planes) {
  if (rows <= 0 || blocks <= 0 || heads <= 0) return GN_OK;
  GN_REQUIRE(dim >= 1 && dim <= 128, "indexer backward: dim %d outside [1,128]", dim);
  if (rows >= 64 && blocks >= 64) {
    const size_t smem = sizeof(float) * (size_t)(2 * 64 * (dim + 1) + 64 * 65);
    static PerDeviceOnce configured;
    if (configured.first()) {
      GN_CUDA(cudaFuncSetAttribute(indexer_bwd_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(float) * (2 * 64 * 129 + 64 * 65))));
      GN_CUDA(cudaFuncSetAttribute(indexer_bwd_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(float) * (2 * 64 * 129 + 64 * 65))));
    }
    const int row_tiles = ceil_div(rows, 64), block_tiles = ceil_div(blocks, 64);
    indexer_bwd_tiled_kernel<false><<<dim3(row_tiles, heads), 256, smem, s>>>(gs, q, key, w, rows, blocks, heads, dim, gq, wpart, block_tiles);
    // key side: few block tiles leave SMs idle, so the row tiles are shared out when the caller gave room for the partial planes
    int splits = 1;
    if (kpart && block_tiles * heads < num_sms()) splits = std::max(1, std::min(std::min(row_tiles, kpart_planes), ceil_div(2 * num_sms(), block_tiles * heads)));
    const int per = ceil_div(row_tiles, splits);
    splits = ceil_div(row_tiles, per);
    if (splits > 1) {
      indexer_bwd_tiled_kernel<true><<<dim3(block_tiles, heads, splits), 256, smem, s>>>(gs, q, key, w, rows, blocks, heads, dim, kpart, nullptr, per);
      const int64_t n = (int64_t)blocks * heads * dim;
      plane_sum_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, s>>>(kpart, splits, n, gk);
    } else {
      indexer_bwd_tiled_kernel<true><<<dim3(block_tiles, heads), 256, smem, s>>>(gs, q, key, w, rows, blocks, heads, dim, gk, nullptr, row_tiles);
    }
    indexer_bwd_weight_kernel<<<heads, 256, 0, s>>>(wpart, rows, heads, gw);
    GN_LAUNCH_CHECK();
    return GN_OK;
  }
  indexer_bwd_query_kernel<<<(unsigned)ceil_div((int64_t)rows * heads, 8), 256, 0, s>>>(gs, q, key, w, rows, blocks, heads, dim, gq, wpart);
  indexer_bwd_key_kernel<<<(unsigned)ceil_div((int64_t)blocks * heads, 8), 256, 0, s>>>(gs, q, key, w, rows, blocks, heads, dim, gk);
  indexer_bwd_weight_kernel<<<heads, 256, 0, s>>>(wpart, rows, heads, gw);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int distillation_target_launch(const float* q, const float* kc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* target, cudaStream_t s,
                               float* qsum) {
  const int64_t n = (int64_t)B * Hkv * T;
  if (n <= 0 || blocks <= 0) return GN_OK;
  GN_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && ratio >= 1 && D >= 1, "distillation target: %d query heads, %d kv heads, ratio %d", Hq, Hkv, ratio);
  if (qsum && T >= 64 && blocks >= 64) {
    float* scale = qsum + n * D;                 // one float behind the sums: 1 / heads of a group
    set_scalar_kernel<<<1, 1, 0, s>>>(scale, 1.0f / (float)(Hq / Hkv));
    head_sum_kernel<<<(unsigned)ceil_div(n * D, 256), 256, 0, s>>>(q, B, Hq, Hkv, T, D, qsum);
    GN_LAUNCH_CHECK();
    for (int64_t i = 0; i < (int64_t)B * Hkv; ++i)
      GN_TRY(dot_scores_launch(target + i * T * blocks, qsum + i * T * D, kc + i * blocks * D, scale, T, blocks, D, s));
    target_softmax_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, s>>>(target, n, T, blocks, ratio);
    GN_LAUNCH_CHECK();
    return GN_OK;
  }
  distillation_target_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, s>>>(q, kc, B, Hq, Hkv, T, D, blocks, ratio, target);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int distillation_grad_launch(const float* scores, const float* target, const int32_t* candidates, const int32_t* candidate_counts, int cap, int64_t rows, int blocks,
                             int seq, int ratio, float weight, float* grad, cudaStream_t s) {
  if (rows <= 0 || blocks <= 0) return GN_OK;
  GN_REQUIRE(seq >= 1 && ratio >= 1 && (!candidates || (candidate_counts && cap >= 1)), "distillation gradient: seq %d, ratio %d, cap %d", seq, ratio, cap);
  distillation_grad_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, s>>>(scores, target, candidates, candidate_counts, cap, rows, blocks, seq, ratio, weight, grad);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int select_hierarchical_launch(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int pool, int budget, float* gmax, int32_t* chosen,
                               int32_t* selection, int32_t* counts, int32_t* candidates, int32_t* candidate_counts, cudaStream_t s) {
  if (tokens <= 0) return GN_OK;
  GN_REQUIRE(ratio >= 1 && pool >= 1 && blocks >= 0 && topk >= 0, "select_blocks_hierarchical: ratio %d, pool %d, blocks %d, topk %d", ratio, pool, blocks, topk);
  const int per_token = max(1, (budget + pool - 1) / pool);
  select_hierarchical_kernel<<<(unsigned)ceil_div(tokens, 8), 256, 0, s>>>(scores, tokens, blocks, offset, ratio, topk, pool, per_token, gmax, chosen, selection, counts,
                                                                           candidates, candidate_counts);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int select_within_pool_launch(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, const int32_t* candidates,
                              const int32_t* candidate_counts, int cap, int32_t* selection, int32_t* counts, cudaStream_t s) {
  if (tokens <= 0) return GN_OK;
  GN_REQUIRE(ratio >= 1 && cap >= 1 && topk >= 0, "select_blocks_within_pool: ratio %d, cap %d, topk %d", ratio, cap, topk);
  select_within_pool_kernel<<<(unsigned)ceil_div(tokens, 8), 256, 0, s>>>(scores, tokens, blocks, offset, ratio, topk, candidates, candidate_counts, cap, selection, counts);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
