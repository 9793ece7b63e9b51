// TEST INFRASTRUCTURE, NOT PRODUCT: CPU restatement of the building blocks of the reference's compressed
// ("flash") attention layers, used only to check the CUDA kernels.
//
//   channel compressor forward        model/compress.go:93-177, backward :182-237
//   compression of K and V per head    model/compress_attention.go:562-621 (compressForward, no segment mask)
//   attention over preceding blocks    model/compress_attention.go:624-673 (compressedAttentionForward)
//   attention over selected blocks     model/compress_attention.go:321-374 (compressedAttentionForwardSparse)
//   backward over preceding blocks     model/compress_attention.go:735-781 (compressedAttentionBackward)
//   local sliding-window branch        model/compress_attention.go:487-536 (attentionForwardWindowed = the ordinary
//                                      attention with a window, kernels/scalar/attention.go:16-205)
//   merge of two softmax branches      model/compress_attention.go:440-466 (mergeAttentionBranches)
//   block selection                    model/indexer.go:160-262 (TopK, SelectBlocks, topKIndices = stable argsort[:k])
//
// Pinned to the reference's known answers in tests/test_oracle_golden.py: model/compress_test.go:10-26,
// model/indexer_test.go:318-325,437-470.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <vector>

#include "backend.h"

namespace gnor {

// hidden [B, T, d], value [B, T, C], weight [C, d] (logits = hidden weight^T), bias [ratio, C]
// -> compressed [B, ceil(T / ratio), C]; probabilities (nullable) [B, blocks, ratio, C].
inline void compressor_forward(const Backend& bk, const float* hidden, const float* value, const float* weight, const float* bias, int B, int T, int d, int C,
                               int ratio, float* compressed, float* probabilities) {
  const int blocks = (T + ratio - 1) / ratio;
  std::vector<float> logits((size_t)B * T * C);
  bk.matmul_t(logits.data(), hidden, weight, B * T, C, d);
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int c = 0; c < C; ++c) logits[((size_t)b * T + t) * C + c] += bias[(size_t)(t % ratio) * C + c];
  std::fill(compressed, compressed + (size_t)B * blocks * C, 0.0f);
  std::vector<float> prob(ratio);
  for (int b = 0; b < B; ++b)
    for (int blk = 0; blk < blocks; ++blk)
      for (int c = 0; c < C; ++c) {
        float mx = -INFINITY;
        for (int r = 0; r < ratio; ++r) {
          const int t = blk * ratio + r;
          if (t >= T) continue;
          mx = std::max(mx, logits[((size_t)b * T + t) * C + c]);
        }
        double total = 0;
        for (int r = 0; r < ratio; ++r) {
          const int t = blk * ratio + r;
          float p = 0.0f;
          if (t < T && mx > -INFINITY) p = (float)std::exp((double)(logits[((size_t)b * T + t) * C + c] - mx));
          prob[r] = p; total += (double)p;
        }
        float acc = 0.0f;
        if (total > 0) {
          const float inv = (float)(1.0 / total);
          for (int r = 0; r < ratio; ++r) {
            prob[r] *= inv;
            const int t = blk * ratio + r;
            if (t < T) acc += prob[r] * value[((size_t)b * T + t) * C + c];
          }
          compressed[((size_t)b * blocks + blk) * C + c] = acc;
        }
        if (probabilities)
          for (int r = 0; r < ratio; ++r) probabilities[(((size_t)b * blocks + blk) * ratio + r) * C + c] = prob[r];
      }
}

// ChannelCompressor.Backward (model/compress.go:182-237, no segment mask): from the gradient of the compressed output to
// grad_hidden [B, T, d] and grad_value [B, T, C] (overwritten) and grad_weight [C, d], grad_bias [ratio, C] (accumulated).
// dlogit_j = p_j g (value_j - compressed); dvalue_j = p_j g; Linear.Backward: dW += dlogits^T hidden, dhidden = dlogits W.
inline void compressor_backward(const Backend& bk, const float* hidden, const float* value, const float* weight, const float* probabilities,
                                const float* compressed, const float* grad_compressed, int B, int T, int d, int C, int ratio, float* grad_hidden,
                                float* grad_value, float* grad_weight, float* grad_bias) {
  const int blocks = (T + ratio - 1) / ratio;
  std::vector<float> gl((size_t)B * T * C, 0.0f);
  std::fill(grad_value, grad_value + (size_t)B * T * C, 0.0f);
  for (int b = 0; b < B; ++b)
    for (int blk = 0; blk < blocks; ++blk)
      for (int c = 0; c < C; ++c) {
        const float g = grad_compressed[((size_t)b * blocks + blk) * C + c], cv = compressed[((size_t)b * blocks + blk) * C + c];
        for (int r = 0; r < ratio; ++r) {
          const int t = blk * ratio + r;
          if (t >= T) continue;
          const float p = probabilities[(((size_t)b * blocks + blk) * ratio + r) * C + c];
          const float v = value[((size_t)b * T + t) * C + c];
          gl[((size_t)b * T + t) * C + c] += p * g * (v - cv);
          grad_value[((size_t)b * T + t) * C + c] += p * g;
        }
      }
  // dhidden = dlogits [BT, C] . W [C, d];  dW += dlogits^T . hidden
  bk.matmul(grad_hidden, gl.data(), weight, B * T, d, C);
  std::vector<float> glt((size_t)C * B * T), dw((size_t)C * d);
  for (int i = 0; i < B * T; ++i) for (int c = 0; c < C; ++c) glt[(size_t)c * B * T + i] = gl[(size_t)i * C + c];
  bk.matmul(dw.data(), glt.data(), hidden, C, d, B * T);
  for (size_t i = 0; i < dw.size(); ++i) grad_weight[i] += dw[i];
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int c = 0; c < C; ++c) grad_bias[(size_t)(t % ratio) * C + c] += gl[((size_t)b * T + t) * C + c];
}

// q [B, Hq, T, D], kc / vc [B, Hkv, blocks, D] -> out [B, Hq, T, D], lse [B, Hq, T]: the queries of block b attend the
// compressed blocks 0 .. b-1 (none for block 0: zero output, lse = -inf).
inline void compressed_attention_forward(const Backend& bk, const float* q, const float* kc, const float* vc, int B, int Hq, int Hkv, int T, int D, int blocks,
                                         int ratio, float* out, float* lse) {
  const int hr = Hq / Hkv;
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h) {
      const size_t qi = (size_t)b * Hq + h;
      const size_t kbase = ((size_t)b * Hkv + h / hr) * blocks * D;
      for (int blk = 0; blk < blocks; ++blk) {
        const int start = blk * ratio, end = std::min(start + ratio, T);
        if (end <= start) continue;
        float* o = out + (qi * T + start) * D;
        float* l = lse ? lse + qi * T + start : nullptr;
        if (blk == 0) {
          std::fill(o, o + (size_t)(end - start) * D, 0.0f);
          if (l) std::fill(l, l + (end - start), -INFINITY);
          continue;
        }
        // position offset = blk: every compressed key index is below every query position (no causal cut inside)
        bk.attention_forward(q + (qi * T + start) * D, kc + kbase, vc + kbase, end - start, blk, D, blk, -1, nullptr, 0, o, l);
      }
    }
}

// The cached inference form (forwardCompressed, model/compress_attention.go:962-1003): T new tokens at positions offset .. over
// `blocks` cached compressed blocks; token t attends to the first min((offset + t) / ratio, blocks) of them, one row at a time.
inline void compressed_attention_forward_at(const Backend& bk, const float* q, const float* kc, const float* vc, int B, int Hq, int Hkv, int T, int D, int blocks,
                                            int ratio, int offset, float* out, float* lse) {
  const int hr = Hq / Hkv;
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h) {
      const size_t qi = (size_t)b * Hq + h;
      const size_t kbase = ((size_t)b * Hkv + h / hr) * blocks * D;
      for (int t = 0; t < T; ++t) {
        const int count = std::min((offset + t) / ratio, blocks);
        float* o = out + (qi * T + t) * D;
        if (count == 0) { std::fill(o, o + D, 0.0f); if (lse) lse[qi * T + t] = -INFINITY; continue; }
        bk.attention_forward(q + (qi * T + t) * D, kc + kbase, vc + kbase, 1, count, D, count, -1, nullptr, 0, o, lse ? lse + qi * T + t : nullptr);
      }
    }
}

// compressedAttentionBackward (model/compress_attention.go:735-781, no segment mask): per block the ordinary attention
// backward of its queries against the blocks before it; dq [B, Hq, T, D], dkc / dvc [B, Hkv, blocks, D] are accumulated into.
// row_correction (nullable, [B, Hq, T]) replaces sum_j p_j dp_j when the branch's output was merged with another branch.
inline void compressed_attention_backward(const Backend& bk, const float* q, const float* kc, const float* vc, const float* dout, const float* lse,
                                          const float* row_correction, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* dq, float* dkc,
                                          float* dvc) {
  const int hr = Hq / Hkv;
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h) {
      const size_t qi = (size_t)b * Hq + h;
      const size_t kbase = ((size_t)b * Hkv + h / hr) * blocks * D;
      for (int blk = 1; blk < blocks; ++blk) {
        const int start = blk * ratio, end = std::min(start + ratio, T);
        if (end <= start) continue;
        bk.attention_backward(q + (qi * T + start) * D, kc + kbase, vc + kbase, dout + (qi * T + start) * D, lse + qi * T + start,
                              row_correction ? row_correction + qi * T + start : nullptr, end - start, blk, D, blk, -1, nullptr, 0,
                              dq + (qi * T + start) * D, dkc + kbase, dvc + kbase);
      }
    }
}

// The same over selected blocks only (model/compress_attention.go:321-374, no segment mask): selection
// [B * Hkv, T, topk] block indices and counts [B * Hkv, T]; a token without a selected block yields zeros, lse = -inf.
inline void compressed_attention_sparse_forward(const Backend& bk, const float* q, const float* kc, const float* vc, const int32_t* selection,
                                                const int32_t* counts, int B, int Hq, int Hkv, int T, int D, int blocks, int topk, float* out, float* lse) {
  const int hr = Hq / Hkv;
  std::vector<float> ks((size_t)std::max(topk, 1) * D), vs((size_t)std::max(topk, 1) * D);
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h) {
      const size_t qi = (size_t)b * Hq + h, kvh = (size_t)b * Hkv + h / hr;
      const size_t kbase = kvh * blocks * D;
      for (int t = 0; t < T; ++t) {
        float* o = out + (qi * T + t) * D;
        const int n = counts[kvh * T + t];
        if (n <= 0) { std::fill(o, o + D, 0.0f); if (lse) lse[qi * T + t] = -INFINITY; continue; }
        const int32_t* sel = selection + (kvh * T + t) * topk;
        for (int i = 0; i < n; ++i) {
          std::copy(kc + kbase + (size_t)sel[i] * D, kc + kbase + (size_t)(sel[i] + 1) * D, ks.begin() + (size_t)i * D);
          std::copy(vc + kbase + (size_t)sel[i] * D, vc + kbase + (size_t)(sel[i] + 1) * D, vs.begin() + (size_t)i * D);
        }
        bk.attention_forward(q + (qi * T + t) * D, ks.data(), vs.data(), 1, n, D, n, -1, nullptr, 0, o, lse ? lse + qi * T + t : nullptr);
      }
    }
}

// Backward of the selected-block form (model/compress_attention.go:376-433, no segment mask): per token the selected blocks are
// gathered, the one-row backward runs on them, and the key / value gradients are scattered back; all three accumulate.
inline void compressed_attention_sparse_backward(const Backend& bk, const float* q, const float* kc, const float* vc, const float* dout, const float* lse,
                                                 const float* row_correction, const int32_t* selection, const int32_t* counts, int B, int Hq, int Hkv, int T,
                                                 int D, int blocks, int topk, float* dq, float* dkc, float* dvc) {
  const int hr = Hq / Hkv;
  const size_t cap = (size_t)std::max(topk, 1) * D;
  std::vector<float> ks(cap), vs(cap), gk(cap), gv(cap);
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < Hq; ++h) {
      const size_t qi = (size_t)b * Hq + h, kvh = (size_t)b * Hkv + h / hr;
      const size_t kbase = kvh * blocks * D;
      for (int t = 0; t < T; ++t) {
        const int n = counts[kvh * T + t];
        if (n <= 0) continue;
        const int32_t* sel = selection + (kvh * T + t) * topk;
        for (int i = 0; i < n; ++i) {
          std::copy(kc + kbase + (size_t)sel[i] * D, kc + kbase + (size_t)(sel[i] + 1) * D, ks.begin() + (size_t)i * D);
          std::copy(vc + kbase + (size_t)sel[i] * D, vc + kbase + (size_t)(sel[i] + 1) * D, vs.begin() + (size_t)i * D);
        }
        std::fill(gk.begin(), gk.begin() + (size_t)n * D, 0.0f); std::fill(gv.begin(), gv.begin() + (size_t)n * D, 0.0f);
        bk.attention_backward(q + (qi * T + t) * D, ks.data(), vs.data(), dout + (qi * T + t) * D, lse + qi * T + t,
                              row_correction ? row_correction + qi * T + t : nullptr, 1, n, D, n, -1, nullptr, 0, dq + (qi * T + t) * D, gk.data(), gv.data());
        for (int i = 0; i < n; ++i)
          for (int c = 0; c < D; ++c) { dkc[kbase + (size_t)sel[i] * D + c] += gk[(size_t)i * D + c]; dvc[kbase + (size_t)sel[i] * D + c] += gv[(size_t)i * D + c]; }
      }
    }
}

// Two normalised branches that share one softmax over the union of their keys: rows x D outputs and rows log-sum-exps.
inline void merge_branches(const float* oa, const float* la, const float* ob, const float* lb, int64_t rows, int D, float* out, float* lse) {
  for (int64_t r = 0; r < rows; ++r) {
    const float a = la[r], b = lb[r];
    const float mx = std::max(a, b);
    float* o = out + r * D;
    if (mx == -INFINITY) { std::fill(o, o + D, 0.0f); if (lse) lse[r] = mx; continue; }
    const float wa = (float)std::exp((double)(a - mx)), wb = (float)std::exp((double)(b - mx));
    const float total = wa + wb;
    const float inv = (float)(1.0 / (double)total);
    for (int c = 0; c < D; ++c) o[c] = (wa * oa[r * D + c] + wb * ob[r * D + c]) * inv;
    if (lse) lse[r] = mx + (float)std::log((double)total);
  }
}

// The k largest of values[0, n) in descending order, ties toward the smaller index (= stable argsort descending, cut).
inline std::vector<int> topk_indices(const float* values, int n, int k) {
  if (k <= 0) return {};
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return values[a] > values[b]; });
  if (k < n) order.resize(k);
  return order;
}

// scores [tokens, blocks] -> selection [tokens, topk] (-1 padded) and counts [tokens]: token t (absolute position
// offset + t) may take the blocks [0, min((offset + t) / ratio, blocks)).
inline void select_blocks(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int32_t* selection, int32_t* counts) {
  for (int t = 0; t < tokens; ++t) {
    int allowed = std::min((offset + t) / ratio, blocks);
    int32_t* sel = selection + (size_t)t * std::max(topk, 0);
    for (int i = 0; i < topk; ++i) sel[i] = -1;
    if (allowed <= 0 || topk <= 0) { counts[t] = 0; continue; }
    const std::vector<int> idx = topk_indices(scores + (size_t)t * blocks, allowed, std::min(topk, allowed));
    counts[t] = (int32_t)idx.size();
    for (size_t i = 0; i < idx.size(); ++i) sel[i] = idx[i];
  }
}

// The score part of SparseIndexer.Backward (model/indexer.go:107-151) for one key set: grad_scores [rows, blocks], query
// [rows, heads, dim], key [blocks, heads, dim]; grad_query and grad_key are overwritten, grad_weight [heads] accumulates.
// float32 accumulation in the reference's loop order (row, block, head).
inline void indexer_scores_backward(const float* grad_scores, const float* query, const float* key, const float* weight, int rows, int blocks, int heads, int dim,
                                    float* grad_query, float* grad_key, float* grad_weight) {
  std::fill(grad_query, grad_query + (size_t)rows * heads * dim, 0.0f);
  std::fill(grad_key, grad_key + (size_t)blocks * heads * dim, 0.0f);
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < blocks; ++b) {
      const float g = grad_scores[(size_t)r * blocks + b];
      for (int h = 0; h < heads; ++h) {
        const size_t qb = ((size_t)r * heads + h) * dim, kb = ((size_t)b * heads + h) * dim;
        float dot = 0.0f;
        for (int i = 0; i < dim; ++i) dot += query[qb + i] * key[kb + i];
        if (dot <= 0) continue;
        grad_weight[h] += g * dot;
        const float wg = g * weight[h];
        for (int i = 0; i < dim; ++i) { grad_query[qb + i] += wg * key[kb + i]; grad_key[kb + i] += wg * query[qb + i]; }
      }
    }
}

// distillationTarget (model/compress_attention.go:155-196) for every (batch, kv head): per token the softmax, over the allowed
// blocks, of the main attention logits averaged over the query heads of the group.  target [B * Hkv, T, blocks], zero elsewhere.
inline void indexer_distillation_target(const float* q, const float* kc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* target) {
  const int hr = Hq / Hkv;
  std::fill(target, target + (size_t)B * Hkv * T * blocks, 0.0f);
  std::vector<float> logits(std::max(blocks, 1));
  for (int b = 0; b < B; ++b)
    for (int hk = 0; hk < Hkv; ++hk)
      for (int t = 0; t < T; ++t) {
        const int allowed = std::min(t / ratio, blocks);
        if (allowed == 0) continue;
        float* row = target + (((size_t)b * Hkv + hk) * T + t) * blocks;
        float mx = -INFINITY;
        for (int j = 0; j < allowed; ++j) {
          float sum = 0.0f;
          for (int hh = 0; hh < hr; ++hh) {
            const float* qr = q + (((size_t)b * Hq + hk * hr + hh) * T + t) * D;
            const float* kr = kc + (((size_t)b * Hkv + hk) * blocks + j) * D;
            float dot = 0.0f;
            for (int c = 0; c < D; ++c) dot += qr[c] * kr[c];
            sum += dot;
          }
          logits[j] = sum / (float)hr;
          mx = std::max(mx, logits[j]);
        }
        double total = 0.0;
        for (int j = 0; j < allowed; ++j) { const double v = std::exp((double)(logits[j] - mx)); row[j] = (float)v; total += v; }
        for (int j = 0; j < allowed; ++j) row[j] /= (float)total;
      }
}

// The gradient of the indexer's distillation loss with respect to its scores (model/compress_attention.go:120-151):
// (softmax over the allowed blocks - target) * weight, row r being token r % seq.  With candidates [rows, cap] the scores and
// the target are first restricted to each row's candidate list (restrictIndexerToPool, :203-231): -inf and 0 outside, the target
// renormalised inside; a row without a finite score gets probabilities 0 (maskedIndexerSoftmax, :266-303).
inline void indexer_distillation_grad(const float* scores, const float* target, const int32_t* candidates, const int32_t* candidate_counts, int cap, int64_t rows,
                                      int blocks, int seq, int ratio, float weight, float* grad) {
  std::vector<float> sc(std::max(blocks, 1)), tg(std::max(blocks, 1));
  std::vector<char> in(std::max(blocks, 1));
  for (int64_t r = 0; r < rows; ++r) {
    std::copy(scores + r * blocks, scores + (r + 1) * blocks, sc.begin());
    std::copy(target + r * blocks, target + (r + 1) * blocks, tg.begin());
    if (candidates) {
      std::fill(in.begin(), in.end(), 0);
      for (int i = 0; i < std::min(candidate_counts[r], cap); ++i) { const int e = candidates[r * cap + i]; if (e >= 0 && e < blocks) in[e] = 1; }
      double total = 0.0;
      for (int e = 0; e < blocks; ++e) { if (!in[e]) { sc[e] = -INFINITY; tg[e] = 0.0f; } else total += (double)tg[e]; }
      if (total > 0) for (int e = 0; e < blocks; ++e) if (in[e]) tg[e] = (float)((double)tg[e] / total);
    }
    float* g = grad + r * blocks;
    const int allowed = std::min((int)(r % seq) / ratio, blocks);
    for (int e = 0; e < blocks; ++e) g[e] = (0.0f - tg[e]) * weight;
    if (allowed == 0) continue;
    float mx = sc[0];
    for (int e = 1; e < allowed; ++e) mx = std::max(mx, sc[e]);
    if (mx == -INFINITY) continue;
    double total = 0.0;
    std::vector<float> p(allowed);
    for (int e = 0; e < allowed; ++e) { const double v = std::exp((double)(sc[e] - mx)); p[e] = (float)v; total += v; }
    for (int e = 0; e < allowed; ++e) g[e] = (p[e] / (float)total - tg[e]) * weight;
  }
}

// selectRowBlockMax over a score matrix (model/indexer.go:442-513): super-blocks of `pool` entries are ranked by the maximum
// score among their causally allowed entries, the best ceil(budget / pool) super-blocks (at least one) give the candidate
// entries -- super-blocks in rank order, entries ascending inside --, and the selection is the top-k of the candidates by
// score, ties toward the earlier candidate.  candidates [tokens, cap], cap = max(1, ceil(budget / pool)) * pool, -1 padded.
inline int hierarchical_cap(int pool, int budget) { pool = std::max(pool, 1); return std::max(1, (budget + pool - 1) / pool) * pool; }
inline void select_blocks_hierarchical(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int pool, int budget, int32_t* selection,
                                       int32_t* counts, int32_t* candidates, int32_t* candidate_counts) {
  pool = std::max(pool, 1);
  const int per_token = std::max(1, (budget + pool - 1) / pool), cap = per_token * pool;
  for (int t = 0; t < tokens; ++t) {
    const int allowed = std::min((offset + t) / ratio, blocks);
    int32_t* sel = selection + (size_t)t * std::max(topk, 0);
    int32_t* cand = candidates + (size_t)t * cap;
    for (int i = 0; i < topk; ++i) sel[i] = -1;
    for (int i = 0; i < cap; ++i) cand[i] = -1;
    counts[t] = 0; candidate_counts[t] = 0;
    if (allowed <= 0 || topk <= 0) continue;
    const float* row = scores + (size_t)t * blocks;
    const int groups = (allowed + pool - 1) / pool;
    std::vector<float> gmax(groups, -INFINITY);
    for (int e = 0; e < allowed; ++e) gmax[e / pool] = std::max(gmax[e / pool], row[e]);
    const std::vector<int> chosen = topk_indices(gmax.data(), groups, std::min(per_token, groups));
    std::vector<int> list; std::vector<float> fine;
    for (int g : chosen)
      for (int e = g * pool; e < std::min((g + 1) * pool, allowed); ++e) { list.push_back(e); fine.push_back(row[e]); }
    candidate_counts[t] = (int32_t)list.size();
    std::copy(list.begin(), list.end(), cand);
    const std::vector<int> order = topk_indices(fine.data(), (int)fine.size(), std::min<int>(topk, (int)fine.size()));
    counts[t] = (int32_t)order.size();
    for (size_t i = 0; i < order.size(); ++i) sel[i] = list[order[i]];
  }
}

// selectWithinPool over a score matrix (model/indexer.go:547-613): the candidates of a token that lie in [0, allowed) are
// kept in their order and the top-k of them by score is the selection, ties toward the earlier kept candidate.
inline void select_blocks_within_pool(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, const int32_t* candidates,
                                      const int32_t* candidate_counts, int cap, int32_t* selection, int32_t* counts) {
  for (int t = 0; t < tokens; ++t) {
    const int allowed = std::min((offset + t) / ratio, blocks);
    int32_t* sel = selection + (size_t)t * std::max(topk, 0);
    for (int i = 0; i < topk; ++i) sel[i] = -1;
    counts[t] = 0;
    if (topk <= 0) continue;
    const float* row = scores + (size_t)t * blocks;
    std::vector<int> kept; std::vector<float> fine;
    for (int i = 0; i < std::min(candidate_counts[t], cap); ++i) {
      const int e = candidates[(size_t)t * cap + i];
      if (e < 0 || e >= allowed) continue;
      kept.push_back(e); fine.push_back(row[e]);
    }
    const std::vector<int> order = topk_indices(fine.data(), (int)fine.size(), std::min<int>(topk, (int)fine.size()));
    counts[t] = (int32_t)order.size();
    for (size_t i = 0; i < order.size(); ++i) sel[i] = kept[order[i]];
  }
}

}  // namespace gnor
