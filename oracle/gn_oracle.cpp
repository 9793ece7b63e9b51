// TEST INFRASTRUCTURE (CPU oracle). Not part of the shipped library; only
// tests, the smoke check and the benchmark's CPU-baseline leg may load it.
//
// C entry points over the CPU restatement of the reference's RL-step path:
//   * the numeric backend (kernels/backend.go), see backend.h
//   * losses and backward primitives (tensors/loss.go:16-46,
//     tensors/backward.go:11-131, tensors/math.go:38-45)
//   * the sampler (inference/sampler.go:16-77, tensors/random.go:60-80)
//   * the dense transformer (model.h)
//   * the generation loop (inference/engine.go:112-369)
//   * the policy-gradient step (trainer/rl.go:14-60) and the batch assembly
//     of cmd/chat_rl/main.go:137-183.
//
// Parity status: the backend, loss, gradient, sampler (argmax / top-k
// membership), rotary, window and padded-vocab functions are pinned against
// the known answers in the reference's own tests (see tests/test_oracle_*.py).
// PolicyGradientStep values, the advantage computation and the stochastic
// sampler's draws are NOT pinned by any reference test: for those this file
// is "parity unpinned" and parity means agreement with this restatement.
#include <cstdio>
#include <cstdlib>
#ifdef _OPENMP
#include <omp.h>
#endif
#include "backend.h"
#include "flash.h"
#include "model.h"
#include "optimizer.h"
#include "philox.h"

namespace gnor {
int Backend::omp_workers() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// ------------------------------------------------------------------ sampler
// inference/sampler.go:62-77
static float kth_largest(const float* values, int n, int rank) {
  std::vector<float> top(values, values + rank);
  std::sort(top.begin(), top.end());
  for (int i = rank; i < n; ++i) {
    float v = values[i];
    if (v > top[0]) {
      top[0] = v;
      for (int j = 0; j + 1 < rank && top[j] > top[j + 1]; ++j) std::swap(top[j], top[j + 1]);
    }
  }
  return top[0];
}

// One row.  `uniforms` (length n) when non-null, else the counter generator.
static int sample_row(const float* logits, int n, const float* uniforms, uint64_t seed, uint32_t step, uint32_t row,
                      float temperature, int top_k) {
  if (temperature <= 0) {  // inference/sampler.go:27-29,37-45
    int best = 0;
    for (int i = 1; i < n; ++i) if (logits[i] > logits[best]) best = i;
    return best;
  }
  const float ninf = -std::numeric_limits<float>::infinity();
  float threshold = ninf;
  bool mask = top_k > 0 && top_k < n;
  if (mask) threshold = kth_largest(logits, n, top_k);
  // tensors/random.go:60-80
  int best = 0;
  float best_score = ninf;
  for (int i = 0; i < n; ++i) {
    float value = logits[i];
    if (mask && !(value >= threshold)) value = ninf;
    float u = uniforms ? uniforms[i] : gnrng::sampler_uniform(seed, step, row, (uint32_t)i);
    if (u <= 0) u = 1e-12f;
    float gumbel = -(float)std::log(-std::log((double)u));
    float score = value / temperature + gumbel;
    if (score > best_score) { best_score = score; best = i; }
  }
  return best;
}

struct Rollouts {
  std::vector<std::vector<int32_t>> rows;  // prompt + generated, terminal token stripped
};

}  // namespace gnor

using namespace gnor;

extern "C" {

int or_num_threads() { return Backend::omp_workers(); }
void or_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#endif
}

// ------------------------------------------------------------ backend (Tier A)
#define BK(MODE_) Backend bk; bk.mode = (MODE_)
void or_add(int m, float* d, const float* a, const float* b, int64_t n) { BK(m); bk.add(d, a, b, n); }
void or_subtract(int m, float* d, const float* a, const float* b, int64_t n) { BK(m); bk.subtract(d, a, b, n); }
void or_multiply(int m, float* d, const float* a, const float* b, int64_t n) { BK(m); bk.multiply(d, a, b, n); }
void or_divide(int m, float* d, const float* a, const float* b, int64_t n) { BK(m); bk.divide(d, a, b, n); }
void or_scale(int m, float* d, const float* s, float f, int64_t n) { BK(m); bk.scale(d, s, f, n); }
void or_add_scaled(int m, float* d, const float* base, const float* s, float f, int64_t n) { BK(m); bk.add_scaled(d, base, s, f, n); }
void or_negate(int m, float* d, const float* s, int64_t n) { BK(m); bk.negate(d, s, n); }
void or_abs(int m, float* d, const float* s, int64_t n) { BK(m); bk.abs(d, s, n); }
void or_square(int m, float* d, const float* s, int64_t n) { BK(m); bk.square(d, s, n); }
void or_relu_squared(int m, float* d, const float* s, int64_t n) { BK(m); bk.relu_squared(d, s, n); }
void or_swiglu(int m, float* d, const float* g, const float* u, float c, int64_t n) { BK(m); bk.swiglu(d, g, u, c, n); }
void or_swiglu_backward(int m, float* gg, float* ug, const float* g, const float* u, const float* og, float c, int64_t n) { BK(m); bk.swiglu_backward(gg, ug, g, u, og, c, n); }
void or_exp(int m, float* d, const float* s, int64_t n) { BK(m); bk.exp(d, s, n); }
void or_sigmoid(int m, float* d, const float* s, int64_t n) { BK(m); bk.sigmoid(d, s, n); }
void or_tanh(int m, float* d, const float* s, int64_t n) { BK(m); bk.tanh(d, s, n); }
void or_rsqrt(int m, float* d, const float* s, int64_t n) { BK(m); bk.rsqrt(d, s, n); }
float or_sum(int m, const float* v, int64_t n) { BK(m); return bk.sum(v, n); }
float or_max(int m, const float* v, int64_t n) { BK(m); return bk.max(v, n); }
int64_t or_argmax(int m, const float* v, int64_t n) { BK(m); return bk.argmax(v, n); }
float or_dot(int m, const float* a, const float* b, int64_t n) { BK(m); return bk.dot(a, b, n); }
void or_matmul(int m, float* d, const float* l, const float* r, int rows, int cols, int inner) { BK(m); bk.matmul(d, l, r, rows, cols, inner); }
void or_matmul_transposed(int m, float* d, const float* l, const float* r, int rows, int cols, int inner) { BK(m); bk.matmul_t(d, l, r, rows, cols, inner); }
void or_softmax_lastdim(int m, float* d, const float* s, int64_t rows, int cols) { BK(m); bk.softmax_lastdim(d, s, rows, cols); }
void or_rmsnorm_lastdim(int m, float* d, const float* s, int64_t rows, int cols, float eps) { BK(m); bk.rmsnorm_lastdim(d, s, rows, cols, eps); }
void or_topk_indices(int m, int32_t* d, const float* s, int rows, int count, int k) { BK(m); bk.topk_indices(d, s, rows, count, k); }
void or_moe_gate_topk(int m, const float* logits, const float* bias, float* probs, int32_t* sel, float* w, int rows, int experts, int k) { BK(m); bk.moe_gate_topk(logits, bias, probs, sel, w, rows, experts, k); }
void or_grouped_matmul_transposed(int m, float* d, const float* in, const float* w, const int32_t* counts, int experts, int cols, int inner) { BK(m); bk.grouped_matmul_t(d, in, w, counts, experts, cols, inner); }
void or_indexer_scores(int m, float* d, const float* q, const float* k, const float* w, int rows, int blocks, int heads, int dim) { BK(m); bk.indexer_scores(d, q, k, w, rows, blocks, heads, dim); }
void or_indexer_block_max(int m, float* d, const float* s, int rows, int blocks, int group) { BK(m); bk.indexer_block_max(d, s, rows, blocks, group); }
void or_attention_forward(int m, const float* q, const float* k, const float* v, int ql, int kl, int hd, int offset, int window,
                          const int32_t* seg, int seg_len, float* out, float* lse) {
  BK(m); bk.attention_forward(q, k, v, ql, kl, hd, offset, window, seg, seg_len, out, lse);
}
void or_attention_forward_split(int m, const float* q, const float* k, const float* v, int ql, int kl, int hd, int offset, int window,
                                int kstart, int kend, const int32_t* seg, int seg_len, float* acc, float* mx, float* sm) {
  BK(m); bk.attention_forward_split(q, k, v, ql, kl, hd, offset, window, kstart, kend, seg, seg_len, acc, mx, sm);
}
// partials packed: acc [parts, ql, hd], mx [parts, ql], sm [parts, ql]
void or_attention_combine(int m, const float* acc, const float* mx, const float* sm, int parts, int ql, int hd, float* out, float* lse) {
  BK(m);
  std::vector<const float*> a(parts), x(parts), s(parts);
  for (int p = 0; p < parts; ++p) { a[p] = acc + (int64_t)p * ql * hd; x[p] = mx + (int64_t)p * ql; s[p] = sm + (int64_t)p * ql; }
  bk.attention_combine(a.data(), x.data(), s.data(), parts, ql, hd, out, lse);
}
void or_attention_backward(int m, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* rowcorr,
                           int ql, int kl, int hd, int offset, int window, const int32_t* seg, int seg_len, float* dq, float* dk, float* dv) {
  BK(m); bk.attention_backward(q, k, v, dout, lse, rowcorr, ql, kl, hd, offset, window, seg, seg_len, dq, dk, dv);
}

// ------------------------------------------------------------------ tensors
// tensors/loss.go:16-46.  Returns the valid count; losses[row] = 0 on ignored rows.
int64_t or_cross_entropy_per_position(int m, const float* logits, const int32_t* targets, int64_t rows, int vocab, int32_t ignore, float* losses) {
  BK(m);
  int64_t valid = 0;
  for (int64_t r = 0; r < rows; ++r) if (targets[r] != ignore) ++valid;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    losses[r] = 0;
    if (targets[r] == ignore) continue;
    const float* x = logits + r * vocab;
    float mx = bk.max(x, vocab);
    double sum = 0;
    for (int v = 0; v < vocab; ++v) sum += std::exp((double)(x[v] - mx));
    losses[r] = mx + (float)std::log(sum) - x[targets[r]];
  }
  return valid;
}
// tensors/backward.go:11-38
void or_cross_entropy_grad(int m, const float* logits, const int32_t* targets, int64_t rows, int vocab, int32_t ignore, float scale, float* grad) {
  BK(m);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float* g = grad + r * vocab;
    std::fill(g, g + vocab, 0.0f);
    if (targets[r] == ignore) continue;
    const float* x = logits + r * vocab;
    float mx = bk.max(x, vocab);
    double sum = 0;
    for (int v = 0; v < vocab; ++v) sum += std::exp((double)(x[v] - mx));
    double inv = 1.0 / sum;
    for (int v = 0; v < vocab; ++v) {
      float p = (float)(std::exp((double)(x[v] - mx)) * inv);
      if (v == targets[r]) p -= 1;
      g[v] = p * scale;
    }
  }
}
// tensors/math.go:38-45
void or_softcap(float* d, const float* s, float cap, int64_t n) {
  float inv = 1.0f / cap;
  for (int64_t i = 0; i < n; ++i) { float t = s[i] * inv; t = (float)std::tanh((double)t); d[i] = t * cap; }
}
// tensors/backward.go:108-116
void or_softcap_backward(float* d, const float* out, const float* gout, float cap, int64_t n) {
  float inv = 1.0f / cap;
  for (int64_t i = 0; i < n; ++i) { double sc = (double)out[i] * (double)inv; d[i] = gout[i] * (float)(1 - sc * sc); }
}
// tensors/backward.go:57-65
void or_relu_squared_backward(float* d, const float* in, const float* gout, int64_t n) {
  for (int64_t i = 0; i < n; ++i) d[i] = in[i] > 0 ? gout[i] * 2 * in[i] : 0.0f;
}
// tensors/backward.go:81-104
void or_rmsnorm_backward(float* d, const float* in, const float* gout, int64_t rows, int cols, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = in + r * cols; const float* g = gout + r * cols; float* o = d + r * cols;
    double ss = 0, dp = 0;
    for (int c = 0; c < cols; ++c) { ss += (double)x[c] * (double)x[c]; dp += (double)g[c] * (double)x[c]; }
    double rms = std::sqrt(ss / (double)cols + (double)eps);
    double inv = 1.0 / rms, coef = dp / ((double)cols * rms * rms * rms);
    for (int c = 0; c < cols; ++c) o[c] = (float)((double)g[c] * inv - coef * (double)x[c]);
  }
}
// tensors/backward.go:120-126
void or_sigmoid_backward(float* d, const float* out, const float* gout, int64_t n) {
  for (int64_t i = 0; i < n; ++i) d[i] = gout[i] * out[i] * (1 - out[i]);
}

// ------------------------------------------------------------------ sampler
// inference/sampler.go:16-25.  uniforms: [rows, vocab] or null (counter generator
// keyed by seeds[row / group], row index within the group, step).
void or_sample_next_token(const float* logits, int rows, int vocab, const float* uniforms, const uint64_t* seeds, int group,
                          uint32_t step, float temperature, int top_k, int32_t* out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    uint64_t seed = seeds ? seeds[r / group] : 0;
    out[r] = sample_row(logits + (int64_t)r * vocab, vocab, uniforms ? uniforms + (int64_t)r * vocab : nullptr, seed, step,
                        (uint32_t)(r % group), temperature, top_k);
  }
}
float or_kth_largest(const float* v, int n, int rank) { return kth_largest(v, n, rank); }
float or_sampler_uniform(uint64_t seed, uint32_t step, uint32_t row, uint32_t col) { return gnrng::sampler_uniform(seed, step, row, col); }
float or_reward_uniform(uint64_t seed, uint32_t rollout) { return gnrng::reward_uniform(seed, rollout); }
void or_philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t* out4) {
  gnrng::U4 r = gnrng::philox4x32_10(c0, c1, c2, c3, k0, k1);
  for (int i = 0; i < 4; ++i) out4[i] = r.v[i];
}

// -------------------------------------------------------------------- model
struct or_config {
  int32_t sequence_len, vocab_size, n_layer, n_head, n_kv_head, embed_dim, rotary_dims;
  char window_pattern[16];
  int32_t n_experts, experts_per_token, expert_hidden, shared_hidden;
  float moe_clamp, moe_scale;
  int32_t mla_latent, mla_rotary_dims;
};

void* or_model_create(const or_config* c, int mode) {
  Config cfg;
  cfg.sequence_len = c->sequence_len; cfg.vocab = c->vocab_size; cfg.n_layer = c->n_layer; cfg.n_head = c->n_head;
  cfg.n_kv_head = c->n_kv_head; cfg.embed_dim = c->embed_dim; cfg.rotary_dims = c->rotary_dims;
  cfg.window_pattern = c->window_pattern[0] ? std::string(c->window_pattern) : std::string("L");
  cfg.n_experts = c->n_experts; cfg.experts_per_token = c->experts_per_token; cfg.expert_hidden = c->expert_hidden; cfg.shared_hidden = c->shared_hidden;
  cfg.moe_clamp = c->moe_clamp; cfg.moe_scale = c->moe_scale; cfg.mla_latent = c->mla_latent; cfg.mla_rotary_dims = c->mla_rotary_dims;
  return new Model(cfg, mode);
}
void or_model_destroy(void* m) { delete (Model*)m; }
int or_model_param_count(void* m) { return (int)((Model*)m)->params.size(); }
// Names come back in sorted order (model/params.go:83-91).
const char* or_model_param_name(void* m, int i) {
  auto it = ((Model*)m)->params.begin(); std::advance(it, i); return it->first.c_str();
}
int64_t or_model_param_numel(void* m, const char* name) { auto& p = ((Model*)m)->P(name); return (int64_t)p.w.size(); }
void or_model_param_shape(void* m, const char* name, int* rows, int* cols) { auto& p = ((Model*)m)->P(name); *rows = p.rows; *cols = p.cols; }
float* or_model_param_data(void* m, const char* name) { return ((Model*)m)->P(name).w.data(); }
float* or_model_param_grad(void* m, const char* name) { return ((Model*)m)->P(name).g.data(); }
void or_model_zero_grad(void* m) { ((Model*)m)->zero_grad(); }
void or_model_window_sizes(void* m, int32_t* out) { auto& w = ((Model*)m)->windows; for (size_t i = 0; i < w.size(); ++i) out[i] = w[i]; }
int or_model_padded_vocab(void* m) { return ((Model*)m)->Vp; }
void or_apply_rotary(void* m, float* x, int B, int T, int H, int offset, float sign) {
  Model* mm = (Model*)m; std::vector<float> v(x, x + (size_t)B * T * H * mm->D); mm->rotary(v, B, T, H, offset, sign); std::copy(v.begin(), v.end(), x);
}
// Stand-alone rotary with caller tables (model/rotary.go:43-75), for the reference's known answers.
void or_rotary_tables(float* x, const float* cosv, const float* sinv, int half, int B, int T, int H, int D, int offset) {
  int R = 2 * half, off = D - R;
  for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) for (int h = 0; h < H; ++h) {
    float* p = x + (((size_t)b * T + t) * H + h) * D + off;
    const float* cw = cosv + (size_t)(offset + t) * half; const float* sw = sinv + (size_t)(offset + t) * half;
    for (int j = 0; j < half; ++j) { float a = p[j], c = p[half + j]; p[j] = a * cw[j] + c * sw[j]; p[half + j] = -a * sw[j] + c * cw[j]; }
  }
}

// Forward without cache ([B,T] -> [B,T,V]); T must be > 1.
void or_model_forward(void* m, const int32_t* ids, int B, int T, float* logits) {
  std::vector<float> out; ((Model*)m)->forward(out, ids, B, T, nullptr); std::copy(out.begin(), out.end(), logits);
}

// MLA models: the same function through the un-absorbed (training) construction (model/mla_test.go:279-293).
void or_model_forward_unabsorbed(void* m, const int32_t* ids, int B, int T, float* logits) {
  std::vector<float> out; ((Model*)m)->forward(out, ids, B, T, nullptr, true); std::copy(out.begin(), out.end(), logits);
}
// Routed-expert contribution of layer l for rows of normalised activations, with the selected expert ids.
void or_model_moe_forward(void* m, int layer, const float* flat, int64_t rows, float* out, int32_t* selected) {
  Model* mm = (Model*)m; std::vector<float> in(flat, flat + (size_t)rows * mm->cfg.embed_dim), o; std::vector<int32_t> sel;
  mm->moe_forward(o, in, rows, layer, &sel); std::copy(o.begin(), o.end(), out); if (selected) std::copy(sel.begin(), sel.end(), selected);
}

void* or_cache_create(void* m, int batch, int max_seq) { KVCache* c = new KVCache(); ((Model*)m)->cache_init(*c, batch, max_seq); return c; }
void or_cache_destroy(void* c) { delete (KVCache*)c; }
int or_cache_position(void* c) { return ((KVCache*)c)->pos; }
void or_cache_replicate(void* m, void* dst, void* src) { ((Model*)m)->cache_replicate(*(KVCache*)dst, *(KVCache*)src); }
void or_model_forward_cached(void* m, void* cache, const int32_t* ids, int B, int T, float* logits) {
  std::vector<float> out; ((Model*)m)->forward(out, ids, B, T, (KVCache*)cache); std::copy(out.begin(), out.end(), logits);
}

// ------------------------------------------------------------------- engine
// inference/engine.go:112-369 for ONE prompt (GenerateBatchWith semantics),
// with the tool/think machinery reduced to what remains when no tokenizer and
// no tool executor exist: every mask is 1, no forced tokens.  Rows complete on
// <|bos|> (= vocab-11) or <|assistant_end|> (= vocab-7), tokenizer/special.go:19-31.
// out_tokens: [group, max_tokens]; out_lengths[group] = generated tokens kept
// (terminal token stripped).  step_logits: optional [max_tokens, group, V]
// logits that each sampling step saw.  Returns the number of sampling steps run.
int or_generate(void* mp, const int32_t* prompt, int prompt_len, int group, int max_tokens, float temperature, int top_k,
                uint64_t seed, int32_t* out_tokens, int32_t* out_lengths, float* step_logits) {
  Model* m = (Model*)mp;
  int V = m->cfg.vocab;
  int bos = V - 11, aend = V - 7;
  KVCache pre; m->cache_init(pre, 1, prompt_len);
  std::vector<float> logits;
  m->forward(logits, prompt, 1, prompt_len, &pre);
  std::vector<float> cur((size_t)group * V);
  for (int g = 0; g < group; ++g) std::copy(logits.begin() + (size_t)(prompt_len - 1) * V, logits.begin() + (size_t)prompt_len * V, cur.begin() + (size_t)g * V);
  KVCache dec; m->cache_init(dec, group, prompt_len + max_tokens);
  m->cache_replicate(dec, pre);
  std::vector<char> completed(group, 0), kept_done(group, 0);
  for (int g = 0; g < group; ++g) out_lengths[g] = 0;
  int generated = 0;
  std::vector<int32_t> col(group);
  while (true) {
    if (max_tokens > 0 && generated >= max_tokens) break;
    bool all = true;
    for (int g = 0; g < group; ++g) if (!completed[g]) { all = false; break; }
    if (all) break;
    if (step_logits) std::copy(cur.begin(), cur.end(), step_logits + (size_t)generated * group * V);
    or_sample_next_token(cur.data(), group, V, nullptr, &seed, group, (uint32_t)generated, temperature, top_k, col.data());
    for (int g = 0; g < group; ++g) {
      int t = col[g];
      if (t == aend || t == bos) completed[g] = 1;
      if (!kept_done[g]) {
        if (t == aend || t == bos) kept_done[g] = 1;
        else out_tokens[(size_t)g * max_tokens + out_lengths[g]++] = t;
      }
    }
    ++generated;
    bool alldone = true;
    for (int g = 0; g < group; ++g) if (!kept_done[g]) { alldone = false; break; }
    if (alldone) break;  // GenerateBatchWith's callback stops the loop (engine.go:316-318,362-367)
    m->forward(cur, col.data(), group, 1, &dec);
  }
  return generated;
}

// Engine.GenerateWith + GenerateBatchWith with the forced-token queue and the thinking-trace state machine
// (inference/engine.go:256-314,349-367).  `forced` [group, forced_stride] with forced_counts[g] tokens queued for row
// g before the first step (what a handled tool call would queue; tool execution itself needs the tokenizer and is
// stubbed to "not handled", so the tool-call flags have no effect).  thinking / thinking_budget as GenerateOptions.
// out_masks parallels out_tokens: 1 = sampled, 0 = forced.
int or_generate_ex(void* mp, const int32_t* prompt, int prompt_len, int group, int max_tokens, float temperature, int top_k, uint64_t seed,
                   int thinking, int thinking_budget, const int32_t* forced, int forced_stride, const int32_t* forced_counts,
                   int32_t* out_tokens, int32_t* out_lengths, int32_t* out_masks) {
  Model* m = (Model*)mp;
  int V = m->cfg.vocab;
  const int bos = V - 11, aend = V - 7, think_start = V - 2, think_end = V - 1;   // tokenizer/special.go:19-31
  KVCache pre; m->cache_init(pre, 1, prompt_len);
  std::vector<float> logits;
  m->forward(logits, prompt, 1, prompt_len, &pre);
  std::vector<float> cur((size_t)group * V);
  for (int g = 0; g < group; ++g) std::copy(logits.begin() + (size_t)(prompt_len - 1) * V, logits.begin() + (size_t)prompt_len * V, cur.begin() + (size_t)g * V);
  KVCache dec; m->cache_init(dec, group, prompt_len + max_tokens);
  m->cache_replicate(dec, pre);
  struct Row { std::vector<int32_t> forced; bool in_thinking = false; int thinking_tokens = 0; bool completed = false, kept_done = false; };
  std::vector<Row> rows(group);
  for (int g = 0; g < group; ++g) {
    out_lengths[g] = 0;
    if ((thinking || thinking_budget > 0) && prompt_len > 0 && prompt[prompt_len - 1] == think_start) rows[g].in_thinking = true;   // engine.go:229-236
    if (forced && forced_counts) rows[g].forced.assign(forced + (size_t)g * forced_stride, forced + (size_t)g * forced_stride + forced_counts[g]);
  }
  int generated = 0;
  std::vector<int32_t> sampled(group), col(group), mask(group);
  while (true) {
    if (max_tokens > 0 && generated >= max_tokens) break;
    bool all = true;
    for (int g = 0; g < group; ++g) if (!rows[g].completed) { all = false; break; }
    if (all) break;
    or_sample_next_token(cur.data(), group, V, nullptr, &seed, group, (uint32_t)generated, temperature, top_k, sampled.data());
    for (int g = 0; g < group; ++g) {
      Row& st = rows[g];
      const bool is_forced = !st.forced.empty();
      mask[g] = is_forced ? 0 : 1;
      int t;
      if (is_forced) { t = st.forced.front(); st.forced.erase(st.forced.begin()); } else t = sampled[g];
      col[g] = t;
      if (t == aend || t == bos) st.completed = true;
      if (thinking || thinking_budget > 0) {
        if (t == think_start) { st.in_thinking = true; st.thinking_tokens = 0; }
        else if (t == think_end && st.in_thinking) st.in_thinking = false;
        else if (st.in_thinking) {
          st.thinking_tokens++;
          if (thinking_budget > 0 && st.thinking_tokens >= thinking_budget) st.forced.push_back(think_end);
        }
      }
      if (!st.kept_done) {
        if (t == aend || t == bos) st.kept_done = true;
        else { out_tokens[(size_t)g * max_tokens + out_lengths[g]] = t; if (out_masks) out_masks[(size_t)g * max_tokens + out_lengths[g]] = mask[g]; out_lengths[g]++; }
      }
    }
    ++generated;
    bool alldone = true;
    for (int g = 0; g < group; ++g) if (!rows[g].kept_done) { alldone = false; break; }
    if (alldone) break;
    m->forward(cur, col.data(), group, 1, &dec);
  }
  return generated;
}

// tensors/loss.go:84-213: forward KL from the student to the teacher's soft distribution per position (float64 inside),
// and its gradient (softmax(student/tau) - softmax(teacher/tau)) / tau * scale.  mask: null or one int per row (0 =
// masked: loss 0, zero gradient).  losses / grad nullable.  Returns the number of valid positions.
int64_t or_distillation(const float* student, const float* teacher, int64_t rows, int vocab, float temperature, const int32_t* mask, float scale,
                        float* losses, float* grad) {
  const double tau = temperature <= 0 ? 1.0 : (double)temperature;
  int64_t valid = 0;
  for (int64_t r = 0; r < rows; ++r) {
    const float* s = student + (size_t)r * vocab; const float* t = teacher + (size_t)r * vocab;
    if (mask && mask[r] == 0) {
      if (losses) losses[r] = 0.0f;
      if (grad) std::fill(grad + (size_t)r * vocab, grad + (size_t)(r + 1) * vocab, 0.0f);
      continue;
    }
    ++valid;
    double smax = -INFINITY, tmax = -INFINITY;
    for (int v = 0; v < vocab; ++v) { smax = std::max(smax, (double)s[v] / tau); tmax = std::max(tmax, (double)t[v] / tau); }
    double ssum = 0, tsum = 0, weighted = 0;
    for (int v = 0; v < vocab; ++v) {
      const double sw = std::exp((double)s[v] / tau - smax), tw = std::exp((double)t[v] / tau - tmax);
      ssum += sw; tsum += tw; weighted += tw * ((double)s[v] / tau);
    }
    if (losses) losses[r] = (float)(smax + std::log(ssum) - weighted / tsum);
    if (grad) {
      const double is = 1.0 / ssum, it = 1.0 / tsum, gs = (double)scale / tau;
      for (int v = 0; v < vocab; ++v)
        grad[(size_t)r * vocab + v] = (float)((std::exp((double)s[v] / tau - smax) * is - std::exp((double)t[v] / tau - tmax) * it) * gs);
    }
  }
  return valid;
}

// ----------------------------------------------------------------------- RL
// cmd/chat_rl/main.go:137-154.  mode 0: reward - group mean (the reference).
// mode 1: (reward - mean) / (population std + 1e-6), float32, a build-side
// definition that the reference does not have.
void or_advantage(const float* rewards, int groups, int group, int mode, float* adv) {
  for (int g = 0; g < groups; ++g) {
    const float* r = rewards + (size_t)g * group; float* a = adv + (size_t)g * group;
    float mean = 0;
    for (int i = 0; i < group; ++i) mean += r[i];
    mean /= (float)group;
    if (mode == 0) { for (int i = 0; i < group; ++i) a[i] = r[i] - mean; continue; }
    float var = 0;
    for (int i = 0; i < group; ++i) { float dlt = r[i] - mean; var += dlt * dlt; }
    var /= (float)group;
    float sd = std::sqrt(var);
    for (int i = 0; i < group; ++i) a[i] = (r[i] - mean) / (sd + 1e-6f);
  }
}

// cmd/chat_rl/main.go:156-182.  rollouts: ragged rows (prompt + kept tokens)
// given as tokens [n, stride] + lengths[n]; returns max_len; inputs/targets are
// [n, max_len-1].
int or_build_batch(const int32_t* tokens, const int32_t* lengths, const int32_t* prompt_lengths, int n, int stride, int pad_token,
                   int32_t* inputs, int32_t* targets) {
  int max_len = 0;
  for (int i = 0; i < n; ++i) max_len = std::max(max_len, (int)lengths[i]);
  int T = max_len - 1;
  for (int i = 0; i < n; ++i) {
    std::vector<int32_t> padded(tokens + (size_t)i * stride, tokens + (size_t)i * stride + lengths[i]);
    while ((int)padded.size() < max_len) padded.push_back(pad_token);
    for (int t = 0; t < T; ++t) {
      inputs[(size_t)i * T + t] = padded[t];
      targets[(size_t)i * T + t] = (t < prompt_lengths[i]) ? -1 : padded[t + 1];
    }
  }
  return max_len;
}

// trainer/rl.go:14-60.  Accumulates parameter gradients; returns the loss.
// nll_out ([B*T]) and dlogits_out ([B*T,V]) are optional taps.
float or_policy_gradient_step(void* mp, const int32_t* inputs, const int32_t* targets, const float* adv, int B, int T, float norm,
                              float* nll_out, float* dlogits_out, float* logits_out) {
  Model* m = (Model*)mp;
  int V = m->cfg.vocab;
  int64_t rows = (int64_t)B * T;
  TrainCtx ctx;
  m->train_forward(ctx, inputs, B, T);
  std::vector<float> nll(rows);
  or_cross_entropy_per_position(m->bk.mode, ctx.logits.data(), targets, rows, V, -1, nll.data());
  double loss = 0;
  for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) {
    int64_t i = (int64_t)b * T + t;
    if (targets[i] == -1) continue;
    loss += (double)nll[i] * (double)adv[b] / (double)norm;
  }
  std::vector<float> probs((size_t)rows * V), grad((size_t)rows * V, 0.0f);
  m->bk.softmax_lastdim(probs.data(), ctx.logits.data(), rows, V);
  for (int b = 0; b < B; ++b) {
    float sc = adv[b] / norm;
    for (int t = 0; t < T; ++t) {
      int64_t i = (int64_t)b * T + t;
      int32_t tg = targets[i];
      if (tg == -1) continue;
      for (int v = 0; v < V; ++v) {
        float g = probs[(size_t)i * V + v];
        if (v == tg) g -= 1;
        grad[(size_t)i * V + v] = g * sc;
      }
    }
  }
  if (nll_out) std::copy(nll.begin(), nll.end(), nll_out);
  if (dlogits_out) std::copy(grad.begin(), grad.end(), dlogits_out);
  if (logits_out) std::copy(ctx.logits.begin(), ctx.logits.end(), logits_out);
  m->train_backward(ctx, grad);
  return (float)loss;
}

// Loss + gradient at given logits only (the loss-path microbenchmark):
// trainer/rl.go:23-56 without the model.  adv is per sequence of seq_len rows.
double or_pg_loss_backward(int mode, const float* logits, const int32_t* targets, const float* adv, int64_t rows, int vocab, int seq_len,
                           float norm, float* nll, float* dlogits) {
  BK(mode);
  or_cross_entropy_per_position(mode, logits, targets, rows, vocab, -1, nll);
  double loss = 0;
  for (int64_t i = 0; i < rows; ++i) if (targets[i] != -1) loss += (double)nll[i] * (double)adv[i / seq_len] / (double)norm;
  if (dlogits) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i) {
      float* g = dlogits + i * vocab;
      std::fill(g, g + vocab, 0.0f);
      int32_t tg = targets[i];
      if (tg == -1) continue;
      std::vector<float> p(vocab);
      bk.softmax_lastdim(p.data(), logits + i * vocab, 1, vocab);
      float sc = adv[i / seq_len] / norm;
      for (int v = 0; v < vocab; ++v) { float x = p[v]; if (v == tg) x -= 1; g[v] = x * sc; }
    }
  }
  return loss;
}

// Training forward only: logits [B*T, V].
void or_train_forward(void* mp, const int32_t* ids, int B, int T, float* logits) {
  TrainCtx ctx; ((Model*)mp)->train_forward(ctx, ids, B, T); std::copy(ctx.logits.begin(), ctx.logits.end(), logits);
}

// ---------------------------------------------------------------- optimizer
void or_adamw_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, int step, float lr, float beta1, float beta2, float eps,
                   float weight_decay) { gnopt::adamw_step(param, grad, exp_avg, exp_avg_sq, n, step, lr, beta1, beta2, eps, weight_decay); }
void or_muon_step(int mode, float* param, const float* grad, float* mom, float* second_mom, int rows, int cols, float lr, float momentum, int ns_steps,
                  float beta2, float weight_decay) {
  BK(mode); gnopt::muon_step(bk, param, grad, mom, second_mom, rows, cols, lr, momentum, ns_steps, beta2, weight_decay);
}
void or_sinkhorn_step(float* param, const float* grad, float* mom, int rows, int cols, float lr, float momentum, float gamma, int steps, float tau,
                      float eps) { gnopt::sinkhorn_step(param, grad, mom, rows, cols, lr, momentum, gamma, steps, tau, eps); }
void* or_optimizer_create(void* model, float ulr, float elr, float mlr, float wd, float slr, float mult) {
  return new gnopt::Optimizer((Model*)model, ulr, elr, mlr, wd, slr, mult);
}
void or_optimizer_destroy(void* o) { delete (gnopt::Optimizer*)o; }
void or_optimizer_step(void* o) { ((gnopt::Optimizer*)o)->step(); }

// ---- building blocks of the compressed attention layers (flash.h)
void or_compressor_forward(int m, const float* hidden, const float* value, const float* weight, const float* bias, int B, int T, int d, int C, int ratio,
                           float* compressed, float* probabilities) {
  BK(m); gnor::compressor_forward(bk, hidden, value, weight, bias, B, T, d, C, ratio, compressed, probabilities);
}
void or_compressor_backward(int m, const float* hidden, const float* value, const float* weight, const float* prob, const float* compressed,
                            const float* grad_compressed, int B, int T, int d, int C, int ratio, float* grad_hidden, float* grad_value, float* grad_weight,
                            float* grad_bias) {
  BK(m); gnor::compressor_backward(bk, hidden, value, weight, prob, compressed, grad_compressed, B, T, d, C, ratio, grad_hidden, grad_value, grad_weight, grad_bias);
}
void or_compressed_attention_forward(int m, const float* q, const float* kc, const float* vc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio,
                                     float* out, float* lse) {
  BK(m); gnor::compressed_attention_forward(bk, q, kc, vc, B, Hq, Hkv, T, D, blocks, ratio, out, lse);
}
void or_compressed_attention_sparse_forward(int m, const float* q, const float* kc, const float* vc, const int32_t* selection, const int32_t* counts, int B,
                                            int Hq, int Hkv, int T, int D, int blocks, int topk, float* out, float* lse) {
  BK(m); gnor::compressed_attention_sparse_forward(bk, q, kc, vc, selection, counts, B, Hq, Hkv, T, D, blocks, topk, out, lse);
}
void or_indexer_scores_backward(const float* gs, const float* q, const float* k, const float* w, int rows, int blocks, int heads, int dim, float* gq, float* gk,
                                float* gw) {
  gnor::indexer_scores_backward(gs, q, k, w, rows, blocks, heads, dim, gq, gk, gw);
}
void or_indexer_distillation_target(const float* q, const float* kc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* target) {
  gnor::indexer_distillation_target(q, kc, B, Hq, Hkv, T, D, blocks, ratio, target);
}
void or_indexer_distillation_grad(const float* scores, const float* target, const int32_t* candidates, const int32_t* candidate_counts, int cap, int64_t rows,
                                  int blocks, int seq, int ratio, float weight, float* grad) {
  gnor::indexer_distillation_grad(scores, target, candidates, candidate_counts, cap, rows, blocks, seq, ratio, weight, grad);
}
int or_hierarchical_cap(int pool, int budget) { return gnor::hierarchical_cap(pool, budget); }
void or_select_blocks_hierarchical(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int pool, int budget, int32_t* selection,
                                   int32_t* counts, int32_t* candidates, int32_t* candidate_counts) {
  gnor::select_blocks_hierarchical(scores, tokens, blocks, offset, ratio, topk, pool, budget, selection, counts, candidates, candidate_counts);
}
void or_select_blocks_within_pool(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, const int32_t* candidates,
                                  const int32_t* candidate_counts, int cap, int32_t* selection, int32_t* counts) {
  gnor::select_blocks_within_pool(scores, tokens, blocks, offset, ratio, topk, candidates, candidate_counts, cap, selection, counts);
}
void or_compressed_attention_sparse_backward(int m, const float* q, const float* kc, const float* vc, const float* dout, const float* lse, const float* rowcorr,
                                             const int32_t* selection, const int32_t* counts, int B, int Hq, int Hkv, int T, int D, int blocks, int topk, float* dq,
                                             float* dkc, float* dvc) {
  BK(m); gnor::compressed_attention_sparse_backward(bk, q, kc, vc, dout, lse, rowcorr, selection, counts, B, Hq, Hkv, T, D, blocks, topk, dq, dkc, dvc);
}
void or_compressed_attention_forward_at(int m, const float* q, const float* kc, const float* vc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, int offset,
                                        float* out, float* lse) {
  BK(m); gnor::compressed_attention_forward_at(bk, q, kc, vc, B, Hq, Hkv, T, D, blocks, ratio, offset, out, lse);
}
void or_compressed_attention_backward(int m, const float* q, const float* kc, const float* vc, const float* dout, const float* lse, const float* rowcorr, int B,
                                      int Hq, int Hkv, int T, int D, int blocks, int ratio, float* dq, float* dkc, float* dvc) {
  BK(m); gnor::compressed_attention_backward(bk, q, kc, vc, dout, lse, rowcorr, B, Hq, Hkv, T, D, blocks, ratio, dq, dkc, dvc);
}
void or_merge_branches(const float* oa, const float* la, const float* ob, const float* lb, int64_t rows, int D, float* out, float* lse) {
  gnor::merge_branches(oa, la, ob, lb, rows, D, out, lse);
}
void or_select_blocks(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int32_t* selection, int32_t* counts) {
  gnor::select_blocks(scores, tokens, blocks, offset, ratio, topk, selection, counts);
}

}  // extern "C"
