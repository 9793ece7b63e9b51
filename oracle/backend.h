// TEST INFRASTRUCTURE (CPU oracle). Not part of the shipped library; only
// tests, the smoke check and the benchmark's CPU-baseline leg may use it.
//
// CPU restatement of the reference's numeric backend contract
// (kernels/backend.go:16-297).  Two flavours share one interface:
//
//   mode 0  "scalar": follows kernels/scalar/*.go - float64 accumulation in
//           matmul, softmax, RMSNorm and attention.  This is the parity oracle.
//   mode 1  "simd port": follows the structure of kernels/simd/*.go -
//           float32 dot products over 16 lanes (matmul.go:56-105), degree-8
//           polynomial exp (exp.go:17-88), row/column-block partition over a
//           static thread pool (internal/parallel/pool.go:54-112, here
//           OpenMP static).  This is the timed CPU baseline, kind "port".
//
// Float32 arithmetic is kept un-fused (-ffp-contract=off) because the Go
// compiler does not contract a*b+c on amd64.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <limits>

namespace gnor {

static const float kMasked = -1e30f;  // kernels/scalar/attention.go:11

struct Backend {
  int mode = 0;  // 0 scalar, 1 simd port

  // ---------------------------------------------------------------- helpers
  static inline float dot_f32_lanes(const float* a, const float* b, int n) {
    // kernels/simd/matmul.go:91-105: 16-lane FMA accumulator, horizontal sum,
    // scalar tail.
    float acc[16] = {0};
    int i = 0;
    for (; i + 16 <= n; i += 16)
      for (int l = 0; l < 16; ++l) acc[l] = std::fmaf(a[i + l], b[i + l], acc[l]);
    float total = 0;
    for (int l = 0; l < 16; ++l) total += acc[l];
    for (; i < n; ++i) total += a[i] * b[i];
    return total;
  }
  static inline float exp_poly(float x) {
    // kernels/simd/exp.go:17-48: clamp, split x*log2(e) into integer and
    // fraction, degree-8 polynomial in the fraction, scale by 2^n.
    static const float c[9] = {1.0f, 0.6931471805599453f, 0.2402265069591007f,
                               0.05550410866482158f, 0.009618129107628477f,
                               0.0013333558146428443f, 0.00015403530393381606f,
                               1.525273380405984e-05f, 1.3215486790144309e-06f};
    x = std::min(std::max(x, -87.0f), 88.0f);
    float t = x * 1.4426950408889634f;
    int n = (int)std::nearbyintf(t);
    float f = t - (float)n;
    float p = c[8];
    for (int i = 7; i >= 0; --i) p = std::fmaf(p, f, c[i]);
    uint32_t bits = (uint32_t)(n + 127) << 23;
    float scale;
    std::memcpy(&scale, &bits, 4);
    return p * scale;
  }

  // ------------------------------------------------------------ elementwise
  // kernels/scalar/elementwise.go:1-162
  void add(float* d, const float* a, const float* b, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = a[i] + b[i]; }
  void subtract(float* d, const float* a, const float* b, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = a[i] - b[i]; }
  void multiply(float* d, const float* a, const float* b, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = a[i] * b[i]; }
  void divide(float* d, const float* a, const float* b, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = a[i] / b[i]; }
  void scale(float* d, const float* s, float f, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = s[i] * f; }
  void add_scaled(float* d, const float* base, const float* s, float f, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = base[i] + f * s[i]; }
  void negate(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = -s[i]; }
  void abs(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = s[i] < 0 ? -s[i] : s[i]; }
  void square(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = s[i] * s[i]; }
  void relu_squared(float* d, const float* s, int64_t n) const {
    for (int64_t i = 0; i < n; ++i) { float v = s[i] < 0 ? 0.0f : s[i]; d[i] = v * v; }
  }
  static inline void clamp_gate(float v, float c, float& out, float& mask) {
    if (c > 0 && v >= c) { out = c; mask = 0; } else { out = v; mask = 1; }
  }
  static inline void clamp_up(float v, float c, float& out, float& mask) {
    out = v; mask = 1;
    if (c > 0) { if (v > c) { out = c; mask = 0; } else if (v < -c) { out = -c; mask = 0; } }
  }
  void swiglu(float* d, const float* gate, const float* up, float clampv, int64_t n) const {
    for (int64_t i = 0; i < n; ++i) {
      float g, gm, u, um; clamp_gate(gate[i], clampv, g, gm); clamp_up(up[i], clampv, u, um);
      float sig = (float)(1.0 / (1.0 + std::exp((double)(-g))));
      d[i] = g * sig * u;
    }
  }
  void swiglu_backward(float* gg, float* ug, const float* gate, const float* up, const float* og, float clampv, int64_t n) const {
    for (int64_t i = 0; i < n; ++i) {
      float g, gm, u, um; clamp_gate(gate[i], clampv, g, gm); clamp_up(up[i], clampv, u, um);
      float sig = (float)(1.0 / (1.0 + std::exp((double)(-g))));
      float silu = g * sig;
      float sg = sig * (1 + g * (1 - sig));
      gg[i] = og[i] * u * sg * gm;
      ug[i] = og[i] * silu * um;
    }
  }
  void exp(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = (float)std::exp((double)s[i]); }
  void sigmoid(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = (float)(1.0 / (1.0 + std::exp((double)(-s[i])))); }
  void tanh(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = (float)std::tanh((double)s[i]); }
  void rsqrt(float* d, const float* s, int64_t n) const { for (int64_t i = 0; i < n; ++i) d[i] = (float)(1.0 / std::sqrt((double)s[i])); }

  // ------------------------------------------------------------- reductions
  // kernels/scalar/reduce.go:3-36
  float sum(const float* v, int64_t n) const { float t = 0; for (int64_t i = 0; i < n; ++i) t += v[i]; return t; }
  float max(const float* v, int64_t n) const {
    if (n == 0) return 0;
    float m = v[0];
    for (int64_t i = 1; i < n; ++i) if (v[i] > m) m = v[i];
    return m;
  }
  int64_t argmax(const float* v, int64_t n) const {
    int64_t b = 0;
    for (int64_t i = 1; i < n; ++i) if (v[i] > v[b]) b = i;
    return b;
  }

  // --------------------------------------------------------- linear algebra
  // kernels/scalar/matmul.go:7-42 (mode 0), kernels/simd/matmul.go:16-105 (mode 1)
  float dot(const float* a, const float* b, int64_t n) const {
    if (mode == 1) return dot_f32_lanes(a, b, (int)n);
    double acc = 0;
    for (int64_t i = 0; i < n; ++i) acc += (double)a[i] * (double)b[i];
    return (float)acc;
  }
  void matmul(float* dst, const float* l, const float* r, int rows, int cols, int inner) const {
    if (mode == 1) {
      // rank-1 updates over the columns of each output row.
#pragma omp parallel for schedule(static)
      for (int row = 0; row < rows; ++row) {
        float* drow = dst + (int64_t)row * cols;
        std::memset(drow, 0, sizeof(float) * cols);
        for (int k = 0; k < inner; ++k) {
          float e = l[(int64_t)row * inner + k];
          const float* rrow = r + (int64_t)k * cols;
          for (int c = 0; c < cols; ++c) drow[c] = std::fmaf(rrow[c], e, drow[c]);
        }
      }
      return;
    }
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row)
      for (int c = 0; c < cols; ++c) {
        double acc = 0;
        for (int k = 0; k < inner; ++k) acc += (double)l[(int64_t)row * inner + k] * (double)r[(int64_t)k * cols + c];
        dst[(int64_t)row * cols + c] = (float)acc;
      }
  }
  void matmul_t(float* dst, const float* l, const float* r, int rows, int cols, int inner) const {
    if (mode == 1) {
      int workers = 1;
#ifdef _OPENMP
      workers = omp_workers();
#endif
      if (rows >= workers) {
#pragma omp parallel for schedule(static)
        for (int row = 0; row < rows; ++row)
          for (int c = 0; c < cols; ++c)
            dst[(int64_t)row * cols + c] = dot_f32_lanes(l + (int64_t)row * inner, r + (int64_t)c * inner, inner);
      } else {
        int blocks = (cols + 63) / 64;  // columnBlockSize = 64
#pragma omp parallel for schedule(static)
        for (int blk = 0; blk < blocks; ++blk) {
          int c0 = blk * 64, c1 = std::min(c0 + 64, cols);
          for (int row = 0; row < rows; ++row)
            for (int c = c0; c < c1; ++c)
              dst[(int64_t)row * cols + c] = dot_f32_lanes(l + (int64_t)row * inner, r + (int64_t)c * inner, inner);
        }
      }
      return;
    }
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row)
      for (int c = 0; c < cols; ++c) {
        double acc = 0;
        const float* a = l + (int64_t)row * inner;
        const float* b = r + (int64_t)c * inner;
        for (int k = 0; k < inner; ++k) acc += (double)a[k] * (double)b[k];
        dst[(int64_t)row * cols + c] = (float)acc;
      }
  }
  static int omp_workers();

  // ------------------------------------------------------------------- rows
  // kernels/scalar/norm.go:7-40
  void softmax_lastdim(float* dst, const float* src, int64_t rows, int cols) const {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
      const float* s = src + row * cols;
      float* d = dst + row * cols;
      float m = max(s, cols);
      if (mode == 1) {
        float total = 0;
        for (int c = 0; c < cols; ++c) { float e = exp_poly(s[c] - m); d[c] = e; total += e; }
        float inv = 1.0f / total;
        for (int c = 0; c < cols; ++c) d[c] *= inv;
      } else {
        double total = 0;
        for (int c = 0; c < cols; ++c) { double e = std::exp((double)(s[c] - m)); d[c] = (float)e; total += e; }
        float inv = (float)(1.0 / total);
        for (int c = 0; c < cols; ++c) d[c] = d[c] * inv;
      }
    }
  }
  void rmsnorm_lastdim(float* dst, const float* src, int64_t rows, int cols, float eps) const {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
      const float* s = src + row * cols;
      float* d = dst + row * cols;
      double ss = 0;
      for (int c = 0; c < cols; ++c) ss += (double)s[c] * (double)s[c];
      float ms = (float)(ss / (double)cols);
      float inv = (float)(1.0 / std::sqrt((double)ms + (double)eps));
      for (int c = 0; c < cols; ++c) d[c] = s[c] * inv;
    }
  }

  // -------------------------------------------------------------------- MoE
  // kernels/scalar/moe.go:8-73
  void topk_indices(int32_t* dst, const float* scores, int rows, int count, int k) const {
    if (count == 0 || k <= 0) return;
    int limit = std::min(k, count);
    std::vector<float> w(count);
    for (int row = 0; row < rows; ++row) {
      std::copy(scores + (int64_t)row * count, scores + (int64_t)(row + 1) * count, w.begin());
      for (int slot = 0; slot < limit; ++slot) {
        int best = 0;
        for (int e = 1; e < count; ++e) if (w[e] > w[best]) best = e;
        dst[(int64_t)row * k + slot] = best;
        w[best] = -std::numeric_limits<float>::infinity();
      }
    }
  }
  void moe_gate_topk(const float* logits, const float* bias, float* probs, int32_t* selected, float* weights,
                     int rows, int experts, int k) const {
    Backend sc; sc.mode = 0;
    sc.softmax_lastdim(probs, logits, rows, experts);
    std::vector<float> scores((size_t)rows * experts);
    for (size_t i = 0; i < scores.size(); ++i) scores[i] = logits[i] + bias[i % experts];
    topk_indices(selected, scores.data(), rows, experts, k);
    int limit = std::min(k, experts);
    for (int row = 0; row < rows; ++row)
      for (int slot = 0; slot < limit; ++slot)
        weights[(int64_t)row * k + slot] = probs[(int64_t)row * experts + selected[(int64_t)row * k + slot]];
  }
  void grouped_matmul_t(float* dst, const float* input, const float* weight, const int32_t* counts,
                        int experts, int cols, int inner) const {
    int64_t off = 0;
    for (int e = 0; e < experts; ++e) {
      int count = counts[e];
      const float* wb = weight + (int64_t)e * cols * inner;
      for (int row = 0; row < count; ++row) {
        const float* in = input + (off + row) * inner;
        float* out = dst + (off + row) * cols;
        for (int c = 0; c < cols; ++c) {
          const float* wr = wb + (int64_t)c * inner;
          float total = 0;
          for (int k = 0; k < inner; ++k) total += in[k] * wr[k];
          out[c] = total;
        }
      }
      off += count;
    }
  }

  // ---------------------------------------------------------------- indexer
  // kernels/scalar/indexer.go:11-61
  void indexer_scores(float* dst, const float* q, const float* key, const float* w, int rows, int blocks, int heads, int dim) const {
    for (int row = 0; row < rows; ++row)
      for (int b = 0; b < blocks; ++b) {
        float total = 0;
        for (int h = 0; h < heads; ++h) {
          const float* qh = q + ((int64_t)row * heads + h) * dim;
          const float* kh = key + ((int64_t)b * heads + h) * dim;
          float d = 0;
          for (int e = 0; e < dim; ++e) d += qh[e] * kh[e];
          if (d > 0) total += w[h] * d;
        }
        dst[(int64_t)row * blocks + b] = total;
      }
  }
  void indexer_block_max(float* dst, const float* scores, int rows, int blocks, int group) const {
    if (group < 1) group = 1;
    int groups = (blocks + group - 1) / group;
    for (int row = 0; row < rows; ++row)
      for (int g = 0; g < groups; ++g) {
        int s = g * group, e = std::min(s + group, blocks);
        float m = -std::numeric_limits<float>::infinity();
        for (int i = s; i < e; ++i) if (scores[(int64_t)row * blocks + i] > m) m = scores[(int64_t)row * blocks + i];
        dst[(int64_t)row * groups + g] = m;
      }
  }

  // -------------------------------------------------------------- attention
  // kernels/scalar/attention.go:16-245.  One (batch, head) per call.
  static inline bool masked(int qpos, int k, int window, const int32_t* seg, int seg_len, int32_t qseg) {
    bool m = k > qpos || (window >= 0 && qpos - k > window);
    if (!m && seg && k < seg_len && seg[k] != qseg) m = true;
    return m;
  }
  void scores_masked(std::vector<float>& scores, const float* q, const float* key, int ql, int kl, int hd,
                     int offset, int window, const int32_t* seg, int seg_len) const {
    scores.resize((size_t)ql * kl);
    Backend sc; sc.mode = 0;
    // Serial matmul: the caller already parallelises over (batch, head).
    for (int i = 0; i < ql; ++i)
      for (int j = 0; j < kl; ++j) {
        if (mode == 1) { scores[(size_t)i * kl + j] = dot_f32_lanes(q + (int64_t)i * hd, key + (int64_t)j * hd, hd); continue; }
        double acc = 0;
        for (int d = 0; d < hd; ++d) acc += (double)q[(int64_t)i * hd + d] * (double)key[(int64_t)j * hd + d];
        scores[(size_t)i * kl + j] = (float)acc;
      }
    int32_t qseg = 0;
    for (int i = 0; i < ql; ++i) {
      int qpos = offset + i;
      if (seg && qpos < seg_len) qseg = seg[qpos];
      for (int j = 0; j < kl; ++j)
        if (masked(qpos, j, window, seg, seg_len, qseg)) scores[(size_t)i * kl + j] = kMasked;
    }
  }
  void attention_forward(const float* q, const float* key, const float* val, int ql, int kl, int hd, int offset,
                         int window, const int32_t* seg, int seg_len, float* out, float* lse) const {
    std::vector<float> scores, probs((size_t)ql * kl);
    scores_masked(scores, q, key, ql, kl, hd, offset, window, seg, seg_len);
    for (int i = 0; i < ql; ++i) {
      const float* s = scores.data() + (size_t)i * kl;
      float* p = probs.data() + (size_t)i * kl;
      float m = max(s, kl);
      double total = 0;
      for (int j = 0; j < kl; ++j) {
        double e = (mode == 1) ? (double)exp_poly(s[j] - m) : std::exp((double)(s[j] - m));
        p[j] = (float)e; total += e;
      }
      if (lse) lse[i] = m + (float)std::log(total);
      float inv = (float)(1.0 / total);
      for (int d = 0; d < hd; ++d) {
        double acc = 0;
        for (int j = 0; j < kl; ++j) acc += (double)p[j] * (double)val[(int64_t)j * hd + d];
        out[(int64_t)i * hd + d] = (float)acc * inv;
      }
    }
  }
  void attention_forward_split(const float* q, const float* key, const float* val, int ql, int kl, int hd, int offset,
                               int window, int kstart, int kend, const int32_t* seg, int seg_len,
                               float* acc, float* mx, float* sm) const {
    if (kend > kl) kend = kl;
    int range = std::max(kend - kstart, 0);
    std::vector<float> scores(range);
    for (int i = 0; i < ql; ++i) {
      const float* qr = q + (int64_t)i * hd;
      int qpos = offset + i;
      float* ar = acc + (int64_t)i * hd;
      std::fill(ar, ar + hd, 0.0f);
      float m = -std::numeric_limits<float>::infinity();
      for (int c = 0; c < range; ++c) {
        int k = kstart + c;
        float s = dot(qr, key + (int64_t)k * hd, hd);
        bool msk = k > qpos || (window >= 0 && qpos - k > window);
        if (!msk && seg && k < seg_len && qpos < seg_len && seg[k] != seg[qpos]) msk = true;
        if (msk) s = kMasked;
        scores[c] = s;
        if (s > m) m = s;
      }
      double total = 0;
      for (int c = 0; c < range; ++c) {
        double p = std::exp((double)(scores[c] - m));
        total += p;
        const float* vr = val + (int64_t)(kstart + c) * hd;
        for (int d = 0; d < hd; ++d) ar[d] += (float)p * vr[d];
      }
      mx[i] = m;
      sm[i] = (float)total;
    }
  }
  void attention_combine(const float* const* accs, const float* const* mxs, const float* const* sms, int parts,
                         int ql, int hd, float* out, float* lse) const {
    const float ninf = -std::numeric_limits<float>::infinity();
    for (int i = 0; i < ql; ++i) {
      float gm = ninf;
      for (int p = 0; p < parts; ++p) if (mxs[p][i] > gm) gm = mxs[p][i];
      double total = 0;
      float* o = out + (int64_t)i * hd;
      std::fill(o, o + hd, 0.0f);
      for (int p = 0; p < parts; ++p) {
        float sc = 0;
        if (mxs[p][i] > ninf) sc = (float)std::exp((double)(mxs[p][i] - gm));
        total += (double)sms[p][i] * (double)sc;
        const float* a = accs[p] + (int64_t)i * hd;
        for (int d = 0; d < hd; ++d) o[d] += a[d] * sc;
      }
      if (total > 0) { float inv = (float)(1.0 / total); for (int d = 0; d < hd; ++d) o[d] *= inv; }
      if (lse) lse[i] = gm + (float)std::log(total);
    }
  }
  // Gradients ACCUMULATE into dq, dk, dv (kernels/backend.go:217-220).
  void attention_backward(const float* q, const float* key, const float* val, const float* dout, const float* lse,
                          const float* rowcorr, int ql, int kl, int hd, int offset, int window,
                          const int32_t* seg, int seg_len, float* dq, float* dk, float* dv) const {
    std::vector<float> scores, probs((size_t)ql * kl), dp((size_t)ql * kl), ds((size_t)ql * kl);
    scores_masked(scores, q, key, ql, kl, hd, offset, window, seg, seg_len);
    for (int i = 0; i < ql; ++i)
      for (int j = 0; j < kl; ++j) {
        float s = scores[(size_t)i * kl + j];
        probs[(size_t)i * kl + j] = (s <= kMasked) ? 0.0f : (float)std::exp((double)(s - lse[i]));
      }
    // dV += P^T dO   (f64 accumulate, rounded to f32 before the add)
    for (int j = 0; j < kl; ++j)
      for (int d = 0; d < hd; ++d) {
        double acc = 0;
        for (int i = 0; i < ql; ++i) acc += (double)probs[(size_t)i * kl + j] * (double)dout[(int64_t)i * hd + d];
        dv[(int64_t)j * hd + d] += (float)acc;
      }
    // dP = dO V^T
    for (int i = 0; i < ql; ++i)
      for (int j = 0; j < kl; ++j) {
        double acc = 0;
        for (int d = 0; d < hd; ++d) acc += (double)dout[(int64_t)i * hd + d] * (double)val[(int64_t)j * hd + d];
        dp[(size_t)i * kl + j] = (float)acc;
      }
    for (int i = 0; i < ql; ++i) {
      double rd = 0;
      if (rowcorr) rd = (double)rowcorr[i];
      else for (int j = 0; j < kl; ++j) rd += (double)dp[(size_t)i * kl + j] * (double)probs[(size_t)i * kl + j];
      for (int j = 0; j < kl; ++j) {
        double p = (double)probs[(size_t)i * kl + j];
        ds[(size_t)i * kl + j] = (float)(p * ((double)dp[(size_t)i * kl + j] - rd));
      }
    }
    for (int i = 0; i < ql; ++i)
      for (int d = 0; d < hd; ++d) {
        double acc = 0;
        for (int j = 0; j < kl; ++j) acc += (double)ds[(size_t)i * kl + j] * (double)key[(int64_t)j * hd + d];
        dq[(int64_t)i * hd + d] += (float)acc;
      }
    for (int j = 0; j < kl; ++j)
      for (int d = 0; d < hd; ++d) {
        double acc = 0;
        for (int i = 0; i < ql; ++i) acc += (double)ds[(size_t)i * kl + j] * (double)q[(int64_t)i * hd + d];
        dk[(int64_t)j * hd + d] += (float)acc;
      }
  }
};

}  // namespace gnor
