// TEST INFRASTRUCTURE (CPU oracle). Not part of the shipped library.
//
// CPU restatement of the dense-preset transformer of the reference: inference
// forward over a KV cache (model/transformer.go:243-342, model/attention.go:
// 235-324, model/kvcache.go:69-140,383-448), training forward that saves
// activations (model/train_transformer.go:63-142, model/train.go:55-192,
// 490-552) and the analytic backward (model/train_transformer.go:147-320,
// model/train.go:198-427,505-572, tensors/backward.go:57-116,
// model/layers/linear.go:45-104).
#pragma once
#include <map>
#include <string>
#include <memory>
#include <cstdio>
#include "backend.h"

namespace gnor {

static const float kNormEps = 1e-6f;      // model/attention.go:11
static const float kQKScale = 1.2f;       // model/attention.go:14
static const int kVeGateChannels = 12;    // model/attention.go:18
static const float kVeGateScale = 3.0f;   // model/attention.go:21
static const int kSmearChannels = 24;     // model/helpers.go:13
static const float kSoftcap = 15.0f;      // model/transformer.go:11
static const int kRotaryOvercompute = 10; // model/transformer.go:15
static const double kRotaryBase = 100000; // model/rotary.go:10

struct Config {
  int sequence_len = 0, vocab = 0, n_layer = 0, n_head = 0, n_kv_head = 0, embed_dim = 0, rotary_dims = 0;
  std::string window_pattern = "L";
  // DeepSeekMoE feed-forward (model/config.go:92-123,137-229): n_experts > 0 enables it.
  int n_experts = 0, experts_per_token = 0, expert_hidden = 0, shared_hidden = 0;
  float moe_clamp = 0.0f, moe_scale = 0.0f;
  // Absorbed multi-head latent attention (model/config.go:80-91,249-279): mla_latent > 0 enables it.
  int mla_latent = 0, mla_rotary_dims = 0;
  int head_dim() const { return embed_dim / n_head; }
  bool moe() const { return n_experts > 0; }
  bool mla() const { return mla_latent > 0; }
  int moe_top_k() const { int k = experts_per_token <= 0 ? 2 : experts_per_token; return k > n_experts ? n_experts : k; }  // model/config.go:141-149,220-225
  int moe_expert_hidden() const { return expert_hidden > 0 ? expert_hidden : embed_dim; }                                  // model/config.go:190-195
  int moe_shared_hidden() const { return shared_hidden > 0 ? shared_hidden : moe_expert_hidden(); }                       // model/config.go:199-204
  float moe_effective_clamp() const { return moe_clamp == 0.0f ? 10.0f : moe_clamp; }                                      // model/config.go:152-157
  float moe_effective_scale() const { return moe_scale == 0.0f ? 1.0f : moe_scale; }                                       // model/config.go:160-165
  int mla_rope() const {                                                                                                   // model/config.go:262-280
    if (mla_rotary_dims > 0) return mla_rotary_dims;
    int w = head_dim() / 2; if (w > 64) w = 64; if (w % 2) --w; return w;
  }
  int mla_content() const { return head_dim() - mla_rope(); }
  // model/config.go:430-444 (with MLA the rotary width is the decoupled rotary width)
  int rotary_dimension() const { return mla() ? mla_rope() : (rotary_dims <= 0 ? head_dim() : rotary_dims); }
  int padded_vocab() const { return ((vocab + 63) / 64) * 64; }                         // model/config.go:619-624
  // model/config.go:629-645 (integer division truncates toward zero, as in Go).
  std::vector<int> windows() const {
    int longw = sequence_len;
    int shortw = -((-sequence_len / 4) / 128) * 128;
    std::vector<int> w(n_layer, longw);
    for (int l = 0; l < n_layer; ++l) {
      char c = window_pattern[l % window_pattern.size()];
      w[l] = (c == 'S' || c == 's') ? shortw : longw;
    }
    w[n_layer - 1] = longw;
    return w;
  }
};

struct Param {
  std::vector<float> w, g;
  int rows = 0, cols = 0;
};

static inline bool has_value_embedding(int layer, int n_layer) { return layer % 2 == (n_layer - 1) % 2; }  // model/helpers.go:69-71

struct KVCache {
  int batch = 0, max_seq = 0, pos = 0;
  // [layer][row*Hkv+head] -> [max_seq, D]
  std::vector<std::vector<std::vector<float>>> k, v;
  std::vector<float> prev;  // [batch, d] pre-smear embedding of the last token
  bool has_prev = false;
  // MLA (model/kvcache.go:53-59,224-258): [layer][row] -> [max_seq, latent] and [max_seq, Hkv*rope]
  std::vector<std::vector<std::vector<float>>> mla_latent, mla_rope;
};

struct LayerCtx {
  std::vector<float> prev_x;      // activations before combineResidual
  std::vector<float> x_in;        // block input (after combineResidual)
  std::vector<float> h;           // norm(x_in)
  std::vector<float> q_rot, k_rot;// [B,T,H,D] post-rotary, pre-norm
  std::vector<float> q_hm, k_hm, v_hm;  // head-major post-norm q,k; final v
  std::vector<float> lse;         // [B,Hq,T]
  std::vector<float> o_hm;        // [B,Hq,T,D]
  std::vector<float> ve_sig;      // [B,T,Hkv] sigmoid gate (pre *3)
  std::vector<float> ve;          // [B,T,Hkv*D] value embedding rows
  std::vector<float> mid;         // x_in + attention output
  std::vector<float> m;           // norm(mid)
  std::vector<float> u;           // c_fc output (pre activation)
  std::vector<float> hid;         // relu(u)^2, or the shared expert's SwiGLU output when the block has routed experts
  // latent attention, training construction (model/train.go:43-45): the two shared latents
  std::vector<float> mla_ql, mla_kvl;   // [rows, latent]
  // shared SwiGLU expert (model/train.go:486-503): c_gate projection (u holds the c_fc = "up" projection)
  std::vector<float> gate;
  // routed experts (model/moe.go:83-97,171-198): router softmax, routing and the expert-major activations
  std::vector<float> probs, gw, gathered, gg, gu, gh, go;   // gw: selected weight per gathered row
  std::vector<int32_t> counts;                             // rows per expert
  std::vector<int64_t> offsets, grow;                      // first gathered row per expert; source row per gathered row
};

struct TrainCtx {
  int B = 0, T = 0;
  std::vector<int32_t> ids;
  std::vector<float> raw;          // wte rows
  std::vector<float> e_alias;      // see note in train_forward on aliasing
  std::vector<float> smear_slice;  // [B,T-1,24]
  std::vector<float> smear_sig;    // [B,T-1]
  std::vector<float> x0;           // after smear
  std::vector<LayerCtx> layers;
  std::vector<float> backout;
  std::vector<float> final_pre, final_norm;
  std::vector<float> logits;       // [B*T, V] softcapped
};

struct Model {
  Config cfg;
  Backend bk;
  std::map<std::string, Param> params;
  std::vector<float> cosv, sinv;  // [sequence_len*10, R/2]
  std::vector<int> windows;
  int D = 0, R = 0, Vp = 0, KV = 0;

  explicit Model(const Config& c, int mode) : cfg(c) {
    bk.mode = mode;
    D = cfg.head_dim(); R = cfg.rotary_dimension(); Vp = cfg.padded_vocab(); KV = cfg.n_kv_head * D;
    windows = cfg.windows();
    auto add = [&](const std::string& name, int rows, int cols) {
      Param p; p.rows = rows; p.cols = cols; p.w.assign((size_t)rows * cols, 0.0f); p.g.assign((size_t)rows * cols, 0.0f);
      params[name] = std::move(p);
    };
    int d = cfg.embed_dim;
    // model/params.go:14-74 names; shapes from model/transformer.go:49-83.
    add("transformer.wte.weight", Vp, d);
    add("lm_head.weight", Vp, d);
    for (int l = 0; l < cfg.n_layer; ++l) {
      std::string p = "transformer.h." + std::to_string(l) + ".";
      if (cfg.mla()) {
        // model/mla.go:41-60, names model/params.go:19-27
        int lat = cfg.mla_latent, rope = cfg.mla_rope(), content = cfg.mla_content();
        add(p + "attn.mla_q_down.weight", lat, d);
        add(p + "attn.mla_q_up.weight", cfg.n_head * content, lat);
        add(p + "attn.mla_q_rope.weight", cfg.n_head * rope, d);
        add(p + "attn.mla_kv_down.weight", lat, d);
        add(p + "attn.mla_k_up.weight", cfg.n_kv_head * content, lat);
        add(p + "attn.mla_v_up.weight", cfg.n_kv_head * D, lat);
        add(p + "attn.mla_k_rope.weight", cfg.n_kv_head * rope, d);
      } else {
        add(p + "attn.c_q.weight", cfg.n_head * D, d);
        add(p + "attn.c_k.weight", KV, d);
        add(p + "attn.c_v.weight", KV, d);
      }
      add(p + "attn.c_proj.weight", d, d);
      if (!cfg.mla() && has_value_embedding(l, cfg.n_layer)) {   // model/transformer.go:73
        add(p + "attn.ve_gate.weight", cfg.n_kv_head, kVeGateChannels);
        add("value_embeds." + std::to_string(l) + ".weight", Vp, KV);
      }
      if (cfg.moe()) {
        // shared expert = SwiGLU MLP (model/block.go:23-25, model/mlp.go:51-60); routed experts model/moe.go:49-70
        int sh = cfg.moe_shared_hidden(), eh = cfg.moe_expert_hidden(), E = cfg.n_experts;
        add(p + "mlp.c_fc.weight", sh, d);
        add(p + "mlp.c_gate.weight", sh, d);
        add(p + "mlp.c_proj.weight", d, sh);
        add(p + "moe.router.weight", E, d);
        add(p + "moe.router_bias", 1, E);
        add(p + "moe.experts.gate.weight", E * eh, d);
        add(p + "moe.experts.up.weight", E * eh, d);
        add(p + "moe.experts.down.weight", E * d, eh);
      } else {
        add(p + "mlp.c_fc.weight", 4 * d, d);
        add(p + "mlp.c_proj.weight", d, 4 * d);
      }
    }
    add("resid_lambdas", 1, cfg.n_layer);
    add("x0_lambdas", 1, cfg.n_layer);
    add("smear_gate.weight", 1, kSmearChannels);
    add("smear_lambda", 1, 1);
    add("backout_lambda", 1, 1);
    // model/rotary.go:16-30
    int half = R / 2, seq = cfg.sequence_len * kRotaryOvercompute;
    cosv.resize((size_t)seq * half); sinv.resize((size_t)seq * half);
    for (int p = 0; p < seq; ++p)
      for (int j = 0; j < half; ++j) {
        double inv = std::pow(kRotaryBase, -2.0 * (double)j / (double)R);
        double f = (double)p * inv;
        cosv[(size_t)p * half + j] = (float)std::cos(f);
        sinv[(size_t)p * half + j] = (float)std::sin(f);
      }
  }
  Param& P(const std::string& n) { return params.at(n); }
  std::string LP(int l, const char* s) const { return "transformer.h." + std::to_string(l) + "." + s; }
  void zero_grad() { for (auto& kv : params) std::fill(kv.second.g.begin(), kv.second.g.end(), 0.0f); }

  // ------------------------------------------------------------ primitives
  void linear(std::vector<float>& out, const std::vector<float>& in, const Param& w, int64_t rows) const {
    out.resize((size_t)rows * w.rows);
    bk.matmul_t(out.data(), in.data(), w.w.data(), (int)rows, w.rows, w.cols);
  }
  // model/layers/linear.go:45-53: dW += dY^T X ; returns dX = dY W.
  void linear_backward(std::vector<float>& dx, const std::vector<float>& x, const std::vector<float>& dy, Param& w, int64_t rows) const {
    int out = w.rows, in = w.cols;
    std::vector<float> dyT((size_t)out * rows), gw((size_t)out * in);
    for (int64_t r = 0; r < rows; ++r) for (int o = 0; o < out; ++o) dyT[(size_t)o * rows + r] = dy[(size_t)r * out + o];
    bk.matmul(gw.data(), dyT.data(), x.data(), out, in, (int)rows);
    for (size_t i = 0; i < gw.size(); ++i) w.g[i] += gw[i];
    dx.resize((size_t)rows * in);
    bk.matmul(dx.data(), dy.data(), w.w.data(), (int)rows, in, out);
  }
  // The same for one expert's [out, in] view of a packed [E*out, in] parameter (model/moe.go:60-81): x and dy are
  // the expert's `rows` gathered rows; the weight gradient accumulates into the view's slice.
  void expert_linear_backward(float* dx, const float* x, const float* dy, Param& w, int expert, int out, int in, int64_t rows) const {
    std::vector<float> dyT((size_t)out * rows), gwt((size_t)out * in);
    for (int64_t r = 0; r < rows; ++r) for (int o = 0; o < out; ++o) dyT[(size_t)o * rows + r] = dy[(size_t)r * out + o];
    bk.matmul(gwt.data(), dyT.data(), x, out, in, (int)rows);
    float* g = w.g.data() + (size_t)expert * out * in;
    for (size_t i = 0; i < gwt.size(); ++i) g[i] += gwt[i];
    bk.matmul(dx, dy, w.w.data() + (size_t)expert * out * in, (int)rows, in, out);
  }
  void norm(std::vector<float>& out, const std::vector<float>& in, int cols) const {
    out.resize(in.size());
    bk.rmsnorm_lastdim(out.data(), in.data(), (int64_t)(in.size() / cols), cols, kNormEps);
  }
  // tensors/backward.go:81-104
  static void norm_backward(std::vector<float>& dx, const std::vector<float>& x, const std::vector<float>& dy, int cols) {
    dx.resize(x.size());
    int64_t rows = (int64_t)(x.size() / cols);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      const float* xr = x.data() + r * cols; const float* gr = dy.data() + r * cols; float* o = dx.data() + r * cols;
      double ss = 0, dp = 0;
      for (int c = 0; c < cols; ++c) { ss += (double)xr[c] * (double)xr[c]; dp += (double)gr[c] * (double)xr[c]; }
      double ms = ss / (double)cols;
      double rms = std::sqrt(ms + (double)kNormEps);
      double inv = 1.0 / rms;
      double coef = dp / ((double)cols * rms * rms * rms);
      for (int c = 0; c < cols; ++c) o[c] = (float)((double)gr[c] * inv - coef * (double)xr[c]);
    }
  }
  void embedding(std::vector<float>& out, const Param& w, const int32_t* ids, int64_t n) const {
    out.resize((size_t)n * w.cols);
    for (int64_t i = 0; i < n; ++i) std::memcpy(out.data() + i * w.cols, w.w.data() + (int64_t)ids[i] * w.cols, sizeof(float) * w.cols);
  }
  // model/rotary.go:43-75 on [B,T,H,D]; sign = +1 forward, -1 backward (negated sine table, model/train.go:14-20).
  void rotary(std::vector<float>& x, int B, int T, int H, int offset, float sign) const {
    int half = R / 2, off = D - R;
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) {
      int pos = offset + t;
      const float* cw = cosv.data() + (size_t)pos * half; const float* sw = sinv.data() + (size_t)pos * half;
      for (int h = 0; h < H; ++h) {
        float* p = x.data() + (((size_t)b * T + t) * H + h) * D + off;
        for (int j = 0; j < half; ++j) {
          float a = p[j], c = p[half + j];
          float s = sign * sw[j];
          p[j] = a * cw[j] + c * s;
          p[half + j] = -a * s + c * cw[j];
        }
      }
    }
  }
  // The same rotation on heads of an explicit width (the MLA rotary heads are `R` wide: every channel rotates).
  void rotary_w(std::vector<float>& x, int B, int T, int H, int width, int offset) const {
    int half = R / 2, off = width - R;
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) {
      int pos = offset + t;
      const float* cw = cosv.data() + (size_t)pos * half; const float* sw = sinv.data() + (size_t)pos * half;
      for (int h = 0; h < H; ++h) {
        float* p = x.data() + (((size_t)b * T + t) * H + h) * width + off;
        for (int j = 0; j < half; ++j) {
          float a = p[j], c = p[half + j];
          p[j] = a * cw[j] + c * sw[j];
          p[half + j] = -a * sw[j] + c * cw[j];
        }
      }
    }
  }
  static void to_head_major(std::vector<float>& out, const std::vector<float>& in, int B, int T, int H, int D) {
    out.resize(in.size());
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) for (int h = 0; h < H; ++h)
      std::memcpy(out.data() + (((size_t)b * H + h) * T + t) * D, in.data() + (((size_t)b * T + t) * H + h) * D, sizeof(float) * D);
  }
  static void to_seq_major(std::vector<float>& out, const std::vector<float>& in, int B, int T, int H, int D) {
    out.resize(in.size());
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) for (int h = 0; h < H; ++h)
      std::memcpy(out.data() + (((size_t)b * T + t) * H + h) * D, in.data() + (((size_t)b * H + h) * T + t) * D, sizeof(float) * D);
  }
  // gate[b,t] = lambda * sigmoid(W_s . e[b,t][0:24])
  float smear_gate_value(const float* e_row, float* sig_out) const {
    const Param& ws = params.at("smear_gate.weight");
    float pre = bk.dot(e_row, ws.w.data(), kSmearChannels);
    float sig = (float)(1.0 / (1.0 + std::exp((double)(-pre))));
    if (sig_out) *sig_out = sig;
    return sig * params.at("smear_lambda").w[0];
  }
  // logits = softcap * tanh((y W_lm^T)[:, :V] / softcap)   (model/transformer.go:338-341, tensors/math.go:38-45)
  void lm_head(std::vector<float>& logits, const std::vector<float>& y, int64_t rows) const {
    const Param& w = params.at("lm_head.weight");
    int V = cfg.vocab;
    logits.resize((size_t)rows * V);
    bk.matmul_t(logits.data(), y.data(), w.w.data(), (int)rows, V, cfg.embed_dim);  // first V rows of W = trimVocab
    float inv = 1.0f / kSoftcap;
    int64_t n = rows * V;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      float s = logits[i] * inv;
      s = (float)std::tanh((double)s);
      logits[i] = s * kSoftcap;
    }
  }

  // ------------------------------------------------- inference forward
  void cache_init(KVCache& c, int batch, int max_seq) const {
    c.batch = batch; c.max_seq = max_seq; c.pos = 0; c.has_prev = false;
    c.k.assign(cfg.n_layer, {}); c.v.assign(cfg.n_layer, {});
    for (int l = 0; l < cfg.n_layer; ++l) {
      c.k[l].assign((size_t)batch * cfg.n_kv_head, std::vector<float>((size_t)max_seq * D, 0.0f));
      c.v[l].assign((size_t)batch * cfg.n_kv_head, std::vector<float>((size_t)max_seq * D, 0.0f));
    }
    if (cfg.mla()) {   // model/kvcache.go:224-237 (inference/engine.go:149-151,199-201)
      c.mla_latent.assign(cfg.n_layer, {}); c.mla_rope.assign(cfg.n_layer, {});
      for (int l = 0; l < cfg.n_layer; ++l) {
        c.mla_latent[l].assign((size_t)batch, std::vector<float>((size_t)max_seq * cfg.mla_latent, 0.0f));
        c.mla_rope[l].assign((size_t)batch, std::vector<float>((size_t)max_seq * cfg.n_kv_head * cfg.mla_rope(), 0.0f));
      }
    }
  }
  // model/kvcache.go:383-448 (dense part)
  void cache_replicate(KVCache& dst, const KVCache& src) const {
    int pos = src.pos;
    for (int l = 0; l < cfg.n_layer; ++l)
      for (int row = 0; row < dst.batch; ++row)
        for (int h = 0; h < cfg.n_kv_head; ++h) {
          std::copy(src.k[l][h].begin(), src.k[l][h].begin() + (size_t)pos * D, dst.k[l][(size_t)row * cfg.n_kv_head + h].begin());
          std::copy(src.v[l][h].begin(), src.v[l][h].begin() + (size_t)pos * D, dst.v[l][(size_t)row * cfg.n_kv_head + h].begin());
        }
    if (cfg.mla()) {   // model/kvcache.go:427-436
      size_t lw = (size_t)cfg.mla_latent, rw = (size_t)cfg.n_kv_head * cfg.mla_rope();
      for (int l = 0; l < cfg.n_layer; ++l)
        for (int row = 0; row < dst.batch; ++row) {
          std::copy(src.mla_latent[l][0].begin(), src.mla_latent[l][0].begin() + (size_t)pos * lw, dst.mla_latent[l][row].begin());
          std::copy(src.mla_rope[l][0].begin(), src.mla_rope[l][0].begin() + (size_t)pos * rw, dst.mla_rope[l][row].begin());
        }
    }
    dst.pos = pos;
    if (src.has_prev) {
      int d = cfg.embed_dim;
      dst.prev.resize((size_t)dst.batch * d);
      for (int row = 0; row < dst.batch; ++row) std::copy(src.prev.begin(), src.prev.begin() + d, dst.prev.begin() + (size_t)row * d);
      dst.has_prev = true;
    }
  }

  // Absorbed MLA attention of one layer (model/mla.go:185-279).  h = norm(x) [B,T,d]; returns the head
  // outputs [B,T,Hq*D] before c_proj.  The absorption sums are float32, in the reference's loop order.
  void mla_inference(std::vector<float>& out, const std::vector<float>& h, int B, int T, int offset, KVCache& cache, int l) const {
    const int Hq = cfg.n_head, Hkv = cfg.n_kv_head, lat = cfg.mla_latent, rope = cfg.mla_rope(), content = cfg.mla_content();
    const int ratio = Hq / Hkv, hd = lat + rope, vd = D;
    const int64_t rows = (int64_t)B * T;
    std::vector<float> ql, qc, qr, kvl, kr;
    linear(ql, h, params.at(LP(l, "attn.mla_q_down.weight")), rows);
    linear(qc, ql, params.at(LP(l, "attn.mla_q_up.weight")), rows);      // [B,T,Hq,content]
    linear(qr, h, params.at(LP(l, "attn.mla_q_rope.weight")), rows);     // [B,T,Hq,rope]
    rotary_w(qr, B, T, Hq, rope, offset);
    linear(kvl, h, params.at(LP(l, "attn.mla_kv_down.weight")), rows);   // [B,T,lat]
    linear(kr, h, params.at(LP(l, "attn.mla_k_rope.weight")), rows);     // [B,T,Hkv,rope]
    rotary_w(kr, B, T, Hkv, rope, offset);
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) {
      std::copy(kvl.begin() + ((size_t)b * T + t) * lat, kvl.begin() + ((size_t)b * T + t + 1) * lat, cache.mla_latent[l][b].begin() + (size_t)(offset + t) * lat);
      std::copy(kr.begin() + ((size_t)b * T + t) * Hkv * rope, kr.begin() + ((size_t)b * T + t + 1) * Hkv * rope,
                cache.mla_rope[l][b].begin() + (size_t)(offset + t) * Hkv * rope);
    }
    const int count = offset + T;
    const float* key_up = params.at(LP(l, "attn.mla_k_up.weight")).w.data();
    const float* value_up = params.at(LP(l, "attn.mla_v_up.weight")).w.data();
    out.assign((size_t)rows * Hq * vd, 0.0f);
#pragma omp parallel for schedule(static)
    for (int idx = 0; idx < B * Hq; ++idx) {
      const int b = idx / Hq, hq = idx % Hq, hk = hq / ratio;
      std::vector<float> q((size_t)T * hd), key((size_t)count * hd), val((size_t)count * hd, 0.0f), ao((size_t)T * hd);
      for (int t = 0; t < T; ++t) {
        const float* qcp = qc.data() + (((size_t)b * T + t) * Hq + hq) * content;
        for (int r = 0; r < lat; ++r) {
          float sum = 0.0f;
          for (int c = 0; c < content; ++c) sum += qcp[c] * key_up[((size_t)hk * content + c) * lat + r];
          q[(size_t)t * hd + r] = sum;
        }
        std::copy(qr.begin() + (((size_t)b * T + t) * Hq + hq) * rope, qr.begin() + (((size_t)b * T + t) * Hq + hq + 1) * rope, q.begin() + (size_t)t * hd + lat);
      }
      const float* lc = cache.mla_latent[l][b].data(); const float* rc = cache.mla_rope[l][b].data();
      for (int j = 0; j < count; ++j) {
        std::copy(lc + (size_t)j * lat, lc + (size_t)(j + 1) * lat, key.begin() + (size_t)j * hd);
        std::copy(rc + ((size_t)j * Hkv + hk) * rope, rc + ((size_t)j * Hkv + hk + 1) * rope, key.begin() + (size_t)j * hd + lat);
        std::copy(lc + (size_t)j * lat, lc + (size_t)(j + 1) * lat, val.begin() + (size_t)j * hd);
      }
      bk.attention_forward(q.data(), key.data(), val.data(), T, count, hd, offset, windows[l], nullptr, 0, ao.data(), nullptr);
      for (int t = 0; t < T; ++t) {
        float* op = out.data() + (((size_t)b * T + t) * Hq + hq) * vd;
        for (int dd = 0; dd < vd; ++dd) {
          float sum = 0.0f;
          for (int r = 0; r < lat; ++r) sum += ao[(size_t)t * hd + r] * value_up[((size_t)hk * vd + dd) * lat + r];
          op[dd] = sum;
        }
      }
    }
  }
  // The un-absorbed construction the training path uses (model/mla.go:106-124, model/train.go:59-86): per-head
  // content|rotary queries and keys, values up-projected from the latent, no QK norm and no 1.2 scale.
  void mla_unabsorbed(std::vector<float>& out, const std::vector<float>& h, int B, int T, int l) const {
    const int Hq = cfg.n_head, Hkv = cfg.n_kv_head, rope = cfg.mla_rope(), content = cfg.mla_content(), ratio = Hq / Hkv;
    const int64_t rows = (int64_t)B * T;
    std::vector<float> ql, qc, qr, kvl, kc, kr, v;
    linear(ql, h, params.at(LP(l, "attn.mla_q_down.weight")), rows);
    linear(qc, ql, params.at(LP(l, "attn.mla_q_up.weight")), rows);
    linear(qr, h, params.at(LP(l, "attn.mla_q_rope.weight")), rows);
    linear(kvl, h, params.at(LP(l, "attn.mla_kv_down.weight")), rows);
    linear(kc, kvl, params.at(LP(l, "attn.mla_k_up.weight")), rows);
    linear(kr, h, params.at(LP(l, "attn.mla_k_rope.weight")), rows);
    linear(v, kvl, params.at(LP(l, "attn.mla_v_up.weight")), rows);
    auto concat = [&](std::vector<float>& dst, const std::vector<float>& c, const std::vector<float>& r, int H) {
      dst.resize((size_t)rows * H * D);
      for (int64_t i = 0; i < rows * H; ++i) {
        std::copy(c.begin() + i * content, c.begin() + (i + 1) * content, dst.begin() + i * D);
        std::copy(r.begin() + i * rope, r.begin() + (i + 1) * rope, dst.begin() + i * D + content);
      }
    };
    std::vector<float> q, k;
    concat(q, qc, qr, Hq); concat(k, kc, kr, Hkv);
    rotary(q, B, T, Hq, 0, 1.0f); rotary(k, B, T, Hkv, 0, 1.0f);
    std::vector<float> qh, kh, vh, oh((size_t)rows * Hq * D);
    to_head_major(qh, q, B, T, Hq, D); to_head_major(kh, k, B, T, Hkv, D); to_head_major(vh, v, B, T, Hkv, D);
#pragma omp parallel for schedule(static)
    for (int idx = 0; idx < B * Hq; ++idx) {
      int b = idx / Hq, hq = idx % Hq, hk = hq / ratio;
      size_t slot = (size_t)b * Hkv + hk;
      bk.attention_forward(qh.data() + (size_t)idx * T * D, kh.data() + slot * T * D, vh.data() + slot * T * D, T, T, D, 0, windows[l], nullptr, 0,
                           oh.data() + (size_t)idx * T * D, nullptr);
    }
    to_seq_major(out, oh, B, T, Hq, D);
  }
  // Routed experts (model/moe.go:118-169): returns the routed contribution [rows, d]; `sel_out` (nullable)
  // receives the selected expert ids [rows, k].
  void moe_forward(std::vector<float>& out, const std::vector<float>& flat, int64_t rows, int l, std::vector<int32_t>* sel_out) const {
    const int d = cfg.embed_dim, E = cfg.n_experts, K = cfg.moe_top_k(), eh = cfg.moe_expert_hidden();
    std::vector<float> logits, probs((size_t)rows * E), selw((size_t)rows * K);
    std::vector<int32_t> sel((size_t)rows * K);
    linear(logits, flat, params.at(LP(l, "moe.router.weight")), rows);
    bk.moe_gate_topk(logits.data(), params.at(LP(l, "moe.router_bias")).w.data(), probs.data(), sel.data(), selw.data(), (int)rows, E, K);
    if (sel_out) *sel_out = sel;
    const int64_t total = rows * K;
    std::vector<int32_t> counts(E, 0);
    for (int64_t i = 0; i < total; ++i) counts[sel[i]]++;
    std::vector<int64_t> offsets(E, 0), fill(E, 0);
    { int64_t cur = 0; for (int e = 0; e < E; ++e) { offsets[e] = cur; cur += counts[e]; } }
    std::vector<float> gathered((size_t)total * d), gw((size_t)total);
    std::vector<int64_t> grow((size_t)total);
    for (int64_t r = 0; r < rows; ++r) for (int s = 0; s < K; ++s) {
      int e = sel[r * K + s];
      int64_t pos = offsets[e] + fill[e]++;
      std::copy(flat.begin() + r * d, flat.begin() + (r + 1) * d, gathered.begin() + pos * d);
      grow[pos] = r; gw[pos] = selw[r * K + s];
    }
    std::vector<float> gg((size_t)total * eh), gu((size_t)total * eh), gh((size_t)total * eh), go((size_t)total * d);
    bk.grouped_matmul_t(gg.data(), gathered.data(), params.at(LP(l, "moe.experts.gate.weight")).w.data(), counts.data(), E, eh, d);
    bk.grouped_matmul_t(gu.data(), gathered.data(), params.at(LP(l, "moe.experts.up.weight")).w.data(), counts.data(), E, eh, d);
    bk.swiglu(gh.data(), gg.data(), gu.data(), cfg.moe_effective_clamp(), (int64_t)gh.size());
    bk.grouped_matmul_t(go.data(), gh.data(), params.at(LP(l, "moe.experts.down.weight")).w.data(), counts.data(), E, d, eh);
    out.assign((size_t)rows * d, 0.0f);
    const float scale = cfg.moe_effective_scale();
    for (int64_t i = 0; i < total; ++i) {
      float w = gw[i] * scale;
      float* o = out.data() + grow[i] * d; const float* g = go.data() + i * d;
      for (int c = 0; c < d; ++c) o[c] += w * g[c];
    }
  }

  // Returns logits [B,T,V].  cache may be null (then T must be > 1).  `unabsorbed` (MLA models, cache == null)
  // evaluates attention in the training construction instead of the absorbed one.
  void forward(std::vector<float>& logits, const int32_t* ids, int B, int T, KVCache* cache, bool unabsorbed = false) const {
    int d = cfg.embed_dim, Hq = cfg.n_head, Hkv = cfg.n_kv_head, L = cfg.n_layer;
    int64_t rows = (int64_t)B * T;
    KVCache scratch;   // model/transformer.go:248-253: a cache-less MLA forward gets a scratch latent cache
    if (!cache && cfg.mla() && !unabsorbed) { cache_init(scratch, B, T); cache = &scratch; }
    std::vector<float> raw, x;
    embedding(raw, params.at("transformer.wte.weight"), ids, rows);
    norm(x, raw, d);
    int offset = cache ? cache->pos : 0;
    // ---- smear (model/transformer.go:266-301)
    std::vector<float> prev_in;
    bool had_prev = false;
    if (cache) {
      had_prev = cache->has_prev;
      if (had_prev) prev_in = cache->prev;
      cache->prev.resize((size_t)B * d);
      for (int b = 0; b < B; ++b) std::copy(x.begin() + ((size_t)b * T + T - 1) * d, x.begin() + ((size_t)b * T + T) * d, cache->prev.begin() + (size_t)b * d);
      cache->has_prev = true;
    }
    if (T > 1) {
      std::vector<float> gates((size_t)B * T, 0.0f);  // gate for t>=1 ; t=0 seed gate when had_prev
      for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t)
        if (t >= 1 || had_prev) gates[(size_t)b * T + t] = smear_gate_value(x.data() + ((size_t)b * T + t) * d, nullptr);
      for (int b = 0; b < B; ++b) {
        for (int t = T - 1; t >= 1; --t) {
          float g = gates[(size_t)b * T + t];
          float* cur = x.data() + ((size_t)b * T + t) * d; const float* pv = x.data() + ((size_t)b * T + t - 1) * d;
          for (int c = 0; c < d; ++c) cur[c] += g * pv[c];
        }
        if (had_prev) {
          float g = gates[(size_t)b * T];
          float* cur = x.data() + (size_t)b * T * d; const float* pv = prev_in.data() + (size_t)b * d;
          for (int c = 0; c < d; ++c) cur[c] += g * pv[c];
        }
      }
    } else if (cache && had_prev) {
      for (int b = 0; b < B; ++b) {
        float g = smear_gate_value(x.data() + (size_t)b * d, nullptr);
        float* cur = x.data() + (size_t)b * d; const float* pv = prev_in.data() + (size_t)b * d;
        for (int c = 0; c < d; ++c) cur[c] += g * pv[c];
      }
    }
    std::vector<float> x0 = x, backout;
    const Param& rl = params.at("resid_lambdas"); const Param& xl = params.at("x0_lambdas");
    for (int l = 0; l < L; ++l) {
      for (size_t i = 0; i < x.size(); ++i) x[i] = rl.w[l] * x[i] + xl.w[l] * x0[i];
      // ---- attention (model/attention.go:235-324)
      std::vector<float> h, q, k, v;
      norm(h, x, d);
      if (cfg.mla()) {
        std::vector<float> heads, ao;
        if (unabsorbed) mla_unabsorbed(heads, h, B, T, l); else mla_inference(heads, h, B, T, offset, *cache, l);
        linear(ao, heads, params.at(LP(l, "attn.c_proj.weight")), rows);
        for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + ao[i];
      } else {
      linear(q, h, params.at(LP(l, "attn.c_q.weight")), rows);
      linear(k, h, params.at(LP(l, "attn.c_k.weight")), rows);
      linear(v, h, params.at(LP(l, "attn.c_v.weight")), rows);
      if (has_value_embedding(l, L)) {
        std::vector<float> ve;
        embedding(ve, params.at("value_embeds." + std::to_string(l) + ".weight"), ids, rows);
        const Param& wg = params.at(LP(l, "attn.ve_gate.weight"));
        for (int64_t r = 0; r < rows; ++r) for (int hh = 0; hh < Hkv; ++hh) {
          float pre = bk.dot(h.data() + r * d, wg.w.data() + (size_t)hh * kVeGateChannels, kVeGateChannels);
          float gate = (float)(1.0 / (1.0 + std::exp((double)(-pre)))) * kVeGateScale;
          float* vr = v.data() + (r * Hkv + hh) * D; const float* er = ve.data() + (r * Hkv + hh) * D;
          for (int c = 0; c < D; ++c) vr[c] += gate * er[c];
        }
      }
      rotary(q, B, T, Hq, offset, 1.0f);
      rotary(k, B, T, Hkv, offset, 1.0f);
      std::vector<float> qn, kn;
      norm(qn, q, D); norm(kn, k, D);
      for (auto& e : qn) e *= kQKScale;
      for (auto& e : kn) e *= kQKScale;
      std::vector<float> qh, kh, vh, oh((size_t)rows * Hq * D);
      to_head_major(qh, qn, B, T, Hq, D); to_head_major(kh, kn, B, T, Hkv, D); to_head_major(vh, v, B, T, Hkv, D);
      int klen = T;
      if (cache) {
        for (int b = 0; b < B; ++b) for (int hh = 0; hh < Hkv; ++hh) {
          size_t slot = (size_t)b * Hkv + hh;
          std::copy(kh.begin() + slot * T * D, kh.begin() + (slot + 1) * T * D, cache->k[l][slot].begin() + (size_t)offset * D);
          std::copy(vh.begin() + slot * T * D, vh.begin() + (slot + 1) * T * D, cache->v[l][slot].begin() + (size_t)offset * D);
        }
        klen = offset + T;
      }
      int ratio = Hq / Hkv;
#pragma omp parallel for schedule(static)
      for (int idx = 0; idx < B * Hq; ++idx) {
        int b = idx / Hq, hq = idx % Hq, hk = hq / ratio;
        size_t slot = (size_t)b * Hkv + hk;
        const float* kp = cache ? cache->k[l][slot].data() : kh.data() + slot * T * D;
        const float* vp = cache ? cache->v[l][slot].data() : vh.data() + slot * T * D;
        bk.attention_forward(qh.data() + (size_t)idx * T * D, kp, vp, T, klen, D, offset, windows[l], nullptr, 0,
                             oh.data() + (size_t)idx * T * D, nullptr);
      }
      std::vector<float> os, ao;
      to_seq_major(os, oh, B, T, Hq, D);
      linear(ao, os, params.at(LP(l, "attn.c_proj.weight")), rows);
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + ao[i];
      }
      // ---- MLP (model/mlp.go:62-76); with MoE: shared SwiGLU expert + routed experts (model/block.go:39-46)
      std::vector<float> m, u, fo;
      norm(m, x, d);
      linear(u, m, params.at(LP(l, "mlp.c_fc.weight")), rows);
      if (cfg.moe()) {
        std::vector<float> gate, hid(u.size()), routed;
        linear(gate, m, params.at(LP(l, "mlp.c_gate.weight")), rows);
        bk.swiglu(hid.data(), gate.data(), u.data(), cfg.moe_effective_clamp(), (int64_t)hid.size());
        linear(fo, hid, params.at(LP(l, "mlp.c_proj.weight")), rows);
        moe_forward(routed, m, rows, l, nullptr);
        for (size_t i = 0; i < fo.size(); ++i) fo[i] = fo[i] + routed[i];
      } else {
        bk.relu_squared(u.data(), u.data(), (int64_t)u.size());
        linear(fo, u, params.at(LP(l, "mlp.c_proj.weight")), rows);
      }
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + fo[i];
      if (l == L / 2) backout = x;
    }
    if (cache && cache != &scratch) cache->pos += T;
    if (!backout.empty()) {
      float lam = -params.at("backout_lambda").w[0];
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + lam * backout[i];
    }
    std::vector<float> y;
    norm(y, x, d);
    lm_head(logits, y, rows);
  }

  // Routed experts of the training pass (model/moe.go:118-198): like moe_forward, keeping the routing and every
  // expert-major activation for the backward.
  void moe_train_forward(LayerCtx& c, std::vector<float>& out, int64_t rows, int l) const {
    const int d = cfg.embed_dim, E = cfg.n_experts, K = cfg.moe_top_k(), eh = cfg.moe_expert_hidden();
    std::vector<float> logits, selw((size_t)rows * K);
    std::vector<int32_t> sel((size_t)rows * K);
    c.probs.assign((size_t)rows * E, 0.0f);
    linear(logits, c.m, params.at(LP(l, "moe.router.weight")), rows);
    bk.moe_gate_topk(logits.data(), params.at(LP(l, "moe.router_bias")).w.data(), c.probs.data(), sel.data(), selw.data(), (int)rows, E, K);
    const int64_t total = rows * K;
    c.counts.assign(E, 0);
    for (int64_t i = 0; i < total; ++i) c.counts[sel[i]]++;
    c.offsets.assign(E, 0);
    std::vector<int64_t> fill(E, 0);
    { int64_t cur = 0; for (int e = 0; e < E; ++e) { c.offsets[e] = cur; cur += c.counts[e]; } }
    c.gathered.assign((size_t)total * d, 0.0f); c.gw.assign((size_t)total, 0.0f); c.grow.assign((size_t)total, 0);
    for (int64_t r = 0; r < rows; ++r) for (int s = 0; s < K; ++s) {
      int e = sel[r * K + s];
      int64_t pos = c.offsets[e] + fill[e]++;
      std::copy(c.m.begin() + r * d, c.m.begin() + (r + 1) * d, c.gathered.begin() + pos * d);
      c.grow[pos] = r; c.gw[pos] = selw[r * K + s];
    }
    c.gg.assign((size_t)total * eh, 0.0f); c.gu.assign((size_t)total * eh, 0.0f); c.gh.assign((size_t)total * eh, 0.0f); c.go.assign((size_t)total * d, 0.0f);
    bk.grouped_matmul_t(c.gg.data(), c.gathered.data(), params.at(LP(l, "moe.experts.gate.weight")).w.data(), c.counts.data(), E, eh, d);
    bk.grouped_matmul_t(c.gu.data(), c.gathered.data(), params.at(LP(l, "moe.experts.up.weight")).w.data(), c.counts.data(), E, eh, d);
    bk.swiglu(c.gh.data(), c.gg.data(), c.gu.data(), cfg.moe_effective_clamp(), (int64_t)c.gh.size());
    bk.grouped_matmul_t(c.go.data(), c.gh.data(), params.at(LP(l, "moe.experts.down.weight")).w.data(), c.counts.data(), E, d, eh);
    out.assign((size_t)rows * d, 0.0f);
    const float scale = cfg.moe_effective_scale();
    for (int64_t i = 0; i < total; ++i) {
      float w = c.gw[i] * scale;
      float* o = out.data() + c.grow[i] * d; const float* g = c.go.data() + i * d;
      for (int cc = 0; cc < d; ++cc) o[cc] += w * g[cc];
    }
  }
  // model/moe.go:203-267 with the sequence-level balance loss of :276-326 (weight 1e-4, model/moe.go:47-58; its
  // gradient enters through the router softmax).  dout: gradient of the block output; returns the gradient at m.
  void moe_train_backward(LayerCtx& c, std::vector<float>& dm, const std::vector<float>& dout, int64_t rows, int seq_len, int l) {
    const int d = cfg.embed_dim, E = cfg.n_experts, K = cfg.moe_top_k(), eh = cfg.moe_expert_hidden();
    const float scale = cfg.moe_effective_scale(), clampv = cfg.moe_effective_clamp();
    dm.assign((size_t)rows * d, 0.0f);
    std::vector<double> gprobs((size_t)rows * E, 0.0);
    Param& wg = P(LP(l, "moe.experts.gate.weight")); Param& wu = P(LP(l, "moe.experts.up.weight")); Param& wd = P(LP(l, "moe.experts.down.weight"));
    for (int e = 0; e < E; ++e) {
      const int64_t cnt = c.counts[e], off = c.offsets[e];
      if (cnt == 0) continue;
      std::vector<float> dgo((size_t)cnt * d);
      for (int64_t i = 0; i < cnt; ++i) {
        const int64_t row = c.grow[off + i];
        const float w = c.gw[off + i] * scale;
        double dot = 0;
        for (int cc = 0; cc < d; ++cc) {
          const float g = dout[(size_t)row * d + cc];
          dgo[(size_t)i * d + cc] = g * w;
          dot += (double)g * (double)c.go[(size_t)(off + i) * d + cc];
        }
        gprobs[(size_t)row * E + e] += dot * (double)scale;
      }
      std::vector<float> dgh((size_t)cnt * eh), dgg((size_t)cnt * eh), dgu((size_t)cnt * eh), dfg((size_t)cnt * d), dfu((size_t)cnt * d);
      expert_linear_backward(dgh.data(), c.gh.data() + (size_t)off * eh, dgo.data(), wd, e, d, eh, cnt);
      bk.swiglu_backward(dgg.data(), dgu.data(), c.gg.data() + (size_t)off * eh, c.gu.data() + (size_t)off * eh, dgh.data(), clampv, (int64_t)cnt * eh);
      expert_linear_backward(dfg.data(), c.gathered.data() + (size_t)off * d, dgg.data(), wg, e, eh, d, cnt);
      expert_linear_backward(dfu.data(), c.gathered.data() + (size_t)off * d, dgu.data(), wu, e, eh, d, cnt);
      for (int64_t i = 0; i < cnt; ++i) {
        float* o = dm.data() + (size_t)c.grow[off + i] * d;
        for (int cc = 0; cc < d; ++cc) o[cc] += dfg[(size_t)i * d + cc] + dfu[(size_t)i * d + cc];
      }
    }
    // sequence-level balance loss (model/moe.go:276-326): dL/dp[t,e] = weight / (S*T) * E/(K*T) * count[s(t), e]
    const float balance_weight = 1e-4f;   // defaultMoEBalanceWeight (model/config.go:133-135,176-186)
    if (balance_weight > 0 && seq_len > 0 && rows > 0 && rows % seq_len == 0) {
      const int64_t sequences = rows / seq_len;
      std::vector<double> cnts((size_t)sequences * E, 0.0);
      for (int e = 0; e < E; ++e) for (int64_t i = 0; i < c.counts[e]; ++i) cnts[(size_t)(c.grow[c.offsets[e] + i] / seq_len) * E + e] += 1.0;
      const double selection_scale = (double)E / ((double)K * (double)seq_len);
      const double coefficient = (double)balance_weight / ((double)sequences * (double)seq_len);
      for (int64_t r = 0; r < rows; ++r) for (int e = 0; e < E; ++e)
        gprobs[(size_t)r * E + e] += coefficient * selection_scale * cnts[(size_t)(r / seq_len) * E + e];
    }
    // router softmax backward and the router's own Linear
    std::vector<float> glog((size_t)rows * E);
    for (int64_t r = 0; r < rows; ++r) {
      double dot = 0;
      for (int e = 0; e < E; ++e) dot += (double)c.probs[(size_t)r * E + e] * gprobs[(size_t)r * E + e];
      for (int e = 0; e < E; ++e) glog[(size_t)r * E + e] = (float)((double)c.probs[(size_t)r * E + e] * (gprobs[(size_t)r * E + e] - dot));
    }
    std::vector<float> gri;
    linear_backward(gri, c.m, glog, P(LP(l, "moe.router.weight")), rows);
    for (size_t i = 0; i < dm.size(); ++i) dm[i] = dm[i] + gri[i];
  }

  // ------------------------------------------------- training forward
  void train_forward(TrainCtx& ctx, const int32_t* ids, int B, int T) const {
    int d = cfg.embed_dim, Hq = cfg.n_head, Hkv = cfg.n_kv_head, L = cfg.n_layer;
    int64_t rows = (int64_t)B * T;
    ctx.B = B; ctx.T = T; ctx.ids.assign(ids, ids + rows);
    embedding(ctx.raw, params.at("transformer.wte.weight"), ids, rows);
    std::vector<float> x;
    norm(x, ctx.raw, d);
    // smear gate input: channels 0..23 of rows 1..T-1 (pre-smear)
    ctx.smear_slice.resize((size_t)B * (T - 1) * kSmearChannels);
    ctx.smear_sig.resize((size_t)B * (T - 1));
    std::vector<float> gates((size_t)B * (T - 1));
    for (int b = 0; b < B; ++b) for (int t = 1; t < T; ++t) {
      const float* er = x.data() + ((size_t)b * T + t) * d;
      size_t gi = (size_t)b * (T - 1) + (t - 1);
      std::copy(er, er + kSmearChannels, ctx.smear_slice.begin() + gi * kSmearChannels);
      gates[gi] = smear_gate_value(er, &ctx.smear_sig[gi]);
    }
    for (int b = 0; b < B; ++b) for (int t = T - 1; t >= 1; --t) {
      float g = gates[(size_t)b * (T - 1) + (t - 1)];
      float* cur = x.data() + ((size_t)b * T + t) * d; const float* pv = x.data() + ((size_t)b * T + t - 1) * d;
      for (int c = 0; c < d; ++c) cur[c] += g * pv[c];
    }
    // The reference stores `embeddedNormalized` as the same tensor object that
    // smearAdd then modifies in place (model/train_transformer.go:75-83), so
    // what smearBackward later reads as the "embedded" activations is the
    // POST-smear tensor.  The oracle keeps that behaviour.
    ctx.e_alias = x;
    ctx.x0 = x;
    ctx.layers.assign(L, LayerCtx());
    const Param& rl = params.at("resid_lambdas"); const Param& xl = params.at("x0_lambdas");
    int ratio = Hq / Hkv;
    for (int l = 0; l < L; ++l) {
      LayerCtx& c = ctx.layers[l];
      c.prev_x = x;
      for (size_t i = 0; i < x.size(); ++i) x[i] = rl.w[l] * x[i] + xl.w[l] * ctx.x0[i];
      c.x_in = x;
      norm(c.h, x, d);
      std::vector<float> q, k, v;
      if (cfg.mla()) {
        // model/mla.go:106-124: per-head [content | rotary] queries and keys, values up-projected from the latent;
        // no QK norm and no 1.2 scale (model/train.go:82-85); value embeddings are off (model/transformer.go:73)
        const int rope = cfg.mla_rope(), content = cfg.mla_content();
        std::vector<float> qc, qr, kc, kr;
        linear(c.mla_ql, c.h, params.at(LP(l, "attn.mla_q_down.weight")), rows);
        linear(qc, c.mla_ql, params.at(LP(l, "attn.mla_q_up.weight")), rows);
        linear(qr, c.h, params.at(LP(l, "attn.mla_q_rope.weight")), rows);
        linear(c.mla_kvl, c.h, params.at(LP(l, "attn.mla_kv_down.weight")), rows);
        linear(kc, c.mla_kvl, params.at(LP(l, "attn.mla_k_up.weight")), rows);
        linear(kr, c.h, params.at(LP(l, "attn.mla_k_rope.weight")), rows);
        linear(v, c.mla_kvl, params.at(LP(l, "attn.mla_v_up.weight")), rows);
        auto concat = [&](std::vector<float>& dst, const std::vector<float>& cc, const std::vector<float>& rr, int H) {
          dst.resize((size_t)rows * H * D);
          for (int64_t i = 0; i < rows * H; ++i) {
            std::copy(cc.begin() + i * content, cc.begin() + (i + 1) * content, dst.begin() + i * D);
            std::copy(rr.begin() + i * rope, rr.begin() + (i + 1) * rope, dst.begin() + i * D + content);
          }
        };
        concat(q, qc, qr, Hq); concat(k, kc, kr, Hkv);
        rotary(q, B, T, Hq, 0, 1.0f);
        rotary(k, B, T, Hkv, 0, 1.0f);
        to_head_major(c.q_hm, q, B, T, Hq, D); to_head_major(c.k_hm, k, B, T, Hkv, D); to_head_major(c.v_hm, v, B, T, Hkv, D);
      } else {
      linear(q, c.h, params.at(LP(l, "attn.c_q.weight")), rows);
      linear(k, c.h, params.at(LP(l, "attn.c_k.weight")), rows);
      linear(v, c.h, params.at(LP(l, "attn.c_v.weight")), rows);
      if (has_value_embedding(l, L)) {
        embedding(c.ve, params.at("value_embeds." + std::to_string(l) + ".weight"), ids, rows);
        const Param& wg = params.at(LP(l, "attn.ve_gate.weight"));
        c.ve_sig.resize((size_t)rows * Hkv);
        for (int64_t r = 0; r < rows; ++r) for (int hh = 0; hh < Hkv; ++hh) {
          float pre = bk.dot(c.h.data() + r * d, wg.w.data() + (size_t)hh * kVeGateChannels, kVeGateChannels);
          float sig = (float)(1.0 / (1.0 + std::exp((double)(-pre))));
          c.ve_sig[r * Hkv + hh] = sig;
          float gate = sig * kVeGateScale;
          float* vr = v.data() + (r * Hkv + hh) * D; const float* er = c.ve.data() + (r * Hkv + hh) * D;
          for (int cc = 0; cc < D; ++cc) vr[cc] += gate * er[cc];
        }
      }
      rotary(q, B, T, Hq, 0, 1.0f);
      rotary(k, B, T, Hkv, 0, 1.0f);
      c.q_rot = q; c.k_rot = k;
      std::vector<float> qn, kn;
      norm(qn, q, D); norm(kn, k, D);
      for (auto& e : qn) e *= kQKScale;
      for (auto& e : kn) e *= kQKScale;
      to_head_major(c.q_hm, qn, B, T, Hq, D); to_head_major(c.k_hm, kn, B, T, Hkv, D); to_head_major(c.v_hm, v, B, T, Hkv, D);
      }
      c.o_hm.assign((size_t)rows * Hq * D, 0.0f);
      c.lse.assign((size_t)B * Hq * T, 0.0f);
#pragma omp parallel for schedule(static)
      for (int idx = 0; idx < B * Hq; ++idx) {
        int b = idx / Hq, hq = idx % Hq, hk = hq / ratio;
        size_t slot = (size_t)b * Hkv + hk;
        bk.attention_forward(c.q_hm.data() + (size_t)idx * T * D, c.k_hm.data() + slot * T * D, c.v_hm.data() + slot * T * D,
                             T, T, D, 0, windows[l], nullptr, 0, c.o_hm.data() + (size_t)idx * T * D, c.lse.data() + (size_t)idx * T);
      }
      std::vector<float> os, ao;
      to_seq_major(os, c.o_hm, B, T, Hq, D);
      linear(ao, os, params.at(LP(l, "attn.c_proj.weight")), rows);
      c.mid.resize(x.size());
      for (size_t i = 0; i < x.size(); ++i) c.mid[i] = x[i] + ao[i];
      norm(c.m, c.mid, d);
      linear(c.u, c.m, params.at(LP(l, "mlp.c_fc.weight")), rows);
      c.hid.resize(c.u.size());
      std::vector<float> fo;
      if (cfg.moe()) {
        // shared SwiGLU expert (model/train.go:490-503) plus the routed experts (model/train.go:538-552)
        linear(c.gate, c.m, params.at(LP(l, "mlp.c_gate.weight")), rows);
        bk.swiglu(c.hid.data(), c.gate.data(), c.u.data(), cfg.moe_effective_clamp(), (int64_t)c.hid.size());
        linear(fo, c.hid, params.at(LP(l, "mlp.c_proj.weight")), rows);
        std::vector<float> mo;
        moe_train_forward(c, mo, rows, l);
        for (size_t i = 0; i < x.size(); ++i) x[i] = c.mid[i] + (fo[i] + mo[i]);
      } else {
        bk.relu_squared(c.hid.data(), c.u.data(), (int64_t)c.u.size());
        linear(fo, c.hid, params.at(LP(l, "mlp.c_proj.weight")), rows);
        for (size_t i = 0; i < x.size(); ++i) x[i] = c.mid[i] + fo[i];
      }
      if (l == L / 2) ctx.backout = x;
    }
    if (!ctx.backout.empty()) {
      float lam = -params.at("backout_lambda").w[0];
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + lam * ctx.backout[i];
    }
    ctx.final_pre = x;
    norm(ctx.final_norm, x, d);
    lm_head(ctx.logits, ctx.final_norm, rows);
  }

  // ------------------------------------------------- training backward
  // dlogits: [B*T, V] gradient at the softcapped logits.
  void train_backward(TrainCtx& ctx, const std::vector<float>& dlogits) {
    int d = cfg.embed_dim, Hq = cfg.n_head, Hkv = cfg.n_kv_head, L = cfg.n_layer, V = cfg.vocab, B = ctx.B, T = ctx.T;
    int64_t rows = (int64_t)B * T;
    int ratio = Hq / Hkv;
    // SoftcapBackward (tensors/backward.go:108-116) then zero-pad to Vp (train_transformer.go:149-153)
    std::vector<float> gpad((size_t)rows * Vp, 0.0f);
    float invcap = 1.0f / kSoftcap;
    for (int64_t r = 0; r < rows; ++r) for (int v = 0; v < V; ++v) {
      double sc = (double)ctx.logits[(size_t)r * V + v] * (double)invcap;
      gpad[(size_t)r * Vp + v] = dlogits[(size_t)r * V + v] * (float)(1 - sc * sc);
    }
    std::vector<float> dy, dx;
    linear_backward(dy, ctx.final_norm, gpad, P("lm_head.weight"), rows);
    norm_backward(dx, ctx.final_pre, dy, d);
    std::vector<float> dbackout;
    if (!ctx.backout.empty()) {
      float lam = P("backout_lambda").w[0];
      dbackout.resize(dx.size());
      double dot = 0;
      for (size_t i = 0; i < dx.size(); ++i) { dbackout[i] = dx[i] * (-lam); dot += (double)dx[i] * (double)(-ctx.backout[i]); }
      P("backout_lambda").g[0] += (float)dot;
    }
    std::vector<float> dx0((size_t)rows * d, 0.0f);
    for (int l = L - 1; l >= 0; --l) {
      LayerCtx& c = ctx.layers[l];
      std::vector<float> dout = dx;
      if (l == L / 2 && !dbackout.empty()) for (size_t i = 0; i < dout.size(); ++i) dout[i] = dx[i] + dbackout[i];
      // ---- block backward (model/train.go:554-572)
      // MLP backward (model/train.go:505-514)
      std::vector<float> dhid, dm, dmid;
      linear_backward(dhid, c.hid, dout, P(LP(l, "mlp.c_proj.weight")), rows);
      std::vector<float> du(dhid.size(), 0.0f);
      if (cfg.moe()) {
        // shared SwiGLU expert (model/train.go:505-514), then the routed experts (model/train.go:563-566)
        std::vector<float> dgate(dhid.size()), t2, dmoe;
        bk.swiglu_backward(dgate.data(), du.data(), c.gate.data(), c.u.data(), dhid.data(), cfg.moe_effective_clamp(), (int64_t)dhid.size());
        linear_backward(dm, c.m, dgate, P(LP(l, "mlp.c_gate.weight")), rows);
        linear_backward(t2, c.m, du, P(LP(l, "mlp.c_fc.weight")), rows);
        for (size_t i = 0; i < dm.size(); ++i) dm[i] = dm[i] + t2[i];
        moe_train_backward(c, dmoe, dout, rows, T, l);
        for (size_t i = 0; i < dm.size(); ++i) dm[i] = dm[i] + dmoe[i];
      } else {
      for (size_t i = 0; i < du.size(); ++i) if (c.u[i] > 0) du[i] = dhid[i] * 2 * c.u[i];   // tensors/backward.go:57-65
      linear_backward(dm, c.m, du, P(LP(l, "mlp.c_fc.weight")), rows);
      }
      std::vector<float> nb;
      norm_backward(nb, c.mid, dm, d);
      dmid.resize(dout.size());
      for (size_t i = 0; i < dmid.size(); ++i) dmid[i] = dout[i] + nb[i];
      // ---- attention backward (model/train.go:198-427)
      std::vector<float> os, dos, doh;
      to_seq_major(os, c.o_hm, B, T, Hq, D);
      linear_backward(dos, os, dmid, P(LP(l, "attn.c_proj.weight")), rows);
      to_head_major(doh, dos, B, T, Hq, D);
      std::vector<float> dq((size_t)rows * Hq * D, 0.0f), dk((size_t)rows * Hkv * D, 0.0f), dv((size_t)rows * Hkv * D, 0.0f);
      // Sequential over (batch, head) as in the reference: K/V gradients of a
      // shared kv head accumulate in query-head order.
      for (int b = 0; b < B; ++b) for (int hq = 0; hq < Hq; ++hq) {
        int hk = hq / ratio; size_t idx = (size_t)b * Hq + hq, slot = (size_t)b * Hkv + hk;
        bk.attention_backward(c.q_hm.data() + idx * T * D, c.k_hm.data() + slot * T * D, c.v_hm.data() + slot * T * D,
                              doh.data() + idx * T * D, c.lse.data() + idx * T, nullptr, T, T, D, 0, windows[l], nullptr, 0,
                              dq.data() + idx * T * D, dk.data() + slot * T * D, dv.data() + slot * T * D);
      }
      std::vector<float> dqs, dks, dvs, dqp, dkp;
      std::vector<float> dh, t1;
      if (cfg.mla()) {
        // model/train.go:414-419 and model/mla.go:126-146: inverse rotation, split into content / rotary parts, the two
        // up-projections into the shared latents, then the down-projections and the rotary projections into h
        const int rope = cfg.mla_rope(), content = cfg.mla_content(), lat = cfg.mla_latent;
        to_seq_major(dqs, dq, B, T, Hq, D); to_seq_major(dks, dk, B, T, Hkv, D); to_seq_major(dvs, dv, B, T, Hkv, D);
        rotary(dqs, B, T, Hq, 0, -1.0f);
        rotary(dks, B, T, Hkv, 0, -1.0f);
        auto split = [&](const std::vector<float>& src, std::vector<float>& cc, std::vector<float>& rr, int H) {
          cc.resize((size_t)rows * H * content); rr.resize((size_t)rows * H * rope);
          for (int64_t i = 0; i < rows * H; ++i) {
            std::copy(src.begin() + i * D, src.begin() + i * D + content, cc.begin() + i * content);
            std::copy(src.begin() + i * D + content, src.begin() + (i + 1) * D, rr.begin() + i * rope);
          }
        };
        std::vector<float> dqc, dqr, dkc, dkr, dql, dkvl, t3;
        split(dqs, dqc, dqr, Hq); split(dks, dkc, dkr, Hkv);
        linear_backward(dql, c.mla_ql, dqc, P(LP(l, "attn.mla_q_up.weight")), rows);
        linear_backward(dh, c.h, dql, P(LP(l, "attn.mla_q_down.weight")), rows);
        linear_backward(t1, c.h, dqr, P(LP(l, "attn.mla_q_rope.weight")), rows);
        for (size_t i = 0; i < dh.size(); ++i) dh[i] = dh[i] + t1[i];
        linear_backward(dkvl, c.mla_kvl, dkc, P(LP(l, "attn.mla_k_up.weight")), rows);
        linear_backward(t3, c.mla_kvl, dvs, P(LP(l, "attn.mla_v_up.weight")), rows);
        for (size_t i = 0; i < dkvl.size(); ++i) dkvl[i] = dkvl[i] + t3[i];
        linear_backward(t1, c.h, dkvl, P(LP(l, "attn.mla_kv_down.weight")), rows);
        for (size_t i = 0; i < dh.size(); ++i) dh[i] = dh[i] + t1[i];
        linear_backward(t1, c.h, dkr, P(LP(l, "attn.mla_k_rope.weight")), rows);
        for (size_t i = 0; i < dh.size(); ++i) dh[i] = dh[i] + t1[i];
        (void)lat;
      } else {
      for (auto& e : dq) e *= kQKScale;
      for (auto& e : dk) e *= kQKScale;
      to_seq_major(dqs, dq, B, T, Hq, D); to_seq_major(dks, dk, B, T, Hkv, D); to_seq_major(dvs, dv, B, T, Hkv, D);
      norm_backward(dqp, c.q_rot, dqs, D);
      norm_backward(dkp, c.k_rot, dks, D);
      rotary(dqp, B, T, Hq, 0, -1.0f);
      rotary(dkp, B, T, Hkv, 0, -1.0f);
      linear_backward(dh, c.h, dqp, P(LP(l, "attn.c_q.weight")), rows);
      linear_backward(t1, c.h, dkp, P(LP(l, "attn.c_k.weight")), rows);
      for (size_t i = 0; i < dh.size(); ++i) dh[i] = dh[i] + t1[i];
      linear_backward(t1, c.h, dvs, P(LP(l, "attn.c_v.weight")), rows);
      for (size_t i = 0; i < dh.size(); ++i) dh[i] = dh[i] + t1[i];
      }
      if (!c.ve.empty()) {
        // model/train.go:375-409
        Param& wg = P(LP(l, "attn.ve_gate.weight"));
        Param& vew = P("value_embeds." + std::to_string(l) + ".weight");
        std::vector<float> dve((size_t)rows * KV), dpre((size_t)rows * Hkv);
        for (int64_t r = 0; r < rows * Hkv; ++r) {
          float scale = c.ve_sig[r] * kVeGateScale;
          double dp = 0;
          for (int cc = 0; cc < D; ++cc) {
            dve[(size_t)r * D + cc] = dvs[(size_t)r * D + cc] * scale;
            dp += (double)dvs[(size_t)r * D + cc] * (double)c.ve[(size_t)r * D + cc];
          }
          float dgate = (float)dp;
          float dsig = dgate * kVeGateScale;
          float sig = c.ve_sig[r];
          dpre[r] = dsig * sig * (1 - sig);
        }
        std::vector<float> slice((size_t)rows * kVeGateChannels), dslice;
        for (int64_t r = 0; r < rows; ++r) std::copy(c.h.begin() + r * d, c.h.begin() + r * d + kVeGateChannels, slice.begin() + r * kVeGateChannels);
        linear_backward(dslice, slice, dpre, wg, rows);
        for (int64_t r = 0; r < rows; ++r) for (int cc = 0; cc < kVeGateChannels; ++cc) dh[(size_t)r * d + cc] = dh[(size_t)r * d + cc] + dslice[(size_t)r * kVeGateChannels + cc];
        // value_embeds scatter-add by token id (train_transformer.go:213-216, layers/linear.go:90-104)
        for (int64_t r = 0; r < rows; ++r) {
          float* gr = vew.g.data() + (size_t)ctx.ids[r] * KV;
          for (int cc = 0; cc < KV; ++cc) gr[cc] += dve[(size_t)r * KV + cc];
        }
      }
      std::vector<float> din;
      norm_backward(din, c.x_in, dh, d);
      for (size_t i = 0; i < din.size(); ++i) din[i] = din[i] + dmid[i];
      // ---- residual mix (train_transformer.go:218-242)
      float rw = P("resid_lambdas").w[l], xw = P("x0_lambdas").w[l];
      double rdot = 0, xdot = 0;
      for (size_t i = 0; i < din.size(); ++i) { rdot += (double)din[i] * (double)c.prev_x[i]; xdot += (double)din[i] * (double)ctx.x0[i]; }
      P("resid_lambdas").g[l] += (float)rdot;
      P("x0_lambdas").g[l] += (float)xdot;
      dx.resize(din.size());
      for (size_t i = 0; i < din.size(); ++i) { dx[i] = din[i] * rw; dx0[i] = dx0[i] + xw * din[i]; }
    }
    for (size_t i = 0; i < dx.size(); ++i) dx[i] = dx[i] + dx0[i];
    // ---- smear backward (train_transformer.go:269-305)
    float lam = P("smear_lambda").w[0];
    std::vector<float> de((size_t)rows * d, 0.0f), dgate((size_t)B * (T - 1), 0.0f);
    double dlam = 0;
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) {
      size_t base = ((size_t)b * T + t) * d;
      if (t == 0) { for (int c = 0; c < d; ++c) de[base + c] += dx[base + c]; continue; }
      size_t gi = (size_t)b * (T - 1) + (t - 1), pb = base - d;
      float gv = lam * ctx.smear_sig[gi];
      double gs = 0;
      for (int c = 0; c < d; ++c) {
        de[base + c] += dx[base + c];
        de[pb + c] += dx[base + c] * gv;
        gs += (double)dx[base + c] * (double)ctx.e_alias[pb + c];
      }
      float sg = ctx.smear_sig[gi];
      dlam += gs * (double)sg;
      dgate[gi] = (float)(gs * (double)lam) * sg * (1 - sg);
    }
    P("smear_lambda").g[0] += (float)dlam;
    std::vector<float> dslice;
    linear_backward(dslice, ctx.smear_slice, dgate, P("smear_gate.weight"), (int64_t)B * (T - 1));
    for (int b = 0; b < B; ++b) for (int t = 1; t < T; ++t) for (int c = 0; c < kSmearChannels; ++c)
      de[((size_t)b * T + t) * d + c] += dslice[((size_t)b * (T - 1) + (t - 1)) * kSmearChannels + c];
    std::vector<float> draw;
    norm_backward(draw, ctx.raw, de, d);
    Param& wte = P("transformer.wte.weight");
    for (int64_t r = 0; r < rows; ++r) {
      float* gr = wte.g.data() + (size_t)ctx.ids[r] * d;
      for (int c = 0; c < d; ++c) gr[c] += draw[(size_t)r * d + c];
    }
  }
};

}  // namespace gnor
