// TEST INFRASTRUCTURE: CPU restatement of the reference's optimizer step (optimizer/optimizer.go,
// optimizer/muon.go, optimizer/sinkhorn.go) and of the parameter routing chat_rl uses
// (model/optimizer.go:20-165, cmd/chat_rl/main.go:68-72).  Only tests/, the smoke check and the
// benchmark's CPU baseline may use it; the product never does.
#pragma once
#include <cmath>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "backend.h"
#include "model.h"

namespace gnopt {
using namespace gnor;

// optimizer/optimizer.go:143-173 (all arithmetic in float64, stored as float32; `step` is the 1-based count)
inline void adamw_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, int step, float lr, float beta1, float beta2,
                       float eps, float weight_decay) {
  const double b1 = beta1, b2 = beta2, e = eps, wd = weight_decay, l = lr;
  const double bias1 = 1 - std::pow(b1, (double)step), bias2 = 1 - std::pow(b2, (double)step);
  const double decay = 1 - l * wd, step_size = l / bias1;
  for (int64_t i = 0; i < n; ++i) {
    param[i] *= (float)decay;
    exp_avg[i] = (float)(b1 * (double)exp_avg[i] + (1 - b1) * (double)grad[i]);
    exp_avg_sq[i] = (float)(b2 * (double)exp_avg_sq[i] + (1 - b2) * (double)grad[i] * (double)grad[i]);
    const double denom = std::sqrt((double)exp_avg_sq[i] / bias2) + e;
    param[i] -= (float)(step_size * (double)exp_avg[i] / denom);
  }
}

inline float frobenius(const float* v, int64_t n) { double s = 0; for (int64_t i = 0; i < n; ++i) s += (double)v[i] * (double)v[i]; return (float)std::sqrt(s); }

// optimizer/muon.go:11-17
static const double kPolarExpress[5][3] = {
    {8.156554524902461, -22.48329292557795, 15.878769915207462},
    {4.042929935166739, -2.808917465908714, 0.5000178451051316},
    {3.8916678022926607, -2.772484153217685, 0.5060648178503393},
    {3.285753657755655, -2.3681294933425376, 0.46449024233003106},
    {2.3465413258596377, -1.7097828382687081, 0.42323551169305323},
};

// optimizer/muon.go:23-173.  second_mom has max(rows, cols) entries (per row when rows >= cols, else per column).
inline void muon_step(const Backend& bk, float* param, const float* grad, float* mom, float* second_mom, int rows, int cols, float lr, float momentum,
                      int ns_steps, float beta2, float weight_decay) {
  const int64_t n = (int64_t)rows * cols;
  std::vector<float> u(n);
  for (int64_t i = 0; i < n; ++i) {
    mom[i] = momentum * mom[i] + (1 - momentum) * grad[i];
    u[i] = (1 - momentum) * grad[i] + momentum * mom[i];
  }
  // row equilibration
  const float target = frobenius(u.data(), n) / (float)std::sqrt((double)rows);
  for (int r = 0; r < rows; ++r) {
    float rn = frobenius(u.data() + (int64_t)r * cols, cols);
    if (rn < 1e-6f) rn = 1e-6f;
    const float sc = target / rn;
    for (int c = 0; c < cols; ++c) u[(int64_t)r * cols + c] *= sc;
  }
  // Polar Express
  const float norm = frobenius(u.data(), n);
  const float sc0 = (float)(1.0 / ((double)norm * 1.01 + 1e-6));
  for (auto& v : u) v *= sc0;
  const bool tall = rows > cols;
  const int g = tall ? cols : rows;
  std::vector<float> ut(n), gram((size_t)g * g), gram2((size_t)g * g), poly((size_t)g * g), prod(n);
  for (int s = 0; s < ns_steps; ++s) {
    const float a = (float)kPolarExpress[s][0], b = (float)kPolarExpress[s][1], c = (float)kPolarExpress[s][2];
    for (int r = 0; r < rows; ++r) for (int cc = 0; cc < cols; ++cc) ut[(int64_t)cc * rows + r] = u[(int64_t)r * cols + cc];
    if (tall) bk.matmul(gram.data(), ut.data(), u.data(), cols, cols, rows);   // U^T U
    else bk.matmul(gram.data(), u.data(), ut.data(), rows, rows, cols);        // U U^T
    bk.matmul(gram2.data(), gram.data(), gram.data(), g, g, g);
    for (size_t i = 0; i < poly.size(); ++i) poly[i] = gram[i] * b + gram2[i] * c;
    if (tall) bk.matmul(prod.data(), u.data(), poly.data(), rows, cols, cols);
    else bk.matmul(prod.data(), poly.data(), u.data(), rows, cols, rows);
    for (int64_t i = 0; i < n; ++i) u[i] = u[i] * a + prod[i];
  }
  // Muon+ renormalisation
  float cur = frobenius(u.data(), n);
  if (cur < 1e-6f) cur = 1e-6f;
  const float renorm = (float)std::sqrt((double)std::min(rows, cols)) / cur;
  for (auto& v : u) v *= renorm;
  // variance reduction
  const bool per_row = rows >= cols;
  const int nv = per_row ? rows : cols, reduce = per_row ? cols : rows;
  std::vector<float> vmean(nv), step(nv), fin(nv);
  if (per_row) {
    for (int r = 0; r < rows; ++r) { double s = 0; for (int c = 0; c < cols; ++c) { double v = u[(int64_t)r * cols + c]; s += v * v; } vmean[r] = (float)(s / (double)cols); }
  } else {
    for (int c = 0; c < cols; ++c) { double s = 0; for (int r = 0; r < rows; ++r) { double v = u[(int64_t)r * cols + c]; s += v * v; } vmean[c] = (float)(s / (double)rows); }
  }
  double vns = 0;
  for (float v : vmean) vns += (double)v;
  vns *= (double)reduce;
  const float vnorm = (float)std::sqrt(vns);
  for (int i = 0; i < nv; ++i) {
    second_mom[i] = beta2 * second_mom[i] + (1 - beta2) * vmean[i];
    float sm = second_mom[i];
    if (sm < 1e-10f) sm = 1e-10f;
    step[i] = (float)(1.0 / std::sqrt((double)sm));
  }
  double nvs = 0;
  for (int i = 0; i < nv; ++i) nvs += (double)vmean[i] * (double)reduce * (double)step[i] * (double)step[i];
  float nvn = (float)std::sqrt(nvs);
  if (nvn < 1e-10f) nvn = 1e-10f;
  const float ratio = vnorm / nvn;
  for (int i = 0; i < nv; ++i) fin[i] = step[i] * ratio;
  for (int r = 0; r < rows; ++r) for (int c = 0; c < cols; ++c) u[(int64_t)r * cols + c] *= fin[per_row ? r : c];
  // cautious weight decay + update
  for (int64_t i = 0; i < n; ++i) {
    const float mask = (u[i] * param[i] >= 0) ? 1.0f : 0.0f;
    param[i] -= lr * u[i] + lr * weight_decay * param[i] * mask;
  }
}

// optimizer/sinkhorn.go:27-95
inline void sinkhorn_step(float* param, const float* grad, float* mom, int rows, int cols, float lr, float momentum, float gamma, int steps, float tau,
                          float eps) {
  const int64_t n = (int64_t)rows * cols;
  const double beta = momentum;
  std::vector<float> u(n);
  for (int64_t i = 0; i < n; ++i) {
    const double mv = beta * (double)mom[i] + (1 - beta) * (double)grad[i];
    mom[i] = (float)mv;
    u[i] = (float)(beta * mv + (1 - beta) * (double)grad[i]);
  }
  auto row_norm = [&](int r) { double s = 0; for (int c = 0; c < cols; ++c) { double v = u[(int64_t)r * cols + c]; s += v * v; } return std::sqrt(s); };
  std::vector<double> rn(rows);
  double nsum = 0;
  for (int r = 0; r < rows; ++r) { rn[r] = row_norm(r); nsum += rn[r]; }
  const double thr = (double)tau * nsum / (double)rows;
  for (int r = 0; r < rows; ++r) if (rn[r] <= thr) for (int c = 0; c < cols; ++c) u[(int64_t)r * cols + c] = 0.0f;
  const double e = eps;
  for (int s = 1; s <= steps; ++s) {
    if (s % 2 == 1) {
      for (int r = 0; r < rows; ++r) { const double sc = 1.0 / (row_norm(r) + e); for (int c = 0; c < cols; ++c) { float& v = u[(int64_t)r * cols + c]; v = (float)((double)v * sc); } }
    } else {
      for (int c = 0; c < cols; ++c) {
        double sum = 0;
        for (int r = 0; r < rows; ++r) { double v = u[(int64_t)r * cols + c]; sum += v * v; }
        const double sc = 1.0 / (std::sqrt(sum) + e);
        for (int r = 0; r < rows; ++r) { float& v = u[(int64_t)r * cols + c]; v = (float)((double)v * sc); }
      }
    }
  }
  const double l = (double)gamma * (double)lr * std::sqrt((double)cols);
  for (int64_t i = 0; i < n; ++i) param[i] -= (float)(l * (double)u[i]);
}

// The optimizer chat_rl builds for a model (dense or latent preset): SetupOptimizer(0.004, 0.2, 0.02, 0.0, 0.5, true) with every
// learning rate multiplied by 0.05 (cmd/chat_rl/main.go:68-72), i.e. Sinkhorn for lm_head / wte / value embeddings,
// AdamW for the scalar groups, Muon for every block matrix (model/optimizer.go:20-165).
struct Optimizer {
  Model* m;
  float unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr, lr_mult;
  int step_count = 0;
  std::map<std::string, std::vector<float>> mom, second;   // momentum / exp_avg ; second moment / exp_avg_sq
  Optimizer(Model* model, float ulr, float elr, float mlr, float wd, float slr, float mult)
      : m(model), unembedding_lr(ulr), embedding_lr(elr), matrix_lr(mlr), weight_decay(wd), scalar_lr(slr), lr_mult(mult) {
    for (auto& kv : m->params) {
      mom[kv.first].assign(kv.second.w.size(), 0.0f);
      second[kv.first].assign(kv.second.w.size(), 0.0f);   // Muon uses the first max(rows, cols) entries
    }
  }
  static bool ends_with(const std::string& s, const char* suf) { std::string t(suf); return s.size() >= t.size() && s.compare(s.size() - t.size(), t.size(), t) == 0; }
  void step() {
    ++step_count;
    const float dscale = (float)std::pow((double)m->cfg.embed_dim / 768.0, -0.5);
    for (auto& kv : m->params) {
      const std::string& name = kv.first; Param& p = kv.second;
      float* mo = mom[name].data(); float* se = second[name].data();
      const int64_t n = (int64_t)p.w.size();
      auto sink = [&](float lr) { sinkhorn_step(p.w.data(), p.g.data(), mo, p.rows, p.cols, lr * lr_mult, 0.95f, 0.18f, 11, 1e-3f, 1e-20f); };
      auto adam = [&](float lr, float b1, float b2, float wd) { adamw_step(p.w.data(), p.g.data(), mo, se, n, step_count, lr * lr_mult, b1, b2, 1e-10f, wd); };
      if (name == "lm_head.weight") sink(unembedding_lr * dscale);
      else if (name == "transformer.wte.weight") sink(embedding_lr * dscale);
      else if (name.rfind("value_embeds.", 0) == 0) sink(embedding_lr * dscale * 0.5f);
      else if (name == "resid_lambdas") adam(scalar_lr * 0.01f, 0.8f, 0.95f, 0.05f);
      else if (name == "x0_lambdas") adam(scalar_lr, 0.96f, 0.95f, 0.0f);
      else if (name == "smear_gate.weight" || name == "smear_lambda" || name == "backout_lambda") adam(0.2f, 0.8f, 0.95f, 0.0f);
      else if (ends_with(name, "moe.router_bias")) continue;   // updated by load, never optimised (model/optimizer.go:83-86)
      else if (name.find(".moe.experts.") != std::string::npos) {
        // packed expert weights: one Muon matrix per expert view (model/optimizer.go:87-93, model/moe.go:60-81)
        const int E = m->cfg.n_experts, er = p.rows / E;
        for (int e = 0; e < E; ++e) {
          const int64_t off = (int64_t)e * er * p.cols;
          muon_step(m->bk, p.w.data() + off, p.g.data() + off, mo + off, se + off, er, p.cols, matrix_lr * lr_mult, 0.95f, 5, 0.9f, weight_decay);
        }
      }
      else muon_step(m->bk, p.w.data(), p.g.data(), mo, se, p.rows, p.cols, matrix_lr * lr_mult, 0.95f, 5, 0.9f, weight_decay);
    }
    m->zero_grad();   // trainer/rl.go:65-66
  }
};

}  // namespace gnopt
