// Resident session (Tier B): the dense transformer of the reference held in
// device memory, with the three phases of the RL step driven from the host in
// C++: batched rollout (inference/engine.go:112-369 over
// model/transformer.go:243-342), the policy-gradient loss and the training
// forward/backward (trainer/rl.go:14-60, model/train_transformer.go:63-320,
// model/train.go:55-572).
//
// Memory layout in HBM
//   parameters / gradients: one flat float32 buffer each, every tensor padded to
//     a multiple of 64 floats; per layer c_q, c_k, c_v are adjacent so that the
//     three projections are one GEMM.  The gradient buffer is what the
//     data-parallel all-reduce sums.
//   KV cache: [layer][k|v][row][kv head][max_seq][head_dim], contiguous per
//     (row, head) like the reference's cache (model/kvcache.go:10-28), all rows
//     of all prompts in one batch.
//   activations: token-major [rows, width]; attention reads Q/K/V in place from
//     the fused projection output through strides (no head-major transposes).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

#include <cstring>
#include "model_internal.cuh"

using namespace gn;



namespace {

int64_t align64(int64_t n) { return (n + 63) / 64 * 64; }

bool has_ve(int layer, int L) { return layer % 2 == (L - 1) % 2; }  // model/helpers.go:69-71

int build_layout(gn_model* m) {
  const int d = m->d, L = m->L, D = m->D, Hq = m->Hq, Hkv = m->Hkv, Vp = m->Vp, KV = m->KV;
  int64_t off = 0;
  auto add = [&](const std::string& name, int rows, int cols, bool align = true) {
    ParamInfo pi; pi.name = name; pi.rows = rows; pi.cols = cols;
    if (align) off = align64(off);
    pi.offset = off; off += (int64_t)rows * cols;
    m->params.push_back(pi);
    return pi.offset;
  };
  m->off_wte = add("transformer.wte.weight", Vp, d);
  m->off_lm = add("lm_head.weight", Vp, d);
  m->lo.resize(L);
  for (int l = 0; l < L; ++l) {
    std::string p = "transformer.h." + std::to_string(l) + ".";
    LayerOffsets& o = m->lo[l];
    o.qkv = -1;
    if (m->mla()) {
      // model/mla.go:41-60.  The four projections of the block input are adjacent: one [2 lat + (Hq+Hkv) rope, d] matrix.
      o.mla_cat = add(p + "attn.mla_q_down.weight", m->lat, d);
      add(p + "attn.mla_kv_down.weight", m->lat, d, false);
      add(p + "attn.mla_q_rope.weight", Hq * m->rope, d, false);
      add(p + "attn.mla_k_rope.weight", Hkv * m->rope, d, false);
      o.mla_q_up = add(p + "attn.mla_q_up.weight", Hq * m->content, m->lat);
      o.mla_k_up = add(p + "attn.mla_k_up.weight", Hkv * m->content, m->lat);
      o.mla_v_up = add(p + "attn.mla_v_up.weight", Hkv * D, m->lat);
    } else {
      o.qkv = add(p + "attn.c_q.weight", Hq * D, d);
      add(p + "attn.c_k.weight", KV, d, false);   // adjacent: [c_q; c_k; c_v] is one [W, d] matrix
      add(p + "attn.c_v.weight", KV, d, false);
    }
    o.proj = add(p + "attn.c_proj.weight", d, d);
    o.has_ve = !m->mla() && has_ve(l, L);        // model/transformer.go:73
    o.ve_gate = o.ve = -1;
    if (o.has_ve) {
      o.ve_gate = add(p + "attn.ve_gate.weight", Hkv, kVeGateChannels);
      o.ve = add("value_embeds." + std::to_string(l) + ".weight", Vp, KV);
    }
    if (m->moe()) {
      // shared SwiGLU expert (model/block.go:23-25): [c_fc; c_gate] adjacent; routed experts packed (model/moe.go:26-45)
      o.fc = add(p + "mlp.c_fc.weight", m->sh, d);
      add(p + "mlp.c_gate.weight", m->sh, d, false);
      o.mproj = add(p + "mlp.c_proj.weight", d, m->sh);
      o.router = add(p + "moe.router.weight", m->E, d);
      o.router_bias = add(p + "moe.router_bias", 1, m->E);
      o.exp_gate = add(p + "moe.experts.gate.weight", m->E * m->eh, d);
      o.exp_up = add(p + "moe.experts.up.weight", m->E * m->eh, d);
      o.exp_down = add(p + "moe.experts.down.weight", m->E * d, m->eh);
    } else {
      o.fc = add(p + "mlp.c_fc.weight", 4 * d, d);
      o.mproj = add(p + "mlp.c_proj.weight", d, 4 * d);
    }
  }
  m->off_smear_gate = add("smear_gate.weight", 1, kSmearChannels);
  // The four scalar parameter groups are adjacent (2L+2 floats) so that their
  // float64 accumulators flush in one launch.
  m->off_rho = add("resid_lambdas", 1, L);
  m->off_chi = add("x0_lambdas", 1, L, false);
  m->off_smear_lambda = add("smear_lambda", 1, 1, false);
  m->off_backout = add("backout_lambda", 1, 1, false);
  m->total = align64(off);
  std::sort(m->params.begin(), m->params.end(), [](const ParamInfo& a, const ParamInfo& b) { return a.name < b.name; });
  for (size_t i = 0; i < m->params.size(); ++i) m->index[m->params[i].name] = (int)i;
  return GN_OK;
}

int enter(gn_model* m) {
  GN_REQUIRE(m && m->ctx, "null model");
  GN_CUDA(cudaSetDevice(m->ctx->device));
  return GN_OK;
}
// Token ids arrive from the host and index the embedding tables, the value-embedding tables and the logits row:
// an id outside the vocabulary is refused before anything is launched (the reference panics on the slice bound,
// model/layers/linear.go:71-85).  allow_ignore admits -1 (the ignored-target marker of tensors/loss.go:16-46).
int check_ids(const int32_t* ids, int64_t n, int vocab, bool allow_ignore, const char* what) {
  for (int64_t i = 0; i < n; ++i) {
    const int32_t v = ids[i];
    if ((v >= 0 && v < vocab) || (allow_ignore && v == -1)) continue;
    set_error("%s[%lld] = %d is outside [0, %d)%s", what, (long long)i, (int)v, vocab, allow_ignore ? " and is not -1" : "");
    return GN_ERR_INVALID;
  }
  return GN_OK;
}

// Entry of a compute phase: stale operand splits are dropped before the first GEMM.
int enter_compute(gn_model* m) {
  GN_TRY(enter(m));
  if (m->weights_dirty) { gemm_mark_static_stale(); m->weights_dirty = false; }
  return GN_OK;
}

// ------------------------------------------------------------------ forward
size_t plan_bufs(gn_model* m, Arena& a, FwdBufs& b, Mode mode, int64_t rows, int64_t logit_rows, int B, int T) {
  const int d = m->d, W = m->W, Hq = m->Hq, Hkv = m->Hkv, D = m->D, V = m->V, L = m->L;
  b.E = a.take(rows * d);
  b.X0 = a.take(rows * d);
  b.Y = a.take(std::max<int64_t>(rows, logit_rows) * d);
  b.LOGITS = a.take(logit_rows * V);
  b.S1h = a.take(std::max<int64_t>(rows, logit_rows) * d); b.S1l = a.take(std::max<int64_t>(rows, logit_rows) * d);
  b.S4h = a.take(rows * 4 * d); b.S4l = a.take(rows * 4 * d);
  if (mode == MODE_TRAIN) {
    b.SIG = a.take((int64_t)B * std::max(T - 1, 1));
    b.FP = a.take(rows * d);
    b.layers.resize(L);
    for (int l = 0; l < L; ++l) {
      LayerSaved& s = b.layers[l];
      s.Xin = a.take(rows * d); s.H = a.take(rows * d); s.QKV = a.take(rows * W);
      s.QKROT = m->mla() ? nullptr : a.take(rows * (int64_t)(Hq + Hkv) * D);
      s.O = a.take(rows * (int64_t)Hq * D); s.LSE = a.take((int64_t)B * Hq * T); s.VESIG = m->mla() ? nullptr : a.take(rows * Hkv);
      s.MID = a.take(rows * d); s.M = a.take(rows * d); s.XOUT = a.take(rows * d);
      if (m->moe()) s.U = s.HID = nullptr; else { s.U = a.take(rows * 4 * d); s.HID = a.take(rows * 4 * d); }
      if (m->ctx->gemm_kind == 1) {
        s.Hh = a.take(rows * d); s.Hl = a.take(rows * d); s.Mh = a.take(rows * d); s.Ml = a.take(rows * d);
        if (!m->moe()) { s.Ph = a.take(rows * 4 * d); s.Pl = a.take(rows * 4 * d); }
      }
      if (m->mla() || m->moe()) {   // what the latent preset's layers keep for their backward (model_latent_train.cu)
        float* base = a.take(latent_saved_layout(m, nullptr, nullptr, rows));
        if (base) latent_saved_layout(m, base, &s, rows);
      }
    }
    b.Xa = b.Xb = b.H = b.QKV = b.O = b.M = b.HID = b.BO = nullptr;
  } else {
    b.Xa = a.take(rows * d); b.Xb = nullptr;
    b.H = a.take(rows * d); b.QKV = a.take(rows * W); b.O = a.take(rows * (int64_t)Hq * D);
    b.M = a.take(rows * d); b.HID = a.take(rows * 4 * d); b.BO = a.take(rows * d);
    b.SIG = b.FP = nullptr;
    if (m->mla()) {
      const int64_t n1 = 2 * m->lat + (int64_t)(Hq + Hkv) * m->rope;
      b.P1 = a.take(rows * n1); b.QC = a.take(rows * (int64_t)Hq * m->content); b.QF = a.take(rows * (int64_t)Hq * (m->lat + m->rope));
      b.AL = a.take(rows * (int64_t)Hq * m->lat);
    }
    if (m->moe()) {
      const int64_t tot = rows * m->topk;
      b.UG = a.take(rows * 2 * m->sh); b.SHH = a.take(rows * m->sh); b.SHO = a.take(rows * d);
      b.RL = a.take(rows * m->E); b.PR = a.take(rows * m->E); b.SELW = a.take(tot);
      b.GATH = a.take(tot * d); b.GG = a.take(tot * m->eh); b.GU = a.take(tot * m->eh); b.GO = a.take(tot * d);
      b.SEL = (int32_t*)a.take(tot); b.CNT = (int32_t*)a.take(m->E + 1); b.POSI = (int32_t*)a.take(tot);
      b.GATHh = a.take(tot * d); b.GATHl = a.take(tot * d); b.GHh = a.take(tot * m->eh); b.GHl = a.take(tot * m->eh);
    }
  }
  return a.planned;
}

int make_bufs(gn_model* m, Arena& a, FwdBufs& b, Mode mode, int64_t rows, int64_t logit_rows, int B, int T, size_t extra_floats, float** extra) {
  a.planning = true; a.planned = 0;
  plan_bufs(m, a, b, mode, rows, logit_rows, B, T);
  if (extra_floats) a.take(extra_floats);
  size_t need = a.planned;
  a.planning = false;
  GN_TRY(a.buf.ensure(need));
  a.used = 0;
  plan_bufs(m, a, b, mode, rows, logit_rows, B, T);
  if (extra_floats) *extra = a.take(extra_floats);
  return GN_OK;
}

// Runs the trunk.  Returns with b.Y = final normalised hidden rows that feed lm_head
// (PREFILL: one row per sequence, the last position) and b.LOGITS filled.
int forward_core(gn_model* m, FwdBufs& b, const FwdArgs& a) {
  const int d = m->d, W = m->W, Hq = m->Hq, Hkv = m->Hkv, D = m->D, V = m->V, L = m->L;
  const int B = a.B, T = a.T;
  const int64_t rows = (int64_t)B * T;
  cudaStream_t s = m->s();
  const bool train = a.mode == MODE_TRAIN;
  const bool cached = a.mode == MODE_PREFILL || a.mode == MODE_DECODE;
  const int prefetch = train ? 0 : 1;   // inference: no kernel in flight writes the parameters, products may request them early

  // Decode (one token per row): embedding, smear and layer 0's mix + norm in one launch.
  const bool front = a.mode == MODE_DECODE && T == 1 && a.cache_row_mul == 1 && sum_norm_supported(d) && d >= 128;
  if (front) {
    const bool tc0 = m->ctx->gemm_kind == 1;
    GN_TRY(decode_front_launch(a.ids, m->p(m->off_wte), m->prev.f(), m->p(m->off_smear_gate), m->p(m->off_smear_lambda), m->p(m->off_rho), m->p(m->off_chi),
                               b.X0, b.Xa, b.H, tc0 ? b.S1h : nullptr, tc0 ? b.S1l : nullptr, rows, d, s));
  } else {
    GN_TRY(embed_norm_launch(a.ids, m->p(m->off_wte), b.E, rows, d, s));
    const float* prev_in = (a.mode == MODE_DECODE) ? m->prev.f() : nullptr;
    float* prev_out = cached ? m->prev.f() : nullptr;
    GN_TRY(smear_launch(b.E, b.X0, prev_in, prev_out, a.cache_row_mul, train ? b.SIG : nullptr, m->p(m->off_smear_gate), m->p(m->off_smear_lambda),
                        B, T, d, s));
  }
  const int64_t layer_stride = (int64_t)a.cache_rows * Hkv * a.max_seq * D;
  const float* x_prev = b.X0;
  const float* backout = nullptr;
  Partials pending;   // the previous layer's output projection, not yet added to its residual
  for (int l = 0; l < L; ++l) {
    const LayerOffsets& o = m->lo[l];
    float *Xin, *H, *QKV, *O, *MID, *Mn, *U, *HID, *XOUT;
    if (train) {
      LayerSaved& sv = b.layers[l];
      Xin = sv.Xin; H = sv.H; QKV = sv.QKV; O = sv.O; MID = sv.MID; Mn = sv.M; U = sv.U; HID = sv.HID; XOUT = sv.XOUT;
    } else {
      Xin = b.Xa; H = b.H; QKV = b.QKV; O = b.O; MID = b.Xa; Mn = b.M; U = nullptr; HID = b.HID; XOUT = b.Xa;
    }
    const bool tc = m->ctx->gemm_kind == 1;
    // where the tf32 splits of H, M and HID go: kept per layer in training (the backward reads them), shared otherwise
    float* Hh = (train && tc) ? b.layers[l].Hh : b.S1h; float* Hl = (train && tc) ? b.layers[l].Hl : b.S1l;
    float* Mh = (train && tc) ? b.layers[l].Mh : b.S1h; float* Ml = (train && tc) ? b.layers[l].Ml : b.S1l;
    float* Ph = (train && tc) ? b.layers[l].Ph : b.S4h; float* Pl = (train && tc) ? b.layers[l].Pl : b.S4l;
    // Inference on the tensor-core path: products whose K loop was split over CTAs are left as partial
    // tiles and summed by the kernel that consumes them (one launch less per product).
    const bool fuse = tc && !train && sum_norm_supported(d) && D % 4 == 0;
    if (pending.on()) {
      SumNorm sn; sn.R = x_prev; sn.part = pending; sn.X0 = b.X0; sn.rho = m->p(m->off_rho); sn.chi = m->p(m->off_chi); sn.layer = l;
      if (l - 1 == L / 2) { sn.Xsum = b.BO; backout = b.BO; }
      sn.V = Xin; sn.Y = H; sn.Yh = Hh; sn.Yl = Hl; sn.rows = rows; sn.d = d;
      GN_TRY(sum_norm_launch(sn, s));
      pending = Partials();
    } else if (!(front && l == 0)) {   // the decode front already produced layer 0's Xin and H
      GN_TRY(mix_norm_launch(x_prev, b.X0, m->p(m->off_rho), m->p(m->off_chi), l, Xin, H, tc ? Hh : nullptr, tc ? Hl : nullptr, rows, d, s));
    }
    bool o_split = false;   // the attention kernel also wrote the tf32 split of O
    if (m->mla()) {
      if (train) GN_TRY(latent_attention_train(m, b.layers[l], *b.lws, l, H, tc ? Hh : nullptr, tc ? Hl : nullptr, B, T));
      else GN_TRY(latent_attention(m, b, a, l, H, O));
    } else {
    // q, k, v projections as one GEMM against [c_q; c_k; c_v]
    Partials qkv_part;
    { GemmArgs g; g.A = H; g.lda = d; g.B = m->p(o.qkv); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = d; g.b_trans = 1; g.C = QKV; g.ldc = W; g.M = (int)rows; g.N = W; g.K = d;
      if (fuse) g.leave = &qkv_part;
      if (tc) { g.a_hi = Hh; g.a_lo = Hl; } GN_TRY(gemm(m, g)); }
    QkvPost qp;
    qp.qkv = QKV; qp.H = H; qp.ids = a.ids;
    if (qkv_part.on() && qkv_part.ptr != QKV) qp.part = qkv_part;
    qp.ve_table = o.has_ve ? m->p(o.ve) : nullptr; qp.ve_gate = o.has_ve ? m->p(o.ve_gate) : nullptr;
    qp.cosv = m->cosb.f(); qp.sinv = m->sinb.f();
    qp.qk_rot = train ? b.layers[l].QKROT : nullptr; qp.ve_sig = train ? b.layers[l].VESIG : nullptr;
    if (cached) {
      qp.kcache = m->cache.f() + (int64_t)(2 * l) * layer_stride; qp.vcache = m->cache.f() + (int64_t)(2 * l + 1) * layer_stride;
      qp.pos = m->pos.i(); qp.cache_row_mul = a.cache_row_mul; qp.max_seq = a.max_seq;
    }
    qp.B = B; qp.T = T; qp.Hq = Hq; qp.Hkv = Hkv; qp.D = D; qp.R = m->R; qp.d = d;
    GN_TRY(qkv_post_launch(qp, s));
    if (a.mode == MODE_DECODE) {
      int splits = attention_decode_splits(B, Hkv, a.max_seq);
      o_split = tc && Hq * D <= 4 * d;
      GN_TRY(attention_decode_launch(QKV, W, m->cache.f() + (int64_t)(2 * l) * layer_stride, m->cache.f() + (int64_t)(2 * l + 1) * layer_stride,
                                     (int64_t)Hkv * a.max_seq * D, (int64_t)a.max_seq * D, m->ctxlen.i(), B, Hq, Hkv, D, m->windows[l], O,
                                     (int64_t)Hq * D, m->part_acc.f(), m->part_ms.f(), splits, s, o_split ? b.S4h : nullptr, o_split ? b.S4l : nullptr,
                                     a.group, a.prefix_len));
    } else {
      AttnShape sh;
      sh.B = B; sh.Hq = Hq; sh.Hkv = Hkv; sh.D = D; sh.Tq = T; sh.Tk = T;
      sh.q_bstride = (int64_t)T * W; sh.q_tstride = W; sh.kv_bstride = (int64_t)T * W; sh.kv_tstride = W; sh.kv_hstride = D;
      sh.o_bstride = (int64_t)T * Hq * D; sh.o_tstride = (int64_t)Hq * D; sh.window = m->windows[l]; sh.offset0 = 0; sh.tensor = m->ctx->gemm_kind == 1;
      GN_TRY(attention_forward_launch(sh, QKV, QKV + (int64_t)Hq * D, QKV + (int64_t)(Hq + Hkv) * D, O, train ? b.layers[l].LSE : nullptr, s));
    }
    }
    if (fuse) {
      // MID = Xin + O Wo^T, summed and normalised in one kernel (H is free after qkv_post and takes an unsplit product)
      Partials op;
      { GemmArgs g; g.A = O; g.lda = (int64_t)Hq * D; g.B = m->p(o.proj); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = (int64_t)Hq * D; g.b_trans = 1; g.C = H; g.ldc = d; g.M = (int)rows; g.N = d; g.K = Hq * D;
        g.leave = &op; if (o_split) { g.a_hi = b.S4h; g.a_lo = b.S4l; } GN_TRY(gemm(m, g)); }
      SumNorm sn; sn.R = Xin; sn.part = op; sn.V = MID; sn.Y = Mn; sn.Yh = Mh; sn.Yl = Ml; sn.rows = rows; sn.d = d;
      GN_TRY(sum_norm_launch(sn, s));
    } else {
      // MID = Xin + O Wo^T
      { GemmArgs g; g.A = O; g.lda = (int64_t)Hq * D; g.B = m->p(o.proj); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = (int64_t)Hq * D; g.b_trans = 1; g.C = MID; g.ldc = d; g.M = (int)rows; g.N = d; g.K = Hq * D;
        g.epilogue = EPI_RESIDUAL; g.aux = Xin; g.ldaux = d; if (o_split) { g.a_hi = b.S4h; g.a_lo = b.S4l; } GN_TRY(gemm(m, g)); }
      GN_TRY(norm_launch(MID, Mn, tc ? Mh : nullptr, tc ? Ml : nullptr, rows, d, s));
    }
    if (m->moe()) {
      if (train) {
        GN_TRY(moe_ffn_train(m, b.layers[l], *b.lws, l, Mn, tc ? Mh : nullptr, tc ? Ml : nullptr, MID, XOUT, rows));
        if (l == L / 2) backout = XOUT;
      } else {
        GN_TRY(moe_ffn(m, b, a, l, Mn, MID, XOUT));
        if (l == L / 2) { GN_CUDA(cudaMemcpyAsync(b.BO, XOUT, sizeof(float) * rows * d, cudaMemcpyDeviceToDevice, s)); backout = b.BO; }
      }
      x_prev = XOUT;
      continue;
    }
    // HID = relu(M Wfc^T)^2   (training also keeps the pre-activation)
    { GemmArgs g; g.A = Mn; g.lda = d; g.B = m->p(o.fc); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = d; g.b_trans = 1; g.C = HID; g.ldc = 4 * d; g.M = (int)rows; g.N = 4 * d; g.K = d;
      g.epilogue = EPI_RELU2; g.aux = U; g.ldaux = 4 * d;
      if (tc) { g.a_hi = Mh; g.a_lo = Ml; g.c_hi = Ph; g.c_lo = Pl; } GN_TRY(gemm(m, g)); }
    // XOUT = MID + HID Wp^T.  When fused the sum is taken by the next layer's mix (or the final norm);
    // a layer whose output is also the backout tap of the last layer is materialised.
    const bool fuse_out = fuse && !(l == L / 2 && l == L - 1);
    if (fuse_out) {
      // Mn was consumed by the product above and takes an unsplit product
      GemmArgs g; g.A = HID; g.lda = 4 * d; g.B = m->p(o.mproj); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = 4 * d; g.b_trans = 1; g.C = Mn; g.ldc = d; g.M = (int)rows; g.N = d; g.K = 4 * d;
      g.leave = &pending; g.a_hi = Ph; g.a_lo = Pl; GN_TRY(gemm(m, g));
      x_prev = MID;   // the residual the pending product is added to
    } else {
      { GemmArgs g; g.A = HID; g.lda = 4 * d; g.B = m->p(o.mproj); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = 4 * d; g.b_trans = 1; g.C = XOUT; g.ldc = d; g.M = (int)rows; g.N = d; g.K = 4 * d;
        g.epilogue = EPI_RESIDUAL; g.aux = MID; g.ldaux = d;
        if (tc) { g.a_hi = Ph; g.a_lo = Pl; } GN_TRY(gemm(m, g)); }
      if (l == L / 2) {
        if (train) backout = XOUT;
        else { GN_CUDA(cudaMemcpyAsync(b.BO, XOUT, sizeof(float) * rows * d, cudaMemcpyDeviceToDevice, s)); backout = b.BO; }
      }
      x_prev = XOUT;
    }
  }
  // final: y = norm(x - lambda_b * backout); logits = softcap(y W_lm^T)[:, :V]
  int64_t lrows = rows;
  const int32_t* sel = nullptr;
  if (a.mode == MODE_PREFILL) { lrows = B; sel = m->sel.i(); }
  const bool tc_head = m->ctx->gemm_kind == 1;
  if (pending.on()) {
    SumNorm sn; sn.R = x_prev; sn.part = pending; sn.sel = sel; sn.BO = backout; sn.lambda_b = m->p(m->off_backout);
    sn.Y = b.Y; sn.Yh = b.S1h; sn.Yl = b.S1l; sn.rows = lrows; sn.d = d;
    GN_TRY(sum_norm_launch(sn, s));
  } else {
    GN_TRY(backout_norm_launch(x_prev, backout, m->p(m->off_backout), sel, train ? b.FP : nullptr, b.Y, tc_head ? b.S1h : nullptr, tc_head ? b.S1l : nullptr, lrows, d, s));
  }
  if (a.skip_head) return GN_OK;
  { GemmArgs g; g.A = b.Y; g.lda = d; g.B = m->p(m->off_lm); g.b_static = 1; g.b_prefetch = prefetch; g.ldb = d; g.b_trans = 1; g.C = b.LOGITS; g.ldc = V; g.M = (int)lrows; g.N = V; g.K = d;
    g.epilogue = EPI_SOFTCAP; g.scalar = kSoftcap;
    if (tc_head) { g.a_hi = b.S1h; g.a_lo = b.S1l; } GN_TRY(gemm(m, g)); }
  return GN_OK;
}

// ----------------------------------------------------------------- backward
struct BwdBufs { float *DFP, *DY, *CUR, *DX0, *DOUT, *DU, *DM, *DMID, *DO, *DQKV, *DH, *DXIN, *DELTA, *DPRE, *DE; };

size_t bwd_floats(gn_model* m, int64_t rows, int B, int T) {
  const int64_t d = m->d, W = m->W, Hq = m->Hq, Hkv = m->Hkv, D = m->D;
  auto r = [](int64_t n) { return (n + 63) / 64 * 64; };
  return r(rows * d) * 9 + r(rows * 4 * d) + r(rows * Hq * D) + r(rows * W) + r((int64_t)B * Hq * T) + r(rows * Hkv);
}
void carve_bwd(gn_model* m, float* base, BwdBufs& w, int64_t rows, int B, int T) {
  const int64_t d = m->d, W = m->W, Hq = m->Hq, Hkv = m->Hkv, D = m->D;
  auto r = [](int64_t n) { return (n + 63) / 64 * 64; };
  float* p = base;
  auto take = [&](int64_t n) { float* q = p; p += r(n); return q; };
  w.DFP = take(rows * d); w.DY = take(rows * d); w.CUR = take(rows * d); w.DX0 = take(rows * d); w.DOUT = take(rows * d);
  w.DM = take(rows * d); w.DMID = take(rows * d); w.DH = take(rows * d); w.DXIN = take(rows * d);
  w.DU = take(rows * 4 * d); w.DO = take(rows * Hq * D); w.DQKV = take(rows * W); w.DELTA = take((int64_t)B * Hq * T); w.DPRE = take(rows * Hkv);
  w.DE = w.DY;  // free again by the time the embedding gradient is formed
}

int backward_core(gn_model* m, FwdBufs& b, BwdBufs& w, const int32_t* ids, int B, int T, bool head_done) {
  const int d = m->d, W = m->W, Hq = m->Hq, Hkv = m->Hkv, D = m->D, V = m->V, L = m->L;
  const int64_t rows = (int64_t)B * T;
  const int64_t n = rows * d;
  cudaStream_t s = m->s();
  double* sacc = (double*)m->sacc.p;
  float* DZ = b.LOGITS;  // the loss kernel turned the logits into dz in place
  // lm_head: dW[:V] += dz^T y ; dy = dz W[:V]      (model/layers/linear.go:45-53); already done in row chunks when head_done
  if (!head_done) {
  { GemmArgs g; g.A = DZ; g.lda = V; g.a_trans = 1; g.B = b.Y; g.ldb = d; g.b_trans = 0; g.b_hi = b.S1h; g.b_lo = b.S1l; g.C = m->g(m->off_lm); g.ldc = d; g.M = V; g.N = d; g.K = (int)rows;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = DZ; g.lda = V; g.a_reuse = 1; g.B = m->p(m->off_lm); g.b_static = 1; g.ldb = d; g.b_trans = 0; g.C = w.DY; g.ldc = d; g.M = (int)rows; g.N = d; g.K = V; GN_TRY(gemm(m, g)); }
  }
  GN_TRY(rmsnorm_backward_launch(w.DFP, b.FP, w.DY, nullptr, rows, d, kNormEps, s));
  const float* backout = b.layers[L / 2].XOUT;
  GN_TRY(dot_accumulate_launch(w.DFP, backout, n, -1.0, sacc + 2 * L + 1, s));   // d lambda_b (train_transformer.go:181-190)
  const float* cur = w.DFP;
  for (int l = L - 1; l >= 0; --l) {
    const LayerOffsets& o = m->lo[l];
    LayerSaved& sv = b.layers[l];
    const float* dout = cur;
    if (l == L / 2) {
      // the backout branch joins here: dout = cur + (-lambda_b) * dFP
      GN_CUDA(cudaMemcpyAsync(w.DOUT, cur, sizeof(float) * n, cudaMemcpyDeviceToDevice, s));
      GN_TRY(axpy_launch(w.DOUT, w.DFP, 0.0f, m->p(m->off_backout), -1.0f, 1, n, s));
      dout = w.DOUT;
    }
    if (m->moe()) {
      // ---- shared SwiGLU expert + routed experts (model/train.go:505-514,560-566, model/moe.go:203-267)
      GN_TRY(moe_ffn_backward(m, sv, *b.lws, l, sv.M, dout, w.DM, rows, T));
    } else {
    // ---- MLP backward (model/train.go:505-514)
    { GemmArgs g; g.A = dout; g.lda = d; g.a_trans = 1; g.B = sv.HID; g.ldb = 4 * d; g.b_hi = sv.Ph; g.b_lo = sv.Pl; g.C = m->g(o.mproj); g.ldc = 4 * d; g.M = d; g.N = 4 * d; g.K = (int)rows;
      g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = dout; g.lda = d; g.a_reuse = 1; g.B = m->p(o.mproj); g.b_static = 1; g.ldb = 4 * d; g.C = w.DU; g.ldc = 4 * d; g.M = (int)rows; g.N = 4 * d; g.K = d;
      g.epilogue = EPI_RELU2_BWD; g.aux = sv.U; g.ldaux = 4 * d; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = w.DU; g.lda = 4 * d; g.a_trans = 1; g.B = sv.M; g.ldb = d; g.b_hi = sv.Mh; g.b_lo = sv.Ml; g.C = m->g(o.fc); g.ldc = d; g.M = 4 * d; g.N = d; g.K = (int)rows;
      g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = w.DU; g.lda = 4 * d; g.a_reuse = 1; g.B = m->p(o.fc); g.b_static = 1; g.ldb = d; g.C = w.DM; g.ldc = d; g.M = (int)rows; g.N = d; g.K = 4 * d; GN_TRY(gemm(m, g)); }
    }
    GN_TRY(rmsnorm_backward_launch(w.DMID, sv.MID, w.DM, dout, rows, d, kNormEps, s));
    // ---- attention backward (model/train.go:198-427)
    { GemmArgs g; g.A = w.DMID; g.lda = d; g.a_trans = 1; g.B = sv.O; g.ldb = (int64_t)Hq * D; g.C = m->g(o.proj); g.ldc = (int64_t)Hq * D; g.M = d; g.N = Hq * D; g.K = (int)rows;
      g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = w.DMID; g.lda = d; g.a_reuse = 1; g.B = m->p(o.proj); g.b_static = 1; g.ldb = (int64_t)Hq * D; g.C = w.DO; g.ldc = (int64_t)Hq * D; g.M = (int)rows; g.N = Hq * D; g.K = d; GN_TRY(gemm(m, g)); }
    AttnShape sh;
    sh.B = B; sh.Hq = Hq; sh.Hkv = Hkv; sh.D = D; sh.Tq = T; sh.Tk = T;
    sh.q_bstride = (int64_t)T * W; sh.q_tstride = W; sh.kv_bstride = (int64_t)T * W; sh.kv_tstride = W; sh.kv_hstride = D;
    sh.o_bstride = (int64_t)T * Hq * D; sh.o_tstride = (int64_t)Hq * D; sh.window = m->windows[l]; sh.offset0 = 0; sh.tensor = m->ctx->gemm_kind == 1;
    GN_TRY(attention_backward_launch(sh, sv.QKV, sv.QKV + (int64_t)Hq * D, sv.QKV + (int64_t)(Hq + Hkv) * D, sv.O, w.DO, sv.LSE, nullptr, w.DQKV,
                                     w.DQKV + (int64_t)Hq * D, w.DQKV + (int64_t)(Hq + Hkv) * D, 0, w.DELTA, s));
    if (m->mla()) {
      // inverse rotation, the up-projections into the two latents and the four projections of H (model/mla.go:126-146)
      GN_TRY(latent_attention_backward(m, sv, *b.lws, l, sv.H, w.DQKV, w.DH, B, T));
    } else {
    QkvPostBwd qb;
    qb.dqkv = w.DQKV; qb.qk_rot = sv.QKROT; qb.ve_sig = sv.VESIG; qb.ve_table = o.has_ve ? m->p(o.ve) : nullptr; qb.ids = ids;
    qb.ve_grad = o.has_ve ? m->g(o.ve) : nullptr; qb.dpre = w.DPRE; qb.cosv = m->cosb.f(); qb.sinv = m->sinb.f();
    qb.B = B; qb.T = T; qb.Hq = Hq; qb.Hkv = Hkv; qb.D = D; qb.R = m->R;
    GN_TRY(qkv_post_backward_launch(qb, s));
    { GemmArgs g; g.A = w.DQKV; g.lda = W; g.a_trans = 1; g.B = sv.H; g.ldb = d; g.b_hi = sv.Hh; g.b_lo = sv.Hl; g.C = m->g(o.qkv); g.ldc = d; g.M = W; g.N = d; g.K = (int)rows;
      g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = w.DQKV; g.lda = W; g.a_reuse = 1; g.B = m->p(o.qkv); g.b_static = 1; g.ldb = d; g.C = w.DH; g.ldc = d; g.M = (int)rows; g.N = d; g.K = W; GN_TRY(gemm(m, g)); }
    if (o.has_ve) GN_TRY(ve_gate_backward_launch(w.DPRE, sv.H, m->p(o.ve_gate), m->g(o.ve_gate), w.DH, rows, Hkv, d, s));
    }
    GN_TRY(rmsnorm_backward_launch(w.DXIN, sv.Xin, w.DH, w.DMID, rows, d, kNormEps, s));
    // ---- residual mix (model/train_transformer.go:218-242)
    const float* prevX = (l == 0) ? b.X0 : b.layers[l - 1].XOUT;
    GN_TRY(mix_backward_launch(w.DXIN, prevX, b.X0, m->p(m->off_rho), m->p(m->off_chi), l, w.CUR, w.DX0, l == L - 1, sacc + l, sacc + L + l, n, s));
    cur = w.CUR;
  }
  GN_TRY(ew_launch(EW_ADD, w.CUR, w.CUR, w.DX0, 0.0f, n, s));
  GN_TRY(smear_backward_launch(w.CUR, b.X0, b.E, b.SIG, m->p(m->off_smear_gate), m->p(m->off_smear_lambda), w.DE, m->g(m->off_smear_gate), sacc + 2 * L,
                               B, T, d, s));
  GN_TRY(embed_backward_launch(ids, m->p(m->off_wte), w.DE, m->g(m->off_wte), rows, d, s));
  return GN_OK;
}

}  // namespace

// =========================================================================
extern "C" {

int gn_ctx_create(int device, void* stream, gn_ctx** out) {
  GN_REQUIRE(out, "gn_ctx_create: null out");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) { set_error("no CUDA device: %s", cudaGetErrorString(e)); return GN_ERR_CUDA; }
  GN_REQUIRE(device >= 0 && device < count, "device %d outside [0,%d)", device, count);
  GN_CUDA(cudaSetDevice(device));
  gn_ctx* c = new gn_ctx();
  c->device = device;
  if (stream) { c->stream = (cudaStream_t)stream; c->own_stream = false; }
  else { GN_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)); c->own_stream = true; }
  c->gemm_kind = gemm_default_kind();
  c->use_graphs = true;
  *out = c;
  return GN_OK;
}
int gn_ctx_destroy(gn_ctx* c) {
  if (!c) return GN_OK;
  cudaSetDevice(c->device);
  gn_ctx_comm_destroy(c);
  gemm_release_stream(c->stream);
  if (c->own_stream) cudaStreamDestroy(c->stream);
  delete c;
  return GN_OK;
}
int gn_ctx_sync(gn_ctx* c) { GN_REQUIRE(c, "null ctx"); GN_CUDA(cudaSetDevice(c->device)); GN_CUDA(cudaStreamSynchronize(c->stream)); return GN_OK; }
int gn_ctx_launch_count(gn_ctx* c, int64_t* out) { GN_REQUIRE(out, "null out"); *out = launch_count(); return GN_OK; }
int gn_ctx_set_option(gn_ctx* c, const char* name, int value) {
  GN_REQUIRE(name, "gn_ctx_set_option: null name");
  const std::string n = name;
  if (n == "decode_prefix_sharing") { attention_decode_prefix_mode(value); return GN_OK; }
#ifdef GN_HAVE_TCGEN05
  if (n == "attention_tcgen05") { attention_tc_enable(value); return GN_OK; }
#endif
  if (c) ++c->option_generation;
  if (c && n == "decode_graph") { c->use_graphs = value != 0; return GN_OK; }
  if (c && n == "optimizer_graph") { c->optimizer_graph = value != 0; return GN_OK; }
  if (c && n == "optimizer_lanes") { GN_REQUIRE(value >= 1 && value <= 4, "optimizer_lanes must be 1..4"); c->optimizer_lanes = value; return GN_OK; }
  if (c && n == "head_chunk_rows") { GN_REQUIRE(value >= 1, "head_chunk_rows must be positive"); c->head_chunk_rows = value; return GN_OK; }
  cudaStream_t s = nullptr;
  if (c) { GN_CUDA(cudaSetDevice(c->device)); s = c->stream; }
  else { s = tier_a_stream_or_null(); GN_REQUIRE(s != nullptr, "gn_ctx_set_option(NULL, ...): no stand-alone call has run yet"); }
  return gemm_set_option(s, name, value);
}
int gn_ctx_set_gemm(gn_ctx* c, int kind) { GN_REQUIRE(c && (kind == 0 || kind == 1), "gemm kind must be 0 or 1"); c->gemm_kind = kind; ++c->option_generation; return GN_OK; }

int gn_model_create(gn_ctx* ctx, const gn_config* cfg, gn_model** out) {
  GN_REQUIRE(ctx && cfg && out, "gn_model_create: null argument");
  GN_REQUIRE(cfg->n_head > 0 && cfg->n_kv_head > 0 && cfg->embed_dim % cfg->n_head == 0, "embed_dim %d not divisible by n_head %d", cfg->embed_dim, cfg->n_head);
  GN_REQUIRE(cfg->n_head % cfg->n_kv_head == 0, "n_head %d not divisible by n_kv_head %d", cfg->n_head, cfg->n_kv_head);
  GN_REQUIRE(cfg->n_layer > 0 && cfg->vocab_size > 11 && cfg->sequence_len > 0, "bad layer/vocab/sequence configuration");
  GN_CUDA(cudaSetDevice(ctx->device));
  gn_model* m = new gn_model();
  m->ctx = ctx; m->cfg = *cfg;
  m->d = cfg->embed_dim; m->L = cfg->n_layer; m->Hq = cfg->n_head; m->Hkv = cfg->n_kv_head; m->D = m->d / m->Hq;
  m->R = cfg->rotary_dims <= 0 ? m->D : cfg->rotary_dims;     // model/config.go:430-444
  m->V = cfg->vocab_size; m->Vp = (m->V + 63) / 64 * 64;      // model/config.go:619-624
  m->W = (m->Hq + 2 * m->Hkv) * m->D; m->KV = m->Hkv * m->D;
  if (cfg->n_experts > 0) {   // model/config.go:137-229
    m->E = cfg->n_experts;
    m->topk = std::min(cfg->experts_per_token <= 0 ? 2 : cfg->experts_per_token, m->E);
    m->eh = cfg->expert_hidden > 0 ? cfg->expert_hidden : m->d;
    m->sh = cfg->shared_hidden > 0 ? cfg->shared_hidden : m->eh;
    m->moe_clamp = cfg->moe_clamp == 0.0f ? 10.0f : cfg->moe_clamp;
    m->moe_scale = cfg->moe_scale == 0.0f ? 1.0f : cfg->moe_scale;
    if (m->E > 64 || m->topk > 8) { set_error("unsupported expert count %d / experts per token %d (limits 64 / 8)", m->E, m->topk); delete m; return GN_ERR_INVALID; }
  }
  if (cfg->mla_latent > 0) {  // model/config.go:249-280
    m->lat = cfg->mla_latent;
    if (cfg->mla_rotary_dims > 0) m->rope = cfg->mla_rotary_dims;
    else { m->rope = std::min(m->D / 2, 64); if (m->rope % 2) --m->rope; }
    m->content = m->D - m->rope;
    if (m->rope % 2 != 0 || m->rope > 64 || m->content <= 0 || m->lat > 512) {
      set_error("unsupported latent attention geometry: latent %d, rotary %d, head_dim %d", m->lat, m->rope, m->D); delete m; return GN_ERR_INVALID;
    }
    m->R = m->rope;           // model/config.go:430-433: the rotary table has the decoupled rotary width
  }
  if (m->D > 128 || m->R > m->D || m->R % 2 != 0 || m->d < kSmearChannels) { set_error("unsupported head_dim %d / rotary %d / embed %d", m->D, m->R, m->d); delete m; return GN_ERR_INVALID; }
  // model/config.go:629-645 (integer division truncating toward zero, as in Go)
  std::string pattern = cfg->window_pattern[0] ? std::string(cfg->window_pattern, strnlen(cfg->window_pattern, 16)) : std::string("L");
  int longw = cfg->sequence_len, shortw = -((-cfg->sequence_len / 4) / 128) * 128;
  m->windows.assign(m->L, longw);
  for (int l = 0; l < m->L; ++l) { char c = pattern[l % pattern.size()]; m->windows[l] = (c == 'S' || c == 's') ? shortw : longw; }
  m->windows[m->L - 1] = longw;
  build_layout(m);
  int st = m->P.ensure(sizeof(float) * m->total);
  if (st == GN_OK) st = m->G.ensure(sizeof(float) * m->total);
  if (st == GN_OK) st = m->sacc.ensure(sizeof(double) * (2 * m->L + 2));
  if (st != GN_OK) { delete m; return st; }
  GN_CUDA(cudaMemsetAsync(m->P.p, 0, sizeof(float) * m->total, ctx->stream));
  GN_CUDA(cudaMemsetAsync(m->G.p, 0, sizeof(float) * m->total, ctx->stream));
  GN_CUDA(cudaMemsetAsync(m->sacc.p, 0, sizeof(double) * (2 * m->L + 2), ctx->stream));
  // rotary tables in float64 -> float32 (model/rotary.go:16-30), sequence_len*10 positions
  int half = m->R / 2; int64_t seq = (int64_t)cfg->sequence_len * 10;
  std::vector<float> c((size_t)seq * half), sn((size_t)seq * half);
  for (int64_t p = 0; p < seq; ++p)
    for (int j = 0; j < half; ++j) {
      double inv = std::pow(100000.0, -2.0 * (double)j / (double)m->R);
      double f = (double)p * inv;
      c[(size_t)p * half + j] = (float)std::cos(f); sn[(size_t)p * half + j] = (float)std::sin(f);
    }
  GN_TRY(m->cosb.ensure(sizeof(float) * c.size())); GN_TRY(m->sinb.ensure(sizeof(float) * sn.size()));
  GN_CUDA(cudaMemcpyAsync(m->cosb.p, c.data(), sizeof(float) * c.size(), cudaMemcpyHostToDevice, ctx->stream));
  GN_CUDA(cudaMemcpyAsync(m->sinb.p, sn.data(), sizeof(float) * sn.size(), cudaMemcpyHostToDevice, ctx->stream));
  for (int i = 0; i < 4; ++i) GN_CUDA(cudaEventCreate(&m->ev[i]));
  GN_CUDA(cudaStreamSynchronize(ctx->stream));
  *out = m;
  return GN_OK;
}

int gn_model_destroy(gn_model* m) {
  if (!m) return GN_OK;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  gemm_invalidate_static();   // cached splits are keyed by addresses that are about to be freed
  DevBuf* bufs[] = {&m->P, &m->G, &m->cosb, &m->sinb, &m->sacc, &m->cache, &m->prev, &m->pos, &m->ctxlen, &m->ids_dev, &m->sampled, &m->seeds,
                    &m->out_tokens, &m->out_lengths, &m->out_masks, &m->engine_state, &m->done, &m->n_done, &m->sel, &m->part_acc, &m->part_ms, &m->step_dev, &m->infer.buf, &m->train.buf,
                    &m->tgt_dev, &m->adv_dev, &m->rowloss, &m->loss_dev, &m->in_dev, &m->lat_ws, &m->cache_lat, &m->cache_rope, &m->opt_mom, &m->opt_second,
                    &m->opt_ws};
  for (DevBuf* b : bufs) b->release();
  for (int l = 1; l < gn_model::kOptLanes; ++l) {
    m->opt_ws_lane[l].release();
    if (m->opt_stream[l]) { cudaStreamSynchronize(m->opt_stream[l]); gemm_release_stream(m->opt_stream[l]); cudaStreamDestroy(m->opt_stream[l]); }
  }
  if (m->opt_graph_exec) cudaGraphExecDestroy(m->opt_graph_exec);
  if (m->opt_graph) cudaGraphDestroy(m->opt_graph);
  for (int l = 0; l <= gn_model::kOptLanes; ++l) if (m->opt_event[l]) cudaEventDestroy(m->opt_event[l]);
  for (int i = 0; i < 4; ++i) if (m->ev[i]) cudaEventDestroy(m->ev[i]);
  delete m;
  return GN_OK;
}

int gn_model_param_count(gn_model* m, int* out) { GN_REQUIRE(m && out, "null argument"); *out = (int)m->params.size(); return GN_OK; }
int gn_model_param_info(gn_model* m, int i, const char** name, int* rows, int* cols) {
  GN_REQUIRE(m && i >= 0 && i < (int)m->params.size(), "parameter index %d out of range", i);
  if (name) *name = m->params[i].name.c_str();
  if (rows) *rows = m->params[i].rows;
  if (cols) *cols = m->params[i].cols;
  return GN_OK;
}
static int find_param(gn_model* m, const char* name, int64_t n, const ParamInfo** out) {
  GN_REQUIRE(m && name, "null argument");
  auto it = m->index.find(name);
  GN_REQUIRE(it != m->index.end(), "unknown parameter '%s'", name);
  const ParamInfo& pi = m->params[it->second];
  GN_REQUIRE(n == (int64_t)pi.rows * pi.cols, "parameter '%s' has %lld elements, got %lld", name, (long long)pi.rows * pi.cols, (long long)n);
  *out = &pi;
  return GN_OK;
}
int gn_model_upload(gn_model* m, const char* name, const float* host, int64_t n) {
  const ParamInfo* pi; GN_TRY(find_param(m, name, n, &pi)); GN_TRY(enter(m));
  GN_CUDA(cudaMemcpyAsync(m->p(pi->offset), host, sizeof(float) * n, cudaMemcpyHostToDevice, m->s()));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  m->weights_dirty = true;
  return GN_OK;
}
int gn_model_download(gn_model* m, const char* name, float* host, int64_t n) {
  const ParamInfo* pi; GN_TRY(find_param(m, name, n, &pi)); GN_TRY(enter(m));
  GN_CUDA(cudaMemcpyAsync(host, m->p(pi->offset), sizeof(float) * n, cudaMemcpyDeviceToHost, m->s()));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  return GN_OK;
}
int gn_model_download_grad(gn_model* m, const char* name, float* host, int64_t n) {
  const ParamInfo* pi; GN_TRY(find_param(m, name, n, &pi)); GN_TRY(enter(m));
  GN_CUDA(cudaMemcpyAsync(host, m->g(pi->offset), sizeof(float) * n, cudaMemcpyDeviceToHost, m->s()));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  return GN_OK;
}
int gn_model_upload_grad(gn_model* m, const char* name, const float* host, int64_t n) {
  const ParamInfo* pi; GN_TRY(find_param(m, name, n, &pi)); GN_TRY(enter(m));
  GN_CUDA(cudaMemcpyAsync(m->g(pi->offset), host, sizeof(float) * n, cudaMemcpyHostToDevice, m->s()));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  return GN_OK;
}
int gn_model_zero_grad(gn_model* m) {
  GN_TRY(enter(m));
  GN_CUDA(cudaMemsetAsync(m->G.p, 0, sizeof(float) * m->total, m->s()));
  GN_CUDA(cudaMemsetAsync(m->sacc.p, 0, sizeof(double) * (2 * m->L + 2), m->s()));
  return GN_OK;
}
int gn_model_grad_buffer(gn_model* m, float** ptr, int64_t* n) { GN_REQUIRE(m && ptr && n, "null argument"); *ptr = m->G.f(); *n = m->total; return GN_OK; }
int gn_model_param_buffer(gn_model* m, float** ptr, int64_t* n) { GN_REQUIRE(m && ptr && n, "null argument"); *ptr = m->P.f(); *n = m->total; return GN_OK; }
int gn_model_checksum(gn_model* m, double* psum, double* gsum) {
  GN_TRY(enter(m));
  std::vector<float> h((size_t)m->total);
  for (int which = 0; which < 2; ++which) {
    GN_CUDA(cudaMemcpyAsync(h.data(), which ? m->G.p : m->P.p, sizeof(float) * m->total, cudaMemcpyDeviceToHost, m->s()));
    GN_CUDA(cudaStreamSynchronize(m->s()));
    double acc = 0; for (float v : h) acc += std::fabs((double)v);
    if (which == 0 && psum) *psum = acc;
    if (which == 1 && gsum) *gsum = acc;
  }
  return GN_OK;
}

int gn_model_forward(gn_model* m, const int32_t* ids, int B, int T, float* logits) {
  GN_TRY(enter_compute(m));
  GN_REQUIRE(ids && logits && B > 0 && T > 1, "gn_model_forward needs ids, logits, batch > 0 and seq > 1");
  GN_REQUIRE(T <= m->cfg.sequence_len, "sequence %d longer than the rotary cache (%d)", T, m->cfg.sequence_len);
  const int64_t rows = (int64_t)B * T;
  GN_TRY(check_ids(ids, rows, m->V, false, "gn_model_forward: ids"));
  GN_TRY(m->ids_dev.ensure(sizeof(int32_t) * rows));
  GN_CUDA(cudaMemcpyAsync(m->ids_dev.p, ids, sizeof(int32_t) * rows, cudaMemcpyHostToDevice, m->s()));
  FwdBufs b;
  GN_TRY(make_bufs(m, m->infer, b, MODE_PLAIN, rows, rows, B, T, 0, nullptr));
  FwdArgs a; a.mode = MODE_PLAIN; a.ids = m->ids_dev.i(); a.B = B; a.T = T;
  if (m->mla()) {
    // model/transformer.go:248-253: a cache-less forward of a latent-attention model runs over a scratch latent cache
    GN_TRY(m->cache_lat.ensure(sizeof(float) * (size_t)m->L * rows * m->lat));
    GN_TRY(m->cache_rope.ensure(sizeof(float) * (size_t)m->L * rows * m->Hkv * m->rope));
    GN_TRY(m->pos.ensure(sizeof(int32_t) * B));
    GN_CUDA(cudaMemsetAsync(m->pos.p, 0, sizeof(int32_t) * B, m->s()));
    a.cache_rows = B; a.cache_row_mul = 1; a.max_seq = T;
  }
  GN_TRY(forward_core(m, b, a));
  GN_CUDA(cudaMemcpyAsync(logits, b.LOGITS, sizeof(float) * rows * m->V, cudaMemcpyDeviceToHost, m->s()));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  return gemm_check_error(m->s());
}

// ---------------------------------------------------------------- optimizer
int gn_model_optimizer_init(gn_model* m, const gn_optimizer_config* cfg) {
  GN_TRY(enter(m));
  GN_REQUIRE(cfg, "gn_model_optimizer_init: null config");
  m->opt_cfg = *cfg; m->opt_steps = 0;
  // the learning rates are arguments of the captured launches: a new configuration starts from an eager step again
  if (m->opt_graph_exec) { GN_CUDA(cudaStreamSynchronize(m->s())); cudaGraphExecDestroy(m->opt_graph_exec); cudaGraphDestroy(m->opt_graph); m->opt_graph_exec = nullptr; m->opt_graph = nullptr; }
  m->opt_eager_runs = 0; m->opt_graph_failed = false;
  GN_TRY(m->opt_mom.ensure(sizeof(float) * m->total)); GN_TRY(m->opt_second.ensure(sizeof(float) * m->total));
  GN_CUDA(cudaMemsetAsync(m->opt_mom.p, 0, sizeof(float) * m->total, m->s()));
  GN_CUDA(cudaMemsetAsync(m->opt_second.p, 0, sizeof(float) * m->total, m->s()));
  size_t ws = 0;
  for (const ParamInfo& pi : m->params) {
    const bool sink = pi.name == "lm_head.weight" || pi.name == "transformer.wte.weight" || pi.name.rfind("value_embeds.", 0) == 0;
    const bool scalar = pi.name.rfind("transformer.h.", 0) != 0 && !sink;
    const bool experts = pi.name.find(".moe.experts.") != std::string::npos;   // per-expert views (model/optimizer.go:87-93)
    if (sink) ws = std::max(ws, sinkhorn_workspace_bytes(pi.rows, pi.cols));
    else if (!scalar) ws = std::max(ws, muon_workspace_bytes(experts ? pi.rows / m->E : pi.rows, pi.cols));
  }
  GN_TRY(m->opt_ws.ensure(ws));
  for (int l = 1; l < gn_model::kOptLanes; ++l) {
    GN_TRY(m->opt_ws_lane[l].ensure(ws));
    if (!m->opt_stream[l]) GN_CUDA(cudaStreamCreateWithFlags(&m->opt_stream[l], cudaStreamNonBlocking));
  }
  for (int l = 0; l <= gn_model::kOptLanes; ++l) if (!m->opt_event[l]) GN_CUDA(cudaEventCreateWithFlags(&m->opt_event[l], cudaEventDisableTiming));
  m->opt_ready = true;
  return GN_OK;
}

// Routing: model/optimizer.go:20-165 (sinkhorn = true).  Parameters are visited in name order; the updates are
// independent of one another, so the order only fixes the launch sequence.  With shard_count > 1 only the tensors
// this shard owns are updated (ownership: greedy balance of an operation-count estimate, identical on every rank).
}  // extern "C"
namespace gnm {
std::vector<int> optimizer_owners(gn_model* m, int shard_count, const std::vector<int>* within, int within_value) {
  const size_t n = m->params.size();
  std::vector<int> owner(n, 0);
  if (shard_count <= 1) return owner;
  std::vector<std::pair<double, size_t>> cost(n);
  for (size_t i = 0; i < n; ++i) {
    const ParamInfo& pi = m->params[i];
    const double elems = (double)pi.rows * pi.cols;
    const bool sink = pi.name == "lm_head.weight" || pi.name == "transformer.wte.weight" || pi.name.rfind("value_embeds.", 0) == 0;
    const bool matrix = pi.name.rfind("transformer.h.", 0) == 0;
    // Muon: 5 iterations of three products + ~35 launches; Sinkhorn: 16 passes over the table; AdamW: nothing
    const double c = sink ? 16.0 * elems : (matrix ? 30.0 * elems * std::min(pi.rows, pi.cols) / 400.0 + 4e6 : 1.0);
    cost[i] = {c, i};
  }
  std::sort(cost.begin(), cost.end(), [](const std::pair<double, size_t>& a, const std::pair<double, size_t>& b) { return a.first != b.first ? a.first > b.first : a.second < b.second; });
  std::vector<double> load(shard_count, 0.0);
  for (auto& c : cost) {
    if (within && (*within)[c.second] != within_value) continue;
    int best = 0;
    for (int r = 1; r < shard_count; ++r) if (load[r] < load[best]) best = r;
    owner[c.second] = best; load[best] += c.first;
  }
  return owner;
}
}  // namespace gnm
extern "C" {
namespace {

// part: 0 everything, 1 all but the AdamW tensors (the part a graph can hold), 2 the AdamW tensors alone
int optimizer_body(gn_model* m, int shard, int shard_count, int part) {
  cudaStream_t s = m->s();
  const gn_optimizer_config& c = m->opt_cfg;
  const float dscale = (float)std::pow((double)m->d / 768.0, -0.5);   // model/optimizer.go:108
  const std::vector<int> owner = optimizer_owners(m, shard_count);
  // lanes: the owned tensors in cost order, each to the least loaded lane (the same cost model as the owners)
  const int lanes = std::max(1, std::min(m->ctx->optimizer_lanes, (int)gn_model::kOptLanes));
  std::vector<int> lane_of(m->params.size(), 0);
  const bool fork = lanes > 1 && part != 2;   // the few AdamW updates stay on the main stream
  if (fork) {
    const std::vector<int> by_lane = optimizer_owners(m, lanes, &owner, shard);
    lane_of = by_lane;
    GN_CUDA(cudaEventRecord(m->opt_event[0], m->s()));
    for (int l = 1; l < lanes; ++l) GN_CUDA(cudaStreamWaitEvent(m->opt_stream[l], m->opt_event[0], 0));
  }
  for (size_t i = 0; i < m->params.size(); ++i) {
    if (owner[i] != shard) continue;
    const int lane = lane_of[i];
    cudaStream_t s = lane == 0 ? m->s() : m->opt_stream[lane];
    void* lane_ws = lane == 0 ? m->opt_ws.p : m->opt_ws_lane[lane].p;
    const ParamInfo& pi = m->params[i];
    float* p = m->p(pi.offset); float* g = m->g(pi.offset);
    float* mo = m->opt_mom.f() + pi.offset; float* se = m->opt_second.f() + pi.offset;
    const int64_t n = (int64_t)pi.rows * pi.cols;
    auto sink = [&](float lr) { return sinkhorn_launch(p, g, mo, pi.rows, pi.cols, lr * c.lr_mult, 0.95f, 0.18f, 11, 1e-3f, 1e-20f, lane_ws, s); };
    auto adam = [&](float lr, float b1, float b2, float wd) { return adamw_launch(p, g, mo, se, n, m->opt_steps, lr * c.lr_mult, b1, b2, 1e-10f, wd, s); };
    const bool is_adam = pi.name == "resid_lambdas" || pi.name == "x0_lambdas" || pi.name == "smear_gate.weight" || pi.name == "smear_lambda" ||
                         pi.name == "backout_lambda";
    if ((part == 1 && is_adam) || (part == 2 && !is_adam)) continue;
    if (pi.name == "lm_head.weight") GN_TRY(sink(c.unembedding_lr * dscale));
    else if (pi.name == "transformer.wte.weight") GN_TRY(sink(c.embedding_lr * dscale));
    else if (pi.name.rfind("value_embeds.", 0) == 0) GN_TRY(sink(c.embedding_lr * dscale * 0.5f));
    else if (pi.name == "resid_lambdas") GN_TRY(adam(c.scalar_lr * 0.01f, 0.8f, 0.95f, 0.05f));
    else if (pi.name == "x0_lambdas") GN_TRY(adam(c.scalar_lr, 0.96f, 0.95f, 0.0f));
    else if (pi.name == "smear_gate.weight" || pi.name == "smear_lambda" || pi.name == "backout_lambda") GN_TRY(adam(0.2f, 0.8f, 0.95f, 0.0f));
    else if (pi.name.size() > 11 && pi.name.compare(pi.name.size() - 11, 11, "router_bias") == 0) continue;   // updated by load, never optimised (model/optimizer.go:83-86)
    else if (pi.name.find(".moe.experts.") != std::string::npos) {
      // packed expert weights: one Muon matrix per expert view (model/optimizer.go:87-93, model/moe.go:60-81)
      const int er = pi.rows / m->E;
      for (int e = 0; e < m->E; ++e) {
        const int64_t off = (int64_t)e * er * pi.cols;
        GN_TRY(muon_launch(p + off, g + off, mo + off, se + off, er, pi.cols, c.matrix_lr * c.lr_mult, 0.95f, 5, 0.9f, c.weight_decay, lane_ws, m->ctx->gemm_kind, s));
      }
    }
    else GN_TRY(muon_launch(p, g, mo, se, pi.rows, pi.cols, c.matrix_lr * c.lr_mult, 0.95f, 5, 0.9f, c.weight_decay, lane_ws, m->ctx->gemm_kind, s));
  }
  if (fork) {
    for (int l = 1; l < lanes; ++l) {
      GN_CUDA(cudaEventRecord(m->opt_event[l], m->opt_stream[l]));
      GN_CUDA(cudaStreamWaitEvent(m->s(), m->opt_event[l], 0));
    }
  }
  if (shard_count > 1 && part != 1) {   // after every update of this rank, the AdamW ones included
    // Exchange form: the gradient buffer becomes "my updated tensors, zero elsewhere"; a SUM all-reduce over it then
    // yields every updated tensor on every rank exactly (x + 0 + ... + 0), and gn_model_optimizer_finish installs it.
    for (size_t i = 0; i < m->params.size(); ++i) {
      const ParamInfo& pi = m->params[i];
      const size_t bytes = sizeof(float) * (size_t)pi.rows * pi.cols;
      if (owner[i] == shard) GN_CUDA(cudaMemcpyAsync(m->g(pi.offset), m->p(pi.offset), bytes, cudaMemcpyDeviceToDevice, s));
      else GN_CUDA(cudaMemsetAsync(m->g(pi.offset), 0, bytes, s));
    }
  }
  return GN_OK;
}

// One optimizer step.  The launch sequence is the same every step (about 2 900 launches for d12, paced by the host), except
// for the bias correction of the few AdamW tensors: the rest is captured once, after an eager step has sized every scratch
// buffer, and replayed; the AdamW tensors and the exchange copies of a sharded step follow on the main stream.
int optimizer_run(gn_model* m, int shard, int shard_count) {
  cudaStream_t s = m->s();
  ++m->opt_steps;
  const int lanes = std::max(1, std::min(m->ctx->optimizer_lanes, (int)gn_model::kOptLanes));
  const int key[5] = {shard, shard_count, lanes, m->ctx->gemm_kind, m->ctx->option_generation};
  const bool want_graph = m->ctx->optimizer_graph && !m->opt_graph_failed && m->opt_eager_runs >= 1;
  if (!want_graph) { ++m->opt_eager_runs; return optimizer_body(m, shard, shard_count, 0); }
  if (m->opt_graph_exec && std::memcmp(key, m->opt_graph_key, sizeof(key)) != 0) {
    cudaGraphExecDestroy(m->opt_graph_exec); cudaGraphDestroy(m->opt_graph); m->opt_graph_exec = nullptr; m->opt_graph = nullptr;
    ++m->opt_eager_runs;
    return optimizer_body(m, shard, shard_count, 0);   // the changed options may want other buffers: one eager step first
  }
  if (!m->opt_graph_exec) {
    GN_CUDA(cudaStreamSynchronize(s));
    for (int l = 1; l < lanes; ++l) GN_CUDA(cudaStreamSynchronize(m->opt_stream[l]));
    bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    int status = GN_OK;
    if (ok) {
      status = optimizer_body(m, shard, shard_count, 1);
      cudaGraph_t graph = nullptr;
      const cudaError_t ce = cudaStreamEndCapture(s, &graph);
      ok = status == GN_OK && ce == cudaSuccess && graph != nullptr;
      if (ok) ok = cudaGraphGetNodes(graph, nullptr, &m->opt_graph_nodes) == cudaSuccess && cudaGraphInstantiate(&m->opt_graph_exec, graph, 0) == cudaSuccess;
      if (ok) { m->opt_graph = graph; std::memcpy(m->opt_graph_key, key, sizeof(key)); }
      else if (graph) cudaGraphDestroy(graph);
    }
    if (!ok) {
      // nothing of the captured part has run: clear the error state and do this step, and every later one, eagerly
      cudaGetLastError();
      m->opt_graph_exec = nullptr; m->opt_graph_failed = true;
      return optimizer_body(m, shard, shard_count, 0);
    }
  }
  GN_CUDA(cudaGraphLaunch(m->opt_graph_exec, s));
  count_launches((int64_t)m->opt_graph_nodes);
  return optimizer_body(m, shard, shard_count, 2);
}
}  // namespace

int gn_model_optimizer_step(gn_model* m) {
  GN_TRY(enter(m));
  GN_REQUIRE(m->opt_ready, "gn_model_optimizer_step: call gn_model_optimizer_init first");
  cudaStream_t s = m->s();
  GN_CUDA(cudaEventRecord(m->ev[0], s));
  GN_TRY(optimizer_run(m, 0, 1));
  GN_CUDA(cudaMemsetAsync(m->G.p, 0, sizeof(float) * m->total, s));   // ZeroGrad (trainer/rl.go:66)
  GN_CUDA(cudaMemsetAsync(m->sacc.p, 0, sizeof(double) * (2 * m->L + 2), s));
  GN_CUDA(cudaEventRecord(m->ev[1], s));
  m->weights_dirty = true;   // cached tensor-core splits of the parameters are stale
  GN_CUDA(cudaStreamSynchronize(s));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1])); m->phase_ms["optimizer"] = ms;
  for (int l = 1; l < gn_model::kOptLanes; ++l) if (m->opt_stream[l]) GN_TRY(gemm_check_error(m->opt_stream[l]));
  return gemm_check_error(s);
}

int gn_model_optimizer_step_shard(gn_model* m, int shard, int shard_count) {
  GN_TRY(enter(m));
  GN_REQUIRE(m->opt_ready, "gn_model_optimizer_step_shard: call gn_model_optimizer_init first");
  GN_REQUIRE(shard_count >= 1 && shard >= 0 && shard < shard_count, "gn_model_optimizer_step_shard: shard %d of %d", shard, shard_count);
  cudaStream_t s = m->s();
  GN_CUDA(cudaEventRecord(m->ev[0], s));
  GN_TRY(optimizer_run(m, shard, shard_count));
  GN_CUDA(cudaEventRecord(m->ev[1], s));
  GN_CUDA(cudaStreamSynchronize(s));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1])); m->phase_ms["optimizer"] = ms;
  for (int l = 1; l < gn_model::kOptLanes; ++l) if (m->opt_stream[l]) GN_TRY(gemm_check_error(m->opt_stream[l]));
  return gemm_check_error(s);
}

int gn_model_optimizer_finish(gn_model* m) {
  GN_TRY(enter(m));
  cudaStream_t s = m->s();
  GN_CUDA(cudaEventRecord(m->ev[0], s));
  for (const ParamInfo& pi : m->params)
    GN_CUDA(cudaMemcpyAsync(m->p(pi.offset), m->g(pi.offset), sizeof(float) * (size_t)pi.rows * pi.cols, cudaMemcpyDeviceToDevice, s));
  GN_CUDA(cudaMemsetAsync(m->G.p, 0, sizeof(float) * m->total, s));   // ZeroGrad (trainer/rl.go:66)
  GN_CUDA(cudaMemsetAsync(m->sacc.p, 0, sizeof(double) * (2 * m->L + 2), s));
  GN_CUDA(cudaEventRecord(m->ev[1], s));
  m->weights_dirty = true;
  GN_CUDA(cudaStreamSynchronize(s));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1])); m->phase_ms["optimizer"] += ms;
  return GN_OK;
}

// ---------------------------------------------------------------- rollout (inference/engine.go:112-369)
namespace {

constexpr int kForcedQueue = 64;   // forced tokens a row can hold at once (a tool result plus the closing tokens)

// Prefill every prompt, replicate its cache over the group, and reset the engine's per-row state
// (inference/engine.go:141-238).  Afterwards m->ro.logits holds the prompts' last-position logits [P, V].
int rollout_begin(gn_model* m, const int32_t* prompts, int P, int plen, int G, int max_tokens, const uint64_t* seeds, const gn_generate_options* opt) {
  GN_REQUIRE(prompts && seeds, "rollout: null argument");
  GN_REQUIRE(P > 0 && plen > 0 && G > 0 && max_tokens > 0, "rollout: sizes must be positive");
  GN_REQUIRE(plen <= m->cfg.sequence_len, "prompt of %d tokens longer than sequence_len %d", plen, m->cfg.sequence_len);
  GN_REQUIRE((int64_t)plen + max_tokens <= (int64_t)m->cfg.sequence_len * 10, "context %d exceeds the rotary table", plen + max_tokens);
  GN_TRY(check_ids(prompts, (int64_t)P * plen, m->V, false, "rollout: prompts"));
  const int d = m->d, Hq = m->Hq, Hkv = m->Hkv, D = m->D, V = m->V, L = m->L;
  const int rows = P * G, max_seq = plen + max_tokens;
  cudaStream_t s = m->s();
  Rollout& ro = m->ro;
  ro = Rollout();
  ro.P = P; ro.plen = plen; ro.G = G; ro.max_tokens = max_tokens; ro.rows = rows; ro.max_seq = max_seq;
  if (opt) { ro.thinking = opt->thinking != 0 || opt->thinking_budget > 0; ro.thinking_budget = opt->thinking_budget; }
  if (m->mla()) {
    GN_TRY(m->cache_lat.ensure(sizeof(float) * (size_t)L * rows * max_seq * m->lat));
    GN_TRY(m->cache_rope.ensure(sizeof(float) * (size_t)L * rows * max_seq * Hkv * m->rope));
  } else {
    GN_TRY(m->cache.ensure(sizeof(float) * (size_t)L * 2 * rows * Hkv * max_seq * D));
  }
  m->kv_rows = rows; m->kv_max_seq = max_seq;
  GN_TRY(m->prev.ensure(sizeof(float) * (size_t)rows * d));
  GN_TRY(m->pos.ensure(sizeof(int32_t) * rows)); GN_TRY(m->ctxlen.ensure(sizeof(int32_t) * rows));
  GN_TRY(m->ids_dev.ensure(sizeof(int32_t) * std::max<int64_t>((int64_t)P * plen, rows)));
  GN_TRY(m->sampled.ensure(sizeof(int32_t) * rows)); GN_TRY(m->seeds.ensure(sizeof(uint64_t) * P));
  GN_TRY(m->out_tokens.ensure(sizeof(int32_t) * (size_t)rows * max_tokens)); GN_TRY(m->out_lengths.ensure(sizeof(int32_t) * rows));
  GN_TRY(m->out_masks.ensure(sizeof(int32_t) * (size_t)rows * max_tokens));
  GN_TRY(m->done.ensure(sizeof(int32_t) * rows)); GN_TRY(m->n_done.ensure(sizeof(int32_t)));
  GN_TRY(m->sel.ensure(sizeof(int32_t) * P));
  // engine state per row: forced-token ring (head, length, tokens), thinking flag and count, this step's mask
  GN_TRY(m->engine_state.ensure(sizeof(int32_t) * (size_t)rows * (5 + kForcedQueue)));
  GN_CUDA(cudaMemsetAsync(m->engine_state.p, 0, sizeof(int32_t) * (size_t)rows * (5 + kForcedQueue), s));
  const bool share_prefix = G > 1;
  int splits = attention_decode_splits(rows, Hkv, max_seq) + (share_prefix ? attention_decode_prefix_splits(rows, G, Hq, Hkv, D, plen) : 0);
  GN_TRY(m->part_acc.ensure(sizeof(float) * (size_t)rows * Hq * splits * D)); GN_TRY(m->part_ms.ensure(sizeof(float) * (size_t)rows * Hq * splits * 2));
  GN_CUDA(cudaMemcpyAsync(m->ids_dev.p, prompts, sizeof(int32_t) * (size_t)P * plen, cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaMemcpyAsync(m->seeds.p, seeds, sizeof(uint64_t) * P, cudaMemcpyHostToDevice, s));
  std::vector<int32_t> sel(P);
  for (int p = 0; p < P; ++p) sel[p] = p * plen + plen - 1;
  GN_CUDA(cudaMemcpyAsync(m->sel.p, sel.data(), sizeof(int32_t) * P, cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaMemsetAsync(m->pos.p, 0, sizeof(int32_t) * rows, s));
  GN_CUDA(cudaMemsetAsync(m->out_lengths.p, 0, sizeof(int32_t) * rows, s));
  GN_CUDA(cudaMemsetAsync(m->done.p, 0, sizeof(int32_t) * rows, s));
  GN_CUDA(cudaMemsetAsync(m->n_done.p, 0, sizeof(int32_t), s));
  // A prompt that already ends in <|think_start|> starts inside the trace (inference/engine.go:229-236)
  bool primed = false;
  if (ro.thinking) for (int p = 0; p < P; ++p) primed = primed || prompts[(size_t)p * plen + plen - 1] == V - 2;
  if ((opt && opt->forced && opt->forced_counts) || primed) {   // tokens queued before the first step / primed traces
    std::vector<int32_t> st((size_t)rows * (5 + kForcedQueue), 0);
    if (ro.thinking) for (int r = 0; r < rows; ++r) st[(size_t)rows * 2 + r] = prompts[(size_t)(r / G) * plen + plen - 1] == V - 2 ? 1 : 0;
    if (opt && opt->forced && opt->forced_counts)
    for (int r = 0; r < rows; ++r) {
      const int n = opt->forced_counts[r];
      GN_REQUIRE(n >= 0 && n <= kForcedQueue && n <= opt->forced_stride, "rollout: %d forced tokens for row %d (at most %d)", n, r, kForcedQueue);
      st[(size_t)rows * 1 + r] = n;
      for (int i = 0; i < n; ++i) st[(size_t)rows * 5 + (size_t)r * kForcedQueue + i] = opt->forced[(size_t)r * opt->forced_stride + i];
    }
    GN_TRY(check_ids(st.data() + (size_t)rows * 5, (int64_t)rows * kForcedQueue, V, false, "rollout: forced tokens"));
    GN_CUDA(cudaMemcpyAsync(m->engine_state.p, st.data(), sizeof(int32_t) * st.size(), cudaMemcpyHostToDevice, s));
    GN_CUDA(cudaStreamSynchronize(s));
  }
  // ---- prefill: all prompts in one batch; prompt p writes cache row p*G (engine.go:141-172)
  GN_CUDA(cudaEventRecord(m->ev[0], s));
  {
    const int64_t prow = (int64_t)P * plen;
    GN_TRY(make_bufs(m, m->infer, ro.b, MODE_PREFILL, std::max<int64_t>(prow, rows), std::max(P, rows), P, plen, 0, nullptr));
    FwdArgs a; a.mode = MODE_PREFILL; a.ids = m->ids_dev.i(); a.B = P; a.T = plen; a.cache_rows = rows; a.cache_row_mul = G; a.max_seq = max_seq;
    GN_TRY(forward_core(m, ro.b, a));
  }
  // replicate each prompt's cache over its group (engine.go:194-209, kvcache.go:383-448)
  if (m->mla()) {
    const int rw = Hkv * m->rope;
    GN_TRY(kv_replicate_launch(m->cache_lat.f(), (int64_t)rows * max_seq * m->lat, L, (int64_t)max_seq * m->lat, 0, 1, m->lat, P, G, plen, m->prev.f(), d, nullptr, s));
    GN_TRY(kv_replicate_launch(m->cache_rope.f(), (int64_t)rows * max_seq * rw, L, (int64_t)max_seq * rw, 0, 1, rw, P, G, plen, nullptr, d, nullptr, s));
  } else {
    GN_TRY(kv_replicate_launch(m->cache.f(), (int64_t)rows * Hkv * max_seq * D, 2 * L, (int64_t)Hkv * max_seq * D, (int64_t)max_seq * D, Hkv, D, P, G, plen,
                               m->prev.f(), d, nullptr, s));
  }
  GN_TRY(fill_i32_launch(m->pos.i(), plen, rows, s));
  GN_CUDA(cudaEventRecord(m->ev[1], s));
  ro.logits_row_div = G;   // every row of a group samples from its prompt's last-position logits (engine.go:182-191)
  ro.active = true;
  return GN_OK;
}

// The sampler's row CTAs also do the engine's bookkeeping: see SampleTail.
SampleTail rollout_tail(gn_model* m) {
  const Rollout& ro = m->ro;
  const int V = m->V;
  int32_t* st = m->engine_state.i();
  SampleTail t;
  t.pos = m->pos.i(); t.ctxlen = m->ctxlen.i(); t.pos_base = ro.plen; t.advance = ro.generated > 0 ? 1 : 0;
  t.out_tokens = m->out_tokens.i(); t.out_lengths = m->out_lengths.i(); t.out_masks = m->out_masks.i(); t.done = m->done.i(); t.n_done = m->n_done.i();
  t.max_tokens = ro.max_tokens; t.bos = V - 11; t.aend = V - 7;   // tokenizer/special.go:19-31
  t.forced_head = st; t.forced_len = st + ro.rows; t.in_think = st + 2 * (size_t)ro.rows; t.think_count = st + 3 * (size_t)ro.rows; t.step_mask = st + 4 * (size_t)ro.rows;
  t.forced_buf = st + 5 * (size_t)ro.rows; t.forced_cap = kForcedQueue;
  t.thinking = ro.thinking ? 1 : 0; t.thinking_budget = ro.thinking_budget; t.think_start = V - 2; t.think_end = V - 1;
  return t;
}
// One sampling step from `logits` (null: the model's own) with the engine's state machine (engine.go:256-314).
int rollout_sample(gn_model* m, const float* logits, float temperature, int top_k) {
  Rollout& ro = m->ro;
  SampleTail tail = rollout_tail(m);
  GN_TRY(sample_launch(logits ? logits : ro.b.LOGITS, ro.rows, m->V, ro.logits_row_div, nullptr, (const uint64_t*)m->seeds.p, ro.G, nullptr, 0, temperature, top_k,
                       m->sampled.i(), m->s(), &tail));
  return GN_OK;
}
// Forward the current token column through the decode cache (engine.go:321-324).
int rollout_forward(gn_model* m) {
  Rollout& ro = m->ro;
  FwdArgs a; a.mode = MODE_DECODE; a.ids = m->sampled.i(); a.B = ro.rows; a.T = 1; a.cache_rows = ro.rows; a.cache_row_mul = 1; a.max_seq = ro.max_seq;
  if (ro.G > 1 && ro.prompt_shared) { a.group = ro.G; a.prefix_len = ro.plen; }
  return forward_core(m, ro.b, a);
}

}  // namespace

int gn_generate_batch_ex(gn_model* m, const int32_t* prompts, int P, int plen, int G, int max_tokens, float temperature, int top_k, const uint64_t* seeds,
                         const gn_generate_options* opt, int32_t* out_tokens, int32_t* out_lengths, int32_t* out_masks, float* step_logits, int* steps_run) {
  GN_TRY(enter_compute(m));
  GN_REQUIRE(out_tokens && out_lengths, "gn_generate_batch: null argument");
  GN_TRY(rollout_begin(m, prompts, P, plen, G, max_tokens, seeds, opt));
  Rollout& ro = m->ro;
  const int rows = ro.rows, V = m->V;
  cudaStream_t s = m->s();
  // ---- decode loop (engine.go:241-325)
  // One iteration = forward the sampled column, then sample the next one.  The sequence of launches is identical from
  // step to step (positions and the engine state live in device memory), so after two eager iterations it is captured
  // once into a CUDA graph and replayed.  With the per-step logits tap the loop stays eager.
  std::vector<float> host_logits;
  int32_t n_done_host = 0;
  auto tap = [&](int div) -> int {
    if (!step_logits) return GN_OK;
    int lr = rows / div;
    host_logits.resize((size_t)lr * V);
    GN_CUDA(cudaMemcpyAsync(host_logits.data(), ro.b.LOGITS, sizeof(float) * (size_t)lr * V, cudaMemcpyDeviceToHost, s));
    GN_CUDA(cudaStreamSynchronize(s));
    float* dst = step_logits + (size_t)ro.generated * rows * V;
    for (int r = 0; r < rows; ++r) std::memcpy(dst + (size_t)r * V, host_logits.data() + (size_t)(r / div) * V, sizeof(float) * V);
    return GN_OK;
  };
  GN_TRY(tap(G));
  GN_TRY(rollout_sample(m, nullptr, temperature, top_k));
  ++ro.generated; ro.logits_row_div = 1;
  auto body = [&]() -> int {
    GN_TRY(rollout_forward(m));
    GN_TRY(rollout_sample(m, nullptr, temperature, top_k));
    return GN_OK;
  };
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  size_t graph_nodes = 0;
  const bool use_graph = !step_logits && m->ctx->use_graphs;
  int status = GN_OK;
  int eager_done = 0;
  auto drop_graph = [&]() { if (exec) cudaGraphExecDestroy(exec); if (graph) cudaGraphDestroy(graph); exec = nullptr; graph = nullptr; };
  while (ro.generated < max_tokens) {
    if (ro.generated % 16 == 0 || step_logits) {  // every row finished: stop early (engine.go:245-254)
      if ((status = cudaMemcpyAsync(&n_done_host, m->n_done.p, sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess ? GN_ERR_CUDA : GN_OK) != GN_OK) break;
      if (cudaStreamSynchronize(s) != cudaSuccess) { status = GN_ERR_CUDA; break; }
      if (n_done_host >= rows) break;
    }
    if (step_logits) {
      // the tap wants the logits each sampling step saw: forward first, copy, then sample
      if ((status = rollout_forward(m)) != GN_OK) break;
      if ((status = tap(1)) != GN_OK) break;
      if ((status = rollout_sample(m, nullptr, temperature, top_k)) != GN_OK) break;
    } else if (!use_graph || eager_done < 2) {
      if ((status = body()) != GN_OK) break;       // eager: also sizes every scratch buffer before the capture
      ++eager_done;
    } else {
      if (!exec) {
        if (cudaStreamSynchronize(s) != cudaSuccess || cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { status = GN_ERR_CUDA; break; }
        status = body();
        cudaError_t ce = cudaStreamEndCapture(s, &graph);
        if (status != GN_OK) break;
        if (ce != cudaSuccess) { set_error("decode graph capture failed: %s", cudaGetErrorString(ce)); status = GN_ERR_CUDA; break; }
        if (cudaGraphGetNodes(graph, nullptr, &graph_nodes) != cudaSuccess || cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
          set_error("decode graph instantiation failed"); status = GN_ERR_CUDA; break;
        }
      }
      if (cudaGraphLaunch(exec, s) != cudaSuccess) { set_error("decode graph launch failed"); status = GN_ERR_CUDA; break; }
      count_launches((int64_t)graph_nodes);
    }
    ++ro.generated;
  }
  if (exec || graph) { cudaStreamSynchronize(s); drop_graph(); }   // also on the error paths
  if (status != GN_OK) { ro.active = false; if (status == GN_ERR_CUDA && !*get_error()) set_error("CUDA error in the decode loop"); return status; }
  GN_CUDA(cudaEventRecord(m->ev[2], s));
  GN_CUDA(cudaMemcpyAsync(out_tokens, m->out_tokens.p, sizeof(int32_t) * (size_t)rows * max_tokens, cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaMemcpyAsync(out_lengths, m->out_lengths.p, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, s));
  if (out_masks) GN_CUDA(cudaMemcpyAsync(out_masks, m->out_masks.p, sizeof(int32_t) * (size_t)rows * max_tokens, cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1])); m->phase_ms["prefill"] = ms;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[1], m->ev[2])); m->phase_ms["decode"] = ms;
  if (steps_run) *steps_run = ro.generated;
  ro.active = false;
  return gemm_check_error(s);
}

int gn_generate_batch(gn_model* m, const int32_t* prompts, int P, int plen, int G, int max_tokens, float temperature, int top_k, const uint64_t* seeds,
                      int32_t* out_tokens, int32_t* out_lengths, float* step_logits, int* steps_run) {
  return gn_generate_batch_ex(m, prompts, P, plen, G, max_tokens, temperature, top_k, seeds, nullptr, out_tokens, out_lengths, nullptr, step_logits, steps_run);
}

// ---- the same engine one step at a time, for hosts that interleave their own logic between steps: tool calls that
//      need the tokenizer (inference/engine.go:284-300), ensembles that blend several models' logits before sampling
//      (inference/ensemble.go:104-243).  Every call returns with the stream idle.
int gn_rollout_begin(gn_model* m, const int32_t* prompts, int P, int plen, int G, int max_tokens, const uint64_t* seeds, const gn_generate_options* opt) {
  GN_TRY(enter_compute(m));
  GN_TRY(rollout_begin(m, prompts, P, plen, G, max_tokens, seeds, opt));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  return gemm_check_error(m->s());
}
int gn_rollout_logits(gn_model* m, float** device_ptr, int* logit_rows, int* row_div) {
  GN_REQUIRE(m && m->ro.active && device_ptr, "gn_rollout_logits: no rollout in progress");
  *device_ptr = m->ro.b.LOGITS;
  if (logit_rows) *logit_rows = m->ro.rows / m->ro.logits_row_div;
  if (row_div) *row_div = m->ro.logits_row_div;
  return GN_OK;
}
int gn_rollout_sample(gn_model* m, const float* logits_device, float temperature, int top_k, int32_t* column, int32_t* mask, int* all_done) {
  GN_TRY(enter(m));
  GN_REQUIRE(m->ro.active, "gn_rollout_sample: no rollout in progress");
  Rollout& ro = m->ro;
  cudaStream_t s = m->s();
  GN_REQUIRE(ro.generated < ro.max_tokens, "gn_rollout_sample: the rollout already has its %d tokens", ro.max_tokens);
  GN_TRY(rollout_sample(m, logits_device, temperature, top_k));
  ++ro.generated; ro.logits_row_div = 1;
  if (column) GN_CUDA(cudaMemcpyAsync(column, m->sampled.p, sizeof(int32_t) * ro.rows, cudaMemcpyDeviceToHost, s));
  if (mask) GN_CUDA(cudaMemcpyAsync(mask, m->engine_state.i() + 4 * (size_t)ro.rows, sizeof(int32_t) * ro.rows, cudaMemcpyDeviceToHost, s));
  int32_t n_done = 0;
  GN_CUDA(cudaMemcpyAsync(&n_done, m->n_done.p, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  if (all_done) *all_done = n_done >= ro.rows ? 1 : 0;
  return GN_OK;
}
int gn_rollout_force(gn_model* m, int row, const int32_t* tokens, int n) {
  GN_TRY(enter(m));
  GN_REQUIRE(m->ro.active && tokens && n >= 0, "gn_rollout_force: no rollout in progress or null tokens");
  Rollout& ro = m->ro;
  GN_REQUIRE(row >= 0 && row < ro.rows, "gn_rollout_force: row %d out of range", row);
  GN_TRY(check_ids(tokens, n, m->V, false, "gn_rollout_force: tokens"));
  cudaStream_t s = m->s();
  int32_t* st = m->engine_state.i();
  int32_t head = 0, len = 0;
  GN_CUDA(cudaMemcpyAsync(&head, st + row, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaMemcpyAsync(&len, st + ro.rows + row, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  GN_REQUIRE(len + n <= kForcedQueue, "gn_rollout_force: row %d would hold %d forced tokens (at most %d)", row, len + n, kForcedQueue);
  for (int i = 0; i < n; ++i) {
    const int slot = (head + len + i) % kForcedQueue;
    GN_CUDA(cudaMemcpyAsync(st + 5 * (size_t)ro.rows + (size_t)row * kForcedQueue + slot, tokens + i, sizeof(int32_t), cudaMemcpyHostToDevice, s));
  }
  len += n;
  GN_CUDA(cudaMemcpyAsync(st + ro.rows + row, &len, sizeof(int32_t), cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaStreamSynchronize(s));
  return GN_OK;
}
int gn_rollout_forward(gn_model* m, const int32_t* column) {
  GN_TRY(enter_compute(m));
  GN_REQUIRE(m->ro.active, "gn_rollout_forward: no rollout in progress");
  Rollout& ro = m->ro;
  cudaStream_t s = m->s();
  if (column) {   // a column sampled elsewhere (an ensemble member follows the member that sampled)
    GN_TRY(check_ids(column, ro.rows, m->V, false, "gn_rollout_forward: column"));
    GN_CUDA(cudaMemcpyAsync(m->sampled.p, column, sizeof(int32_t) * ro.rows, cudaMemcpyHostToDevice, s));
    if (ro.follower_steps++ > 0) GN_TRY(add_i32_launch(m->pos.i(), 1, ro.rows, s));   // a follower advances its own positions
    GN_TRY(ctx_from_pos_launch(m->pos.i(), m->ctxlen.i(), ro.rows, s));
  }
  GN_TRY(rollout_forward(m));
  GN_CUDA(cudaStreamSynchronize(s));
  ro.logits_row_div = 1;
  return gemm_check_error(s);
}
int gn_rollout_end(gn_model* m, int32_t* out_tokens, int32_t* out_lengths, int32_t* out_masks) {
  GN_TRY(enter(m));
  GN_REQUIRE(m->ro.active, "gn_rollout_end: no rollout in progress");
  Rollout& ro = m->ro;
  cudaStream_t s = m->s();
  if (out_tokens) GN_CUDA(cudaMemcpyAsync(out_tokens, m->out_tokens.p, sizeof(int32_t) * (size_t)ro.rows * ro.max_tokens, cudaMemcpyDeviceToHost, s));
  if (out_lengths) GN_CUDA(cudaMemcpyAsync(out_lengths, m->out_lengths.p, sizeof(int32_t) * ro.rows, cudaMemcpyDeviceToHost, s));
  if (out_masks) GN_CUDA(cudaMemcpyAsync(out_masks, m->out_masks.p, sizeof(int32_t) * (size_t)ro.rows * ro.max_tokens, cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  ro.active = false;
  return GN_OK;
}

int gn_policy_gradient_step(gn_model* m, const int32_t* inputs, const int32_t* targets, const float* adv, int B, int T, float norm, int rows_per_pass,
                            float* loss, float* nll_tap, float* dlogits_tap, float* logits_tap) {
  GN_TRY(enter_compute(m));
  GN_REQUIRE(inputs && targets && adv && loss, "gn_policy_gradient_step: null argument");
  GN_REQUIRE(B > 0 && T > 1, "gn_policy_gradient_step: batch must be positive and seq > 1 (model/transformer.go:269-271)");
  GN_REQUIRE(T <= m->cfg.sequence_len, "sequence %d longer than sequence_len %d", T, m->cfg.sequence_len);
  GN_TRY(check_ids(inputs, (int64_t)B * T, m->V, false, "gn_policy_gradient_step: inputs"));
  GN_TRY(check_ids(targets, (int64_t)B * T, m->V, true, "gn_policy_gradient_step: targets"));
  const int V = m->V, L = m->L;
  cudaStream_t s = m->s();
  // ~48 K tokens per pass: measured on d12, 128-row passes cost 1.86 ms per sequence against 2.00 ms for 32-row passes
  // (fuller waves in the products); the pass's saved tensors are ~1.1 MB per token (54 GB at this size)
  if (rows_per_pass <= 0) rows_per_pass = std::max(1, 49152 / T);
  rows_per_pass = std::min(rows_per_pass, B);
  const int64_t all = (int64_t)B * T;
  GN_TRY(m->in_dev.ensure(sizeof(int32_t) * all)); GN_TRY(m->tgt_dev.ensure(sizeof(int32_t) * all)); GN_TRY(m->adv_dev.ensure(sizeof(float) * B));
  GN_TRY(m->loss_dev.ensure(sizeof(double)));
  GN_CUDA(cudaMemcpyAsync(m->in_dev.p, inputs, sizeof(int32_t) * all, cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaMemcpyAsync(m->tgt_dev.p, targets, sizeof(int32_t) * all, cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaMemcpyAsync(m->adv_dev.p, adv, sizeof(float) * B, cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaMemsetAsync(m->loss_dev.p, 0, sizeof(double), s));
  FwdBufs b; BwdBufs w; float* extra = nullptr;
  const int64_t prow = (int64_t)rows_per_pass * T;
  // lm_head, the loss and lm_head's backward run in chunks of rows, so that the [tokens, vocab] logits of a pass never
  // exist as a whole: a chunk is produced, turned into dz in place and consumed by the two gradient products
  // (model/train_transformer.go:137-156 materialises logits, softmax and gradient for the whole batch).
  const int64_t head_chunk = std::min<int64_t>(prow, std::max(1, m->ctx->head_chunk_rows));
  GN_TRY(m->rowloss.ensure(sizeof(double) * (size_t)head_chunk));
  GN_TRY(make_bufs(m, m->train, b, MODE_TRAIN, prow, head_chunk, rows_per_pass, T, bwd_floats(m, prow, rows_per_pass, T), &extra));
  carve_bwd(m, extra, w, prow, rows_per_pass, T);
  LatentWs lws;
  if (m->mla() || m->moe()) {
    GN_TRY(m->lat_ws.ensure(sizeof(float) * latent_ws_layout(m, nullptr, nullptr, prow, rows_per_pass)));
    latent_ws_layout(m, m->lat_ws.f(), &lws, prow, rows_per_pass);
    lws.total_sequences = B;
    b.lws = &lws;
  }
  const bool tc = m->ctx->gemm_kind == 1;
  const int d = m->d;
  float t_fwd = 0, t_loss = 0, t_bwd = 0;
  DevBuf tap_scratch;
  for (int b0 = 0; b0 < B; b0 += rows_per_pass) {
    const int Bm = std::min(rows_per_pass, B - b0);
    const int64_t rows = (int64_t)Bm * T;
    const int32_t* ids = m->in_dev.i() + (int64_t)b0 * T;
    GN_CUDA(cudaEventRecord(m->ev[0], s));
    FwdArgs a; a.mode = MODE_TRAIN; a.ids = ids; a.B = Bm; a.T = T; a.skip_head = true;
    GN_TRY(forward_core(m, b, a));
    GN_CUDA(cudaEventRecord(m->ev[1], s));
    float* nll_dev = w.DELTA;  // [Bm*Hq*T] >= rows floats; free until the attention backward
    for (int64_t r0 = 0; r0 < rows; r0 += head_chunk) {
      const int64_t rc = std::min(head_chunk, rows - r0);
      const int32_t* tg = m->tgt_dev.i() + (int64_t)b0 * T + r0;
      // logits of the chunk: softcap(y W_lm^T)[:, :V]
      { GemmArgs g; g.A = b.Y + r0 * d; g.lda = d; g.B = m->p(m->off_lm); g.b_static = 1; g.ldb = d; g.b_trans = 1; g.C = b.LOGITS; g.ldc = V; g.M = (int)rc; g.N = V; g.K = d;
        g.epilogue = EPI_SOFTCAP; g.scalar = kSoftcap;
        if (tc) { g.a_hi = b.S1h + r0 * d; g.a_lo = b.S1l + r0 * d; } GN_TRY(gemm(m, g)); }
      if (logits_tap) GN_CUDA(cudaMemcpyAsync(logits_tap + ((size_t)b0 * T + r0) * V, b.LOGITS, sizeof(float) * rc * V, cudaMemcpyDeviceToHost, s));
      if (dlogits_tap) {
        // The tap is the gradient at the softcapped logits (what trainer/rl.go hands to TrainBackward), so it takes
        // its own pass without the folded softcap backward.
        GN_TRY(tap_scratch.ensure(sizeof(float) * head_chunk * V));
        GN_TRY(pg_loss_launch(b.LOGITS, tg, m->adv_dev.f() + b0, rc, V, V, T, norm, 0.0f, nullptr, tap_scratch.f(), V, (double*)m->rowloss.p, nullptr, 2, s,
                              nullptr, r0));
        GN_CUDA(cudaMemcpyAsync(dlogits_tap + ((size_t)b0 * T + r0) * V, tap_scratch.p, sizeof(float) * rc * V, cudaMemcpyDeviceToHost, s));
        GN_CUDA(cudaStreamSynchronize(s));
      }
      // loss + dlogits with the softcap backward folded in; dz overwrites the chunk's logits
      GN_TRY(pg_loss_launch(b.LOGITS, tg, m->adv_dev.f() + b0, rc, V, V, T, norm, kSoftcap, nll_dev + r0, b.LOGITS, V, (double*)m->rowloss.p,
                            (double*)m->loss_dev.p, 1, s, nullptr, r0));
      // lm_head: dW[:V] += dz^T y ; dy = dz W[:V]      (model/layers/linear.go:45-53)
      { GemmArgs g; g.A = b.LOGITS; g.lda = V; g.a_trans = 1; g.B = b.Y + r0 * d; g.ldb = d; g.b_trans = 0; if (tc) { g.b_hi = b.S1h + r0 * d; g.b_lo = b.S1l + r0 * d; }
        g.C = m->g(m->off_lm); g.ldc = d; g.M = V; g.N = d; g.K = (int)rc; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
      { GemmArgs g; g.A = b.LOGITS; g.lda = V; g.a_reuse = 1; g.B = m->p(m->off_lm); g.b_static = 1; g.ldb = d; g.b_trans = 0; g.C = w.DY + r0 * d; g.ldc = d; g.M = (int)rc; g.N = d; g.K = V;
        GN_TRY(gemm(m, g)); }
    }
    if (nll_tap) GN_CUDA(cudaMemcpyAsync(nll_tap + (size_t)b0 * T, nll_dev, sizeof(float) * rows, cudaMemcpyDeviceToHost, s));
    GN_CUDA(cudaEventRecord(m->ev[2], s));
    GN_TRY(backward_core(m, b, w, ids, Bm, T, true));
    GN_CUDA(cudaEventRecord(m->ev[3], s));
    GN_CUDA(cudaStreamSynchronize(s));
    float ms = 0;
    GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1])); t_fwd += ms;
    GN_CUDA(cudaEventElapsedTime(&ms, m->ev[1], m->ev[2])); t_loss += ms;
    GN_CUDA(cudaEventElapsedTime(&ms, m->ev[2], m->ev[3])); t_bwd += ms;
  }
  tap_scratch.release();
  GN_TRY(scalar_flush_launch(m->g(m->off_rho), (double*)m->sacc.p, 2 * L + 2, s));
  double loss_host = 0;
  GN_CUDA(cudaMemcpyAsync(&loss_host, m->loss_dev.p, sizeof(double), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  *loss = (float)loss_host;
  m->phase_ms["train_forward"] = t_fwd; m->phase_ms["loss"] = t_loss; m->phase_ms["train_backward"] = t_bwd;
  return gemm_check_error(s);
}

// ---------------------------------------------------------------- KV cache access (wire format support)
namespace {
// Address and float count of one slice of the cache: kind 0 / 1 = key / value of (layer, row, head), 2 = latent of
// (layer, row), 3 = rotary keys of (layer, row), 4 = previous embedding of row.  `positions` cached positions.
int kv_slice(gn_model* m, int layer, int kind, int row, int head, int positions, float** ptr, int64_t* n) {
  GN_REQUIRE(m->kv_rows > 0, "no KV cache: run gn_generate_batch or gn_model_kv_alloc first");
  GN_REQUIRE(row >= 0 && row < m->kv_rows && positions >= 0 && positions <= m->kv_max_seq, "KV slice: row %d / positions %d out of range", row, positions);
  const int64_t S = m->kv_max_seq;
  if (kind == 4) { *ptr = m->prev.f() + (int64_t)row * m->d; *n = m->d; return GN_OK; }
  GN_REQUIRE(layer >= 0 && layer < m->L, "KV slice: layer %d out of range", layer);
  if (kind == 0 || kind == 1) {
    GN_REQUIRE(!m->mla(), "a latent-attention cache holds no per-head keys or values");
    GN_REQUIRE(head >= 0 && head < m->Hkv, "KV slice: head %d out of range", head);
    const int64_t layer_stride = (int64_t)m->kv_rows * m->Hkv * S * m->D;
    *ptr = m->cache.f() + (int64_t)(2 * layer + kind) * layer_stride + ((int64_t)row * m->Hkv + head) * S * m->D;
    *n = (int64_t)positions * m->D;
    return GN_OK;
  }
  GN_REQUIRE(m->mla() && (kind == 2 || kind == 3), "KV slice: kind %d not available for this model", kind);
  if (kind == 2) { *ptr = m->cache_lat.f() + ((int64_t)layer * m->kv_rows + row) * S * m->lat; *n = (int64_t)positions * m->lat; }
  else { const int rw = m->Hkv * m->rope; *ptr = m->cache_rope.f() + ((int64_t)layer * m->kv_rows + row) * S * rw; *n = (int64_t)positions * rw; }
  return GN_OK;
}
}  // namespace

int gn_model_kv_info(gn_model* m, int* rows, int* max_seq, int* position) {
  GN_TRY(enter(m));
  if (rows) *rows = m->kv_rows;
  if (max_seq) *max_seq = m->kv_max_seq;
  if (position) {
    int32_t p = 0;
    if (m->kv_rows > 0) { GN_CUDA(cudaMemcpyAsync(&p, m->pos.p, sizeof(int32_t), cudaMemcpyDeviceToHost, m->s())); GN_CUDA(cudaStreamSynchronize(m->s())); }
    *position = p;
  }
  return GN_OK;
}
int gn_model_kv_alloc(gn_model* m, int rows, int max_seq, int position) {
  GN_TRY(enter(m));
  GN_REQUIRE(rows > 0 && max_seq > 0 && position >= 0 && position <= max_seq, "gn_model_kv_alloc: bad geometry");
  if (m->mla()) {
    GN_TRY(m->cache_lat.ensure(sizeof(float) * (size_t)m->L * rows * max_seq * m->lat));
    GN_TRY(m->cache_rope.ensure(sizeof(float) * (size_t)m->L * rows * max_seq * m->Hkv * m->rope));
  } else {
    GN_TRY(m->cache.ensure(sizeof(float) * (size_t)m->L * 2 * rows * m->Hkv * max_seq * m->D));
  }
  GN_TRY(m->prev.ensure(sizeof(float) * (size_t)rows * m->d));
  GN_TRY(m->pos.ensure(sizeof(int32_t) * rows)); GN_TRY(m->ctxlen.ensure(sizeof(int32_t) * rows));
  m->kv_rows = rows; m->kv_max_seq = max_seq;
  GN_TRY(fill_i32_launch(m->pos.i(), position, rows, m->s()));
  GN_TRY(fill_i32_launch(m->ctxlen.i(), position + 1, rows, m->s()));
  GN_CUDA(cudaStreamSynchronize(m->s()));
  return GN_OK;
}
int gn_model_kv_read(gn_model* m, int layer, int kind, int row, int head, int positions, float* host, int64_t n) {
  GN_TRY(enter(m));
  GN_REQUIRE(host, "gn_model_kv_read: null buffer");
  float* p = nullptr; int64_t want = 0;
  GN_TRY(kv_slice(m, layer, kind, row, head, positions, &p, &want));
  GN_REQUIRE(n == want, "gn_model_kv_read: the slice has %lld floats, got room for %lld", (long long)want, (long long)n);
  if (n > 0) { GN_CUDA(cudaMemcpyAsync(host, p, sizeof(float) * n, cudaMemcpyDeviceToHost, m->s())); GN_CUDA(cudaStreamSynchronize(m->s())); }
  return GN_OK;
}
int gn_model_kv_write(gn_model* m, int layer, int kind, int row, int head, int positions, const float* host, int64_t n) {
  GN_TRY(enter(m));
  GN_REQUIRE(host, "gn_model_kv_write: null buffer");
  float* p = nullptr; int64_t want = 0;
  GN_TRY(kv_slice(m, layer, kind, row, head, positions, &p, &want));
  GN_REQUIRE(n == want, "gn_model_kv_write: the slice has %lld floats, got %lld", (long long)want, (long long)n);
  if (n > 0) { GN_CUDA(cudaMemcpyAsync(p, host, sizeof(float) * n, cudaMemcpyHostToDevice, m->s())); GN_CUDA(cudaStreamSynchronize(m->s())); }
  m->ro.prompt_shared = false;   // the decode attention may no longer take the prompt's keys from the group's first row
  return GN_OK;
}

int gn_model_phase_ms(gn_model* m, const char* phase, float* ms) {
  GN_REQUIRE(m && phase && ms, "null argument");
  auto it = m->phase_ms.find(phase);
  GN_REQUIRE(it != m->phase_ms.end(), "no timing recorded for phase '%s'", phase);
  *ms = it->second;
  return GN_OK;
}

}  // extern "C"
