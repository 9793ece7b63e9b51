// The latent preset in the training pass of the RL step (trainer/rl.go:14-60 through model/train.go):
//   latent attention in its un-absorbed training construction (model/mla.go:106-146, model/train.go:59-60,82-85,
//   414-419): per-head [content | rotary] queries and keys and up-projected values, then ordinary attention;
//   DeepSeekMoE feed-forward with its backward (model/train.go:490-514,538-572, model/moe.go:118-326): a shared
//   SwiGLU expert plus top-k routed experts, the router's softmax backward and the sequence-level balance loss
//   whose gradient enters through that softmax.
//
// Products run on the GEMM family of the dense path; the routed experts' forward products are the grouped
// tensor-core product, their backward products are one launch per (expert, product) over that expert's rows (the
// counts are read back to the host once per layer in the forward pass).  Row kernels: one warp per row or entry.
#include "model_internal.cuh"

namespace gnm {

namespace {

constexpr int WPB = 8;

int grid_for(int64_t n) { return (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 16)); }

// ------------------------------------------------------------------ latent attention glue
// Forward: QKV[r, slot, :] = [content | rotate(rope)] for the Hq query and Hkv key slots (model/mla.go:114-121,
// model/rotary.go:43-75).  The rotary parts of all heads sit side by side in P1 after the two latents.
struct MlaHeads {
  const float* QC; const float* KC; const float* P1; int64_t n1;
  float* QKV;
  const float* cosv; const float* sinv;
  int64_t rows; int T, Hq, Hkv, D, lat, rope, content;
};
__global__ void __launch_bounds__(WPB * 32) mla_assemble_kernel(MlaHeads p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.Hq + p.Hkv;
  const int64_t idx = (int64_t)blockIdx.x * WPB + warp;
  if (idx >= p.rows * slots) return;
  const int64_t r = idx / slots; const int slot = (int)(idx % slots);
  const int t = (int)(r % p.T);
  const int W = (p.Hq + 2 * p.Hkv) * p.D;
  float* dst = p.QKV + r * W + (int64_t)slot * p.D;
  const float* cs = slot < p.Hq ? p.QC + (r * p.Hq + slot) * (int64_t)p.content : p.KC + (r * p.Hkv + (slot - p.Hq)) * (int64_t)p.content;
  for (int c = lane; c < p.content; c += 32) dst[c] = cs[c];
  const float* rs = p.P1 + r * p.n1 + 2 * p.lat + (int64_t)slot * p.rope;
  const int half = p.rope / 2;
  const float* cw = p.cosv + (int64_t)t * half; const float* sw = p.sinv + (int64_t)t * half;
  for (int j = lane; j < half; j += 32) {
    const float a = rs[j], b = rs[half + j];
    dst[p.content + j] = __fadd_rn(__fmul_rn(a, cw[j]), __fmul_rn(b, sw[j]));
    dst[p.content + half + j] = __fadd_rn(__fmul_rn(-a, sw[j]), __fmul_rn(b, cw[j]));
  }
}
// Backward: the gradient of a head goes back to its content part (DQC / DKC) and, through the rotation transposed
// (the same routine with the sine negated, model/train.go:414-417), to the rotary columns of DP1.
struct MlaHeadsBwd {
  const float* DQKV; float* DQC; float* DKC; float* DP1; int64_t n1;
  const float* cosv; const float* sinv;
  int64_t rows; int T, Hq, Hkv, D, lat, rope, content;
};
__global__ void __launch_bounds__(WPB * 32) mla_disassemble_kernel(MlaHeadsBwd p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.Hq + p.Hkv;
  const int64_t idx = (int64_t)blockIdx.x * WPB + warp;
  if (idx >= p.rows * slots) return;
  const int64_t r = idx / slots; const int slot = (int)(idx % slots);
  const int t = (int)(r % p.T);
  const int W = (p.Hq + 2 * p.Hkv) * p.D;
  const float* g = p.DQKV + r * W + (int64_t)slot * p.D;
  float* cd = slot < p.Hq ? p.DQC + (r * p.Hq + slot) * (int64_t)p.content : p.DKC + (r * p.Hkv + (slot - p.Hq)) * (int64_t)p.content;
  for (int c = lane; c < p.content; c += 32) cd[c] = g[c];
  float* rd = p.DP1 + r * p.n1 + 2 * p.lat + (int64_t)slot * p.rope;
  const int half = p.rope / 2;
  const float* cw = p.cosv + (int64_t)t * half; const float* sw = p.sinv + (int64_t)t * half;
  for (int j = lane; j < half; j += 32) {
    const float a = g[p.content + j], b = g[p.content + half + j];
    const float sn = -sw[j];
    rd[j] = __fadd_rn(__fmul_rn(a, cw[j]), __fmul_rn(b, sn));
    rd[half + j] = __fadd_rn(__fmul_rn(-a, sn), __fmul_rn(b, cw[j]));
  }
}

// ------------------------------------------------------------------ shared SwiGLU expert
// UG = [up | gate] per row.  hidden = silu(min(gate, clamp)) * clamp(up)  (kernels/scalar/elementwise.go:105-134)
__global__ void __launch_bounds__(256) swiglu_rows_split_kernel(float* dst, float* hi, float* lo, const float* ug, int64_t rows, int width, float clampv) {
  const int64_t total = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width; const int c = (int)(i % width);
    float u = ug[r * 2 * width + c], g = ug[r * 2 * width + width + c];
    if (clampv > 0.0f && g >= clampv) g = clampv;
    if (clampv > 0.0f) { if (u > clampv) u = clampv; else if (u < -clampv) u = -clampv; }
    const float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
    const float v = g * sg * u;
    dst[i] = v;
    if (hi) { float h, l; split_tf32(v, h, l); hi[i] = h; lo[i] = l; }
  }
}
// Backward of the same in the [up | gate] layout: DUG = [d up | d gate] from d hidden (kernels/scalar/elementwise.go:
// 136-162: a clamped input passes no gradient).
__global__ void __launch_bounds__(256) swiglu_rows_bwd_kernel(float* dug, const float* ug, const float* dh, int64_t rows, int width, float clampv) {
  const int64_t total = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width; const int c = (int)(i % width);
    const float u0 = ug[r * 2 * width + c], g0 = ug[r * 2 * width + width + c];
    float u = u0, g = g0;
    bool gpass = true, upass = true;
    if (clampv > 0.0f) {
      if (g >= clampv) { g = clampv; gpass = false; }
      if (u > clampv) { u = clampv; upass = false; } else if (u < -clampv) { u = -clampv; upass = false; }
    }
    const float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
    const float silu = g * sg;
    const float og = dh[i];
    dug[r * 2 * width + c] = upass ? og * silu : 0.0f;
    dug[r * 2 * width + width + c] = gpass ? og * u * (sg * (1.0f + g * (1.0f - sg))) : 0.0f;
  }
}

// ------------------------------------------------------------------ routed experts, forward glue
// gathered[posi[i]] = x[i / k] with the tf32 split (model/moe.go:141-153)
__global__ void __launch_bounds__(WPB * 32) gather_rows_kernel(float* gathered, float* hi, float* lo, const float* x, const int32_t* posi, int64_t total, int k, int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * WPB + warp;
  if (i >= total) return;
  const float* src = x + (i / k) * d; const int64_t o = (int64_t)posi[i] * d;
  for (int c = lane; c < d; c += 32) {
    const float v = src[c];
    gathered[o + c] = v;
    if (hi) { float h, l; split_tf32(v, h, l); hi[o + c] = h; lo[o + c] = l; }
  }
}
// hidden = swiglu(gate, up) kept beside its inputs (the backward needs all three), with the tf32 split
__global__ void __launch_bounds__(256) swiglu_keep_kernel(float* hid, float* hi, float* lo, const float* gate, const float* up, int64_t n, float clampv) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float g = gate[i], u = up[i];
    if (clampv > 0.0f && g >= clampv) g = clampv;
    if (clampv > 0.0f) { if (u > clampv) u = clampv; else if (u < -clampv) u = -clampv; }
    const float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
    const float v = g * sg * u;
    hid[i] = v;
    if (hi) { float h, l; split_tf32(v, h, l); hi[i] = h; lo[i] = l; }
  }
}
// XOUT[r] = MID[r] + (shared[r] + routed[r]); routed[r] = sum over the row's entries in ascending position of
// (weight * scale) * expert_out[position] (model/moe.go:160-169, model/train.go:549-551)
__global__ void __launch_bounds__(256) combine_kernel(float* xout, const float* mid, const float* shared, const float* expert_out, const int32_t* posi,
                                                      const float* selw, float scale, int64_t rows, int k, int d) {
  const int64_t total = rows * d;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / d; const int c = (int)(i % d);
    int ps[8]; float ws[8];
    for (int s = 0; s < k; ++s) { ps[s] = posi[r * k + s]; ws[s] = __fmul_rn(selw[r * k + s], scale); }
    for (int a = 1; a < k; ++a) {
      const int pa = ps[a]; const float wa = ws[a]; int j = a - 1;
      while (j >= 0 && ps[j] > pa) { ps[j + 1] = ps[j]; ws[j + 1] = ws[j]; --j; }
      ps[j + 1] = pa; ws[j + 1] = wa;
    }
    float routed = 0.0f;
    for (int s = 0; s < k; ++s) routed = __fadd_rn(routed, __fmul_rn(ws[s], expert_out[(int64_t)ps[s] * d + c]));
    xout[i] = __fadd_rn(mid[i], __fadd_rn(shared[i], routed));
  }
}

// ------------------------------------------------------------------ routed experts, backward glue
// One warp per (row, slot) entry: dGO[pos] = dout[row] * (weight * scale) and the probability gradient
// gprobs[row, expert] = scale * <dout[row], GO[pos]> in float64 (model/moe.go:215-230).
__global__ void __launch_bounds__(WPB * 32) moe_bwd_entry_kernel(float* dgo, double* gprobs, const float* dout, const float* go, const int32_t* posi,
                                                                 const int32_t* sel, const float* selw, float scale, int64_t total, int k, int d, int E) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * WPB + warp;
  if (i >= total) return;
  const int64_t row = i / k; const int64_t pos = posi[i];
  const float w = __fmul_rn(selw[i], scale);
  const float* g = dout + row * d; const float* o = go + pos * d; float* dst = dgo + pos * d;
  double dot = 0.0;
  for (int c = lane; c < d; c += 32) { const float gv = g[c]; dst[c] = gv * w; dot += (double)gv * (double)o[c]; }
  dot = warp_sum_d(dot);
  if (lane == 0) gprobs[row * E + sel[i]] = dot * (double)scale;
}
// count[s, e]: how many tokens of sequence s selected expert e (model/moe.go:287-294).  One block per sequence.
__global__ void __launch_bounds__(256) moe_seq_counts_kernel(int32_t* counts, const int32_t* sel, int seq_len, int k, int E) {
  __shared__ int cnt[64];
  if (threadIdx.x < 64) cnt[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * seq_len * k;
  for (int i = threadIdx.x; i < seq_len * k; i += blockDim.x) atomicAdd(&cnt[sel[base + i]], 1);
  __syncthreads();
  if (threadIdx.x < E) counts[(int64_t)blockIdx.x * E + threadIdx.x] = cnt[threadIdx.x];
}
// Per row: add the balance loss's probability gradient (model/moe.go:316-325), then the router softmax backward
// dlogits = p * (dprobs - <dprobs, p>) in float64 (model/moe.go:250-262).
__global__ void __launch_bounds__(256) moe_router_bwd_kernel(float* dlogits, const double* gprobs, const float* probs, const int32_t* seq_counts, int64_t rows,
                                                             int seq_len, int64_t sequences, int E, int k, double balance_weight) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const double coefficient = balance_weight / ((double)sequences * (double)seq_len);
  const double selection_scale = (double)E / ((double)k * (double)seq_len);
  const int32_t* sc = seq_counts + (r / seq_len) * E;
  double dot = 0.0;
  for (int e = 0; e < E; ++e) dot += (double)probs[r * E + e] * (gprobs[r * E + e] + coefficient * selection_scale * (double)sc[e]);
  for (int e = 0; e < E; ++e) {
    const double gp = gprobs[r * E + e] + coefficient * selection_scale * (double)sc[e];
    dlogits[r * E + e] = (float)((double)probs[r * E + e] * (gp - dot));
  }
}
// dm[r] = shared[r] + (sum over the row's entries in ascending position of dgath[position]) + router[r]
// (model/moe.go:236-241,263-265, model/train.go:563-566)
__global__ void __launch_bounds__(256) moe_bwd_combine_kernel(float* dm, const float* shared, const float* dgath, const float* router, const int32_t* posi,
                                                              int64_t rows, int k, int d) {
  const int64_t total = rows * d;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / d; const int c = (int)(i % d);
    int ps[8];
    for (int s = 0; s < k; ++s) ps[s] = posi[r * k + s];
    for (int a = 1; a < k; ++a) { const int pa = ps[a]; int j = a - 1; while (j >= 0 && ps[j] > pa) { ps[j + 1] = ps[j]; --j; } ps[j + 1] = pa; }
    float routed = 0.0f;
    for (int s = 0; s < k; ++s) routed = __fadd_rn(routed, dgath[(int64_t)ps[s] * d + c]);
    dm[i] = __fadd_rn(shared[i], __fadd_rn(routed, router[i]));
  }
}
__global__ void __launch_bounds__(256) add2_kernel(float* dst, const float* a, const float* b, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = __fadd_rn(a[i], b[i]);
}

}  // namespace

// What a layer of the latent preset keeps from the training forward for its backward, carved from `base`
// (base == null: only counts).  Returns the floats used.
size_t latent_saved_layout(const gn_model* m, float* base, LayerSaved* s, int64_t rows) {
  size_t used = 0;
  auto take = [&](int64_t n) { float* q = base ? base + used : nullptr; used += (size_t)((n + 63) / 64 * 64); return q; };
  if (m->mla()) { float* q = take(rows * (2 * m->lat + (int64_t)(m->Hq + m->Hkv) * m->rope)); if (s) s->P1 = q; }
  if (m->moe()) {
    const int64_t tot = rows * m->topk;
    float* q;
    q = take(rows * 2 * m->sh); if (s) s->UG = q;
    q = take(rows * m->sh); if (s) s->SHH = q;
    q = take(rows * m->sh); if (s) s->SHHh = q;
    q = take(rows * m->sh); if (s) s->SHHl = q;
    q = take(rows * m->E); if (s) s->PR = q;
    q = take(tot); if (s) s->SELW = q;
    q = take(tot); if (s) s->SEL = (int32_t*)q;
    q = take(tot); if (s) s->POSI = (int32_t*)q;
    q = take(m->E + 1); if (s) s->CNT = (int32_t*)q;
    q = take(tot * m->eh); if (s) s->GG = q;
    q = take(tot * m->eh); if (s) s->GU = q;
    q = take(tot * m->eh); if (s) s->GH = q;
    q = take(tot * m->eh); if (s) s->GHh = q;
    q = take(tot * m->eh); if (s) s->GHl = q;
    q = take(tot * (int64_t)m->d); if (s) s->GO = q;
  }
  return used;
}
// Scratch of one pass shared by all layers (forward and backward), carved from `base` (null: only counts).
size_t latent_ws_layout(const gn_model* m, float* base, LatentWs* w, int64_t rows, int B) {
  size_t used = 0;
  auto take = [&](int64_t n) { float* q = base ? base + used : nullptr; used += (size_t)((n + 63) / 64 * 64); return q; };
  float* q;
  if (m->mla()) {
    const int64_t n1 = 2 * m->lat + (int64_t)(m->Hq + m->Hkv) * m->rope;
    q = take(rows * (int64_t)m->Hq * m->content); if (w) w->QC = q;
    q = take(rows * (int64_t)m->Hkv * m->content); if (w) w->KC = q;
    q = take(rows * (int64_t)m->Hq * m->content); if (w) w->DQC = q;
    q = take(rows * (int64_t)m->Hkv * m->content); if (w) w->DKC = q;
    q = take(rows * n1); if (w) w->DP1 = q;
  }
  if (m->moe()) {
    const int64_t tot = rows * m->topk;
    q = take(rows * (int64_t)m->d); if (w) w->SHO = q;
    q = take(rows * m->E); if (w) w->RL = q;
    q = take(tot * (int64_t)m->d); if (w) w->GATH = q;
    q = take(tot * (int64_t)m->d); if (w) w->GATHh = q;
    q = take(tot * (int64_t)m->d); if (w) w->GATHl = q;
    q = take(rows * m->sh); if (w) w->DSHH = q;
    q = take(rows * 2 * m->sh); if (w) w->DUG = q;
    q = take(rows * (int64_t)m->d); if (w) w->DMS = q;
    q = take(rows * (int64_t)m->d); if (w) w->DMR = q;
    q = take(tot * (int64_t)m->d); if (w) w->DGO = q;
    q = take(tot * m->eh); if (w) w->DGH = q;
    q = take(tot * m->eh); if (w) w->DGG = q;
    q = take(tot * m->eh); if (w) w->DGU = q;
    q = take(tot * (int64_t)m->d); if (w) w->DGATH = q;
    q = take(2 * rows * m->E); if (w) w->GPROB = (double*)q;
    q = take(rows * m->E); if (w) w->GLOG = q;
    q = take((int64_t)B * m->E + m->E); if (w) w->SEQCNT = (int32_t*)q;
  }
  return used;
}

// ------------------------------------------------------------------ latent attention, training forward
// H = norm(x) with its split Hh / Hl.  Fills sv.P1, sv.QKV (post-rotary q, k and v, the layout the attention kernels
// read), sv.O and sv.LSE.
int latent_attention_train(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* H, const float* Hh, const float* Hl, int B, int T) {
  const int d = m->d, Hq = m->Hq, Hkv = m->Hkv, D = m->D, lat = m->lat, rope = m->rope, content = m->content;
  const int64_t rows = (int64_t)B * T;
  const int n1 = 2 * lat + (Hq + Hkv) * rope, W = m->W;
  const LayerOffsets& o = m->lo[l];
  const bool tc = m->ctx->gemm_kind == 1;
  cudaStream_t s = m->s();
  { GemmArgs g; g.A = H; g.lda = d; g.B = m->p(o.mla_cat); g.b_static = 1; g.ldb = d; g.b_trans = 1; g.C = sv.P1; g.ldc = n1; g.M = (int)rows; g.N = n1; g.K = d;
    if (tc) { g.a_hi = Hh; g.a_lo = Hl; } GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = sv.P1; g.lda = n1; g.B = m->p(o.mla_q_up); g.b_static = 1; g.ldb = lat; g.b_trans = 1; g.C = w.QC; g.ldc = (int64_t)Hq * content;
    g.M = (int)rows; g.N = Hq * content; g.K = lat; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = sv.P1 + lat; g.lda = n1; g.B = m->p(o.mla_k_up); g.b_static = 1; g.ldb = lat; g.b_trans = 1; g.C = w.KC; g.ldc = (int64_t)Hkv * content;
    g.M = (int)rows; g.N = Hkv * content; g.K = lat; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = sv.P1 + lat; g.lda = n1; g.B = m->p(o.mla_v_up); g.b_static = 1; g.ldb = lat; g.b_trans = 1; g.C = sv.QKV + (int64_t)(Hq + Hkv) * D; g.ldc = W;
    g.M = (int)rows; g.N = Hkv * D; g.K = lat; GN_TRY(gemm(m, g)); }
  MlaHeads ph; ph.QC = w.QC; ph.KC = w.KC; ph.P1 = sv.P1; ph.n1 = n1; ph.QKV = sv.QKV; ph.cosv = m->cosb.f(); ph.sinv = m->sinb.f();
  ph.rows = rows; ph.T = T; ph.Hq = Hq; ph.Hkv = Hkv; ph.D = D; ph.lat = lat; ph.rope = rope; ph.content = content;
  mla_assemble_kernel<<<ceil_div(rows * (Hq + Hkv), WPB), WPB * 32, 0, s>>>(ph); GN_LAUNCH_CHECK();
  AttnShape sh;
  sh.B = B; sh.Hq = Hq; sh.Hkv = Hkv; sh.D = D; sh.Tq = T; sh.Tk = T;
  sh.q_bstride = (int64_t)T * W; sh.q_tstride = W; sh.kv_bstride = (int64_t)T * W; sh.kv_tstride = W; sh.kv_hstride = D;
  sh.o_bstride = (int64_t)T * Hq * D; sh.o_tstride = (int64_t)Hq * D; sh.window = m->windows[l]; sh.offset0 = 0; sh.tensor = tc;
  return attention_forward_launch(sh, sv.QKV, sv.QKV + (int64_t)Hq * D, sv.QKV + (int64_t)(Hq + Hkv) * D, sv.O, sv.LSE, s);
}

// DQKV: gradient at the post-rotary q, k and at v (what the attention backward leaves).  Accumulates the seven
// projection gradients and writes DH = gradient at H.
int latent_attention_backward(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* H, const float* DQKV, float* DH, int B, int T) {
  const int d = m->d, Hq = m->Hq, Hkv = m->Hkv, D = m->D, lat = m->lat, rope = m->rope, content = m->content;
  const int64_t rows = (int64_t)B * T;
  const int n1 = 2 * lat + (Hq + Hkv) * rope, W = m->W;
  const LayerOffsets& o = m->lo[l];
  cudaStream_t s = m->s();
  MlaHeadsBwd pb; pb.DQKV = DQKV; pb.DQC = w.DQC; pb.DKC = w.DKC; pb.DP1 = w.DP1; pb.n1 = n1; pb.cosv = m->cosb.f(); pb.sinv = m->sinb.f();
  pb.rows = rows; pb.T = T; pb.Hq = Hq; pb.Hkv = Hkv; pb.D = D; pb.lat = lat; pb.rope = rope; pb.content = content;
  mla_disassemble_kernel<<<ceil_div(rows * (Hq + Hkv), WPB), WPB * 32, 0, s>>>(pb); GN_LAUNCH_CHECK();
  const float* DV = DQKV + (int64_t)(Hq + Hkv) * D;
  // q_up: dW += DQC^T q_latent ; d q_latent = DQC W
  { GemmArgs g; g.A = w.DQC; g.lda = (int64_t)Hq * content; g.a_trans = 1; g.B = sv.P1; g.ldb = n1; g.C = m->g(o.mla_q_up); g.ldc = lat; g.M = Hq * content; g.N = lat; g.K = (int)rows;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = w.DQC; g.lda = (int64_t)Hq * content; g.B = m->p(o.mla_q_up); g.b_static = 1; g.ldb = lat; g.C = w.DP1; g.ldc = n1; g.M = (int)rows; g.N = lat; g.K = Hq * content; GN_TRY(gemm(m, g)); }
  // k_up and v_up share the kv latent: d kv_latent = DKC Wk + DV Wv
  { GemmArgs g; g.A = w.DKC; g.lda = (int64_t)Hkv * content; g.a_trans = 1; g.B = sv.P1 + lat; g.ldb = n1; g.C = m->g(o.mla_k_up); g.ldc = lat; g.M = Hkv * content; g.N = lat; g.K = (int)rows;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = w.DKC; g.lda = (int64_t)Hkv * content; g.B = m->p(o.mla_k_up); g.b_static = 1; g.ldb = lat; g.C = w.DP1 + lat; g.ldc = n1; g.M = (int)rows; g.N = lat; g.K = Hkv * content; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = DV; g.lda = W; g.a_trans = 1; g.B = sv.P1 + lat; g.ldb = n1; g.C = m->g(o.mla_v_up); g.ldc = lat; g.M = Hkv * D; g.N = lat; g.K = (int)rows;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = DV; g.lda = W; g.B = m->p(o.mla_v_up); g.b_static = 1; g.ldb = lat; g.C = w.DP1 + lat; g.ldc = n1; g.M = (int)rows; g.N = lat; g.K = Hkv * D;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  // the four projections of H are one [n1, d] matrix: dW += DP1^T H ; DH = DP1 W
  { GemmArgs g; g.A = w.DP1; g.lda = n1; g.a_trans = 1; g.B = H; g.ldb = d; g.C = m->g(o.mla_cat); g.ldc = d; g.M = n1; g.N = d; g.K = (int)rows; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = w.DP1; g.lda = n1; g.B = m->p(o.mla_cat); g.b_static = 1; g.ldb = d; g.C = DH; g.ldc = d; g.M = (int)rows; g.N = d; g.K = n1; GN_TRY(gemm(m, g)); }
  return GN_OK;
}

// ------------------------------------------------------------------ DeepSeekMoE feed-forward, training forward
// Mn = norm(MID) with its split.  XOUT = MID + (shared(Mn) + routed(Mn)); keeps what the backward needs in sv and the
// per-expert row counts on the host.
int moe_ffn_train(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* Mn, const float* Mh, const float* Ml, const float* MID, float* XOUT, int64_t rows) {
  const int d = m->d, E = m->E, K = m->topk, eh = m->eh, sh = m->sh;
  const int64_t total = rows * K;
  const LayerOffsets& o = m->lo[l];
  const bool tc = m->ctx->gemm_kind == 1;
  cudaStream_t s = m->s();
  { GemmArgs g; g.A = Mn; g.lda = d; g.B = m->p(o.fc); g.b_static = 1; g.ldb = d; g.b_trans = 1; g.C = sv.UG; g.ldc = 2 * sh; g.M = (int)rows; g.N = 2 * sh; g.K = d;
    if (tc) { g.a_hi = Mh; g.a_lo = Ml; } GN_TRY(gemm(m, g)); }
  swiglu_rows_split_kernel<<<grid_for(rows * sh), 256, 0, s>>>(sv.SHH, tc ? sv.SHHh : nullptr, tc ? sv.SHHl : nullptr, sv.UG, rows, sh, m->moe_clamp); GN_LAUNCH_CHECK();
  { GemmArgs g; g.A = sv.SHH; g.lda = sh; g.B = m->p(o.mproj); g.b_static = 1; g.ldb = sh; g.b_trans = 1; g.C = w.SHO; g.ldc = d; g.M = (int)rows; g.N = d; g.K = sh;
    if (tc) { g.a_hi = sv.SHHh; g.a_lo = sv.SHHl; } GN_TRY(gemm(m, g)); }
  GN_TRY(moe_router_logits(m, l, Mn, w.RL, rows));   // plain float32: routing must not depend on a split's rounding
  GN_TRY(moe_gate_topk_launch(w.RL, m->p(o.router_bias), sv.PR, sv.SEL, sv.SELW, (int)rows, E, K, s));
  GN_TRY(moe_route_launch(sv.SEL, total, E, sv.CNT, sv.POSI, s));
  gather_rows_kernel<<<ceil_div(total, WPB), WPB * 32, 0, s>>>(w.GATH, tc ? w.GATHh : nullptr, tc ? w.GATHl : nullptr, Mn, sv.POSI, total, K, d); GN_LAUNCH_CHECK();
  const int kind = m->ctx->gemm_kind;
  auto grouped = [&](const float* A, const float* Ah, const float* Al, int64_t w_off, float* C, int n, int k) -> int {
    GemmArgs g; g.A = A; g.lda = k; g.B = m->p(w_off); g.b_static = 1; g.ldb = k; g.b_trans = 1; g.C = C; g.ldc = n; g.M = (int)total; g.N = n; g.K = k;
    g.group_counts = sv.CNT; g.groups = E; if (tc) { g.a_hi = Ah; g.a_lo = Al; }
    return gemm_grouped_dispatch(g, kind, s);
  };
  GN_TRY(grouped(w.GATH, w.GATHh, w.GATHl, o.exp_gate, sv.GG, eh, d));
  GN_TRY(grouped(w.GATH, w.GATHh, w.GATHl, o.exp_up, sv.GU, eh, d));
  swiglu_keep_kernel<<<grid_for(total * eh), 256, 0, s>>>(sv.GH, tc ? sv.GHh : nullptr, tc ? sv.GHl : nullptr, sv.GG, sv.GU, total * eh, m->moe_clamp); GN_LAUNCH_CHECK();
  GN_TRY(grouped(sv.GH, sv.GHh, sv.GHl, o.exp_down, sv.GO, d, eh));
  combine_kernel<<<grid_for(rows * d), 256, 0, s>>>(XOUT, MID, w.SHO, sv.GO, sv.POSI, sv.SELW, m->moe_scale, rows, K, d); GN_LAUNCH_CHECK();
  // the backward launches one product per expert over that expert's rows: the counts come to the host here
  sv.host_counts.assign(E, 0);
  GN_CUDA(cudaMemcpyAsync(sv.host_counts.data(), sv.CNT, sizeof(int32_t) * E, cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  return GN_OK;
}

// DOUT: gradient of the block output.  Accumulates the gradients of the shared expert, the router and the packed
// experts, and writes DM = gradient at Mn (model/train.go:505-514,560-566, model/moe.go:203-267).
int moe_ffn_backward(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* Mn, const float* DOUT, float* DM, int64_t rows, int seq_len) {
  const int d = m->d, E = m->E, K = m->topk, eh = m->eh, sh = m->sh;
  const int64_t total = rows * K;
  const LayerOffsets& o = m->lo[l];
  cudaStream_t s = m->s();
  // ---- shared SwiGLU expert
  { GemmArgs g; g.A = DOUT; g.lda = d; g.a_trans = 1; g.B = sv.SHH; g.ldb = sh; g.C = m->g(o.mproj); g.ldc = sh; g.M = d; g.N = sh; g.K = (int)rows; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = DOUT; g.lda = d; g.B = m->p(o.mproj); g.b_static = 1; g.ldb = sh; g.C = w.DSHH; g.ldc = sh; g.M = (int)rows; g.N = sh; g.K = d; GN_TRY(gemm(m, g)); }
  swiglu_rows_bwd_kernel<<<grid_for(rows * sh), 256, 0, s>>>(w.DUG, sv.UG, w.DSHH, rows, sh, m->moe_clamp); GN_LAUNCH_CHECK();
  { GemmArgs g; g.A = w.DUG; g.lda = 2 * sh; g.a_trans = 1; g.B = Mn; g.ldb = d; g.C = m->g(o.fc); g.ldc = d; g.M = 2 * sh; g.N = d; g.K = (int)rows; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
  { GemmArgs g; g.A = w.DUG; g.lda = 2 * sh; g.B = m->p(o.fc); g.b_static = 1; g.ldb = d; g.C = w.DMS; g.ldc = d; g.M = (int)rows; g.N = d; g.K = 2 * sh; GN_TRY(gemm(m, g)); }
  // ---- routed experts
  GN_CUDA(cudaMemsetAsync(w.GPROB, 0, sizeof(double) * rows * E, s));
  moe_bwd_entry_kernel<<<ceil_div(total, WPB), WPB * 32, 0, s>>>(w.DGO, w.GPROB, DOUT, sv.GO, sv.POSI, sv.SEL, sv.SELW, m->moe_scale, total, K, d, E); GN_LAUNCH_CHECK();
  gather_rows_kernel<<<ceil_div(total, WPB), WPB * 32, 0, s>>>(w.GATH, nullptr, nullptr, Mn, sv.POSI, total, K, d); GN_LAUNCH_CHECK();
  int64_t off = 0;
  for (int e = 0; e < E; ++e) {
    const int cnt = sv.host_counts[e];
    if (cnt == 0) continue;
    const float* dgo = w.DGO + off * d; const float* gh = sv.GH + off * eh;
    float* dgh = w.DGH + off * eh;
    // down_e [d, eh]: dW += dGO^T GH ; dGH = dGO W
    { GemmArgs g; g.A = dgo; g.lda = d; g.a_trans = 1; g.B = gh; g.ldb = eh; g.C = m->g(o.exp_down) + (int64_t)e * d * eh; g.ldc = eh; g.M = d; g.N = eh; g.K = cnt; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = dgo; g.lda = d; g.B = m->p(o.exp_down) + (int64_t)e * d * eh; g.b_static = 1; g.ldb = eh; g.C = dgh; g.ldc = eh; g.M = cnt; g.N = eh; g.K = d; GN_TRY(gemm(m, g)); }
    off += cnt;
  }
  GN_TRY(swiglu_backward_launch(w.DGG, w.DGU, sv.GG, sv.GU, w.DGH, m->moe_clamp, total * eh, s));
  off = 0;
  for (int e = 0; e < E; ++e) {
    const int cnt = sv.host_counts[e];
    if (cnt == 0) continue;
    const float* x = w.GATH + off * d;
    const float* dgg = w.DGG + off * eh; const float* dgu = w.DGU + off * eh;
    float* dx = w.DGATH + off * d;
    { GemmArgs g; g.A = dgg; g.lda = eh; g.a_trans = 1; g.B = x; g.ldb = d; g.C = m->g(o.exp_gate) + (int64_t)e * eh * d; g.ldc = d; g.M = eh; g.N = d; g.K = cnt; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = dgg; g.lda = eh; g.B = m->p(o.exp_gate) + (int64_t)e * eh * d; g.b_static = 1; g.ldb = d; g.C = dx; g.ldc = d; g.M = cnt; g.N = d; g.K = eh; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = dgu; g.lda = eh; g.a_trans = 1; g.B = x; g.ldb = d; g.C = m->g(o.exp_up) + (int64_t)e * eh * d; g.ldc = d; g.M = eh; g.N = d; g.K = cnt; g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    { GemmArgs g; g.A = dgu; g.lda = eh; g.B = m->p(o.exp_up) + (int64_t)e * eh * d; g.b_static = 1; g.ldb = d; g.C = dx; g.ldc = d; g.M = cnt; g.N = d; g.K = eh;
      g.epilogue = EPI_ACCUM; GN_TRY(gemm(m, g)); }
    off += cnt;
  }
  // ---- router: balance loss + softmax backward, then its own Linear
  const bool balance = seq_len > 0 && rows % seq_len == 0;
  const int64_t sequences = balance ? rows / seq_len : 1;
  if (balance) { moe_seq_counts_kernel<<<(unsigned)sequences, 256, 0, s>>>(w.SEQCNT, sv.SEL, seq_len, K, E); GN_LAUNCH_CHECK(); }
  else GN_CUDA(cudaMemsetAsync(w.SEQCNT, 0, sizeof(int32_t) * E, s));
  // the loss is a mean over the sequences of the whole call (the reference runs the batch as one forward), not of this pass
  const int64_t all_sequences = w.total_sequences > 0 ? w.total_sequences : sequences;
  moe_router_bwd_kernel<<<ceil_div(rows, 256), 256, 0, s>>>(w.GLOG, w.GPROB, sv.PR, w.SEQCNT, rows, balance ? seq_len : (int)rows, all_sequences, E, K,
                                                            balance ? (double)kMoEBalanceWeight : 0.0);
  GN_LAUNCH_CHECK();
  { GemmArgs g; g.A = w.GLOG; g.lda = E; g.a_trans = 1; g.B = Mn; g.ldb = d; g.C = m->g(o.router); g.ldc = d; g.M = E; g.N = d; g.K = (int)rows; g.epilogue = EPI_ACCUM; GN_TRY(gemm_dispatch(g, 0, s)); }
  { GemmArgs g; g.A = w.GLOG; g.lda = E; g.B = m->p(o.router); g.ldb = d; g.C = w.DMR; g.ldc = d; g.M = (int)rows; g.N = d; g.K = E; GN_TRY(gemm_dispatch(g, 0, s)); }
  moe_bwd_combine_kernel<<<grid_for(rows * d), 256, 0, s>>>(DM, w.DMS, w.DGATH, w.DMR, sv.POSI, rows, K, d); GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gnm
