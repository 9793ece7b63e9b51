// Fused glue kernels of the dense transformer: everything the reference does in
// plain Go loops around its backend calls (embedding gather, smear, residual
// mix, rotary, QK-norm, value-embedding gate, KV-cache writes, backout, and
// their backward forms).  Device pointers, asynchronous on `stream`.
#pragma once
#include "common.cuh"

namespace gn {

constexpr float kNormEps = 1e-6f;     // model/attention.go:11
constexpr float kQKScale = 1.2f;      // model/attention.go:14
constexpr int kVeGateChannels = 12;   // model/attention.go:18
constexpr float kVeGateScale = 3.0f;  // model/attention.go:21
constexpr int kSmearChannels = 24;    // model/helpers.go:13
constexpr float kSoftcap = 15.0f;     // model/transformer.go:11

// E[r] = rmsnorm(wte[ids[r]])    (model/transformer.go:255-256)
int embed_norm_launch(const int32_t* ids, const float* wte, float* E, int64_t rows, int d, cudaStream_t s);

// Smear (model/transformer.go:266-301, model/helpers.go:35-66):
//   X[b,t] = E[b,t] + lambda*sigmoid(Ws . E[b,t][0:24]) * prev     prev = E[b,t-1] for t >= 1,
//   prev_in[b*prev_mul] for t == 0 when prev_in != null (no smear at t == 0 otherwise).
// prev_out (nullable) receives E[b,T-1] at row b*prev_mul.  sig_out (nullable, [B,T-1]) the
// sigmoid of positions t >= 1.
int smear_launch(const float* E, float* X, const float* prev_in, float* prev_out, int prev_mul, float* sig_out, const float* Ws,
                 const float* lambda, int B, int T, int d, cudaStream_t s);

// Xin = rho[l]*X + chi[l]*X0 ; H = rmsnorm(Xin)   (model/transformer.go:312, model/block.go:39)
// Hh/Hl (nullable): the tf32 hi/lo split of H for the tensor-core product that consumes it.
int mix_norm_launch(const float* X, const float* X0, const float* rho, const float* chi, int layer, float* Xin, float* H, float* Hh, float* Hl,
                    int64_t rows, int d, cudaStream_t s);
// Y = rmsnorm(X) (+ optional split)
int norm_launch(const float* X, float* Y, float* Yh, float* Yl, int64_t rows, int d, cudaStream_t s);
// FP = X - lambda_b*BO (BO nullable) ; Y = rmsnorm(FP).  When sel != null row i reads X/BO row sel[i].
int backout_norm_launch(const float* X, const float* BO, const float* lambda_b, const int32_t* sel, float* FP, float* Y, float* Yh, float* Yl,
                        int64_t rows, int d, cudaStream_t s);

// Inference glue that also finishes a product left as split-K partial tiles, one block per row:
//   x = R[src] + sum of the partial tiles at row src        (src = sel[r] when sel != null, else r)
//   v = rho[layer]*x + chi[layer]*X0[r]   when X0 != null   (the residual mix of the next layer)
//   v = v - lambda_b*BO[src]              when BO != null   (the backout before the final norm)
//   y = rmsnorm(v), also written as its tf32 hi/lo split when Yh != null
// Xsum and V (nullable) receive x and v; each may alias R when sel == null.  Needs d % 4 == 0, d <= 4096.
struct SumNorm {
  const float* R = nullptr; Partials part; const int32_t* sel = nullptr;
  float* Xsum = nullptr;
  const float* X0 = nullptr; const float* rho = nullptr; const float* chi = nullptr; int layer = 0;
  const float* BO = nullptr; const float* lambda_b = nullptr;
  float* V = nullptr;
  float* Y = nullptr; float* Yh = nullptr; float* Yl = nullptr;
  int64_t rows = 0; int d = 0;
};
int sum_norm_launch(const SumNorm& p, cudaStream_t s);
// Decode step, T = 1: embedding + norm, smear against the cached previous embedding (updated in place), layer 0's mix
// and norm with the tf32 split of H.  prev [rows, d] is read and rewritten.
int decode_front_launch(const int32_t* ids, const float* wte, float* prev, const float* Ws, const float* lambda, const float* rho, const float* chi,
                        float* X0, float* Xin, float* H, float* Hh, float* Hl, int64_t rows, int d, cudaStream_t s);
inline bool sum_norm_supported(int d) { return d % 4 == 0 && d <= 4096; }

struct QkvPost {
  float* qkv = nullptr;        // [rows, (Hq+2Hkv)*D]  in: projections; out: q,k normalised, v final (in place)
  Partials part;               // when on: the projections are read from this unreduced product instead of qkv (needs D % 4 == 0)
  const float* H = nullptr;    // [rows, d] attention input (for the value-embedding gate)
  const int32_t* ids = nullptr;
  const float* ve_table = nullptr;  // [Vp, Hkv*D] or null
  const float* ve_gate = nullptr;   // [Hkv, 12] or null
  const float* cosv = nullptr; const float* sinv = nullptr;  // [positions, R/2]
  float* qk_rot = nullptr;     // train: [rows, (Hq+Hkv)*D] post-rotary pre-norm q,k
  float* ve_sig = nullptr;     // train: [rows, Hkv]
  float* kcache = nullptr; float* vcache = nullptr;  // inference: [cache_rows][Hkv][max_seq][D]
  const int32_t* pos = nullptr;  // per cache row: position of token t == 0 (null: 0)
  int cache_row_mul = 1;         // sequence b lives in cache row b*cache_row_mul
  int max_seq = 0;
  int B = 0, T = 0, Hq = 0, Hkv = 0, D = 0, R = 0, d = 0;
};
int qkv_post_launch(const QkvPost& p, cudaStream_t s);

// Copy the first `len` positions of cache row p*group to rows p*group+1 .. p*group+group-1
// for every layer/head, and the smear state likewise (model/kvcache.go:383-448).
int kv_replicate_launch(float* cache, int64_t layer_stride, int n_layer2, int64_t row_stride, int64_t head_stride, int Hkv, int D, int n_prompts,
                        int group, int len, float* prev, int d, int32_t* pos, cudaStream_t s);
int fill_i32_launch(int32_t* dst, int32_t value, int64_t n, cudaStream_t s);
int add_i32_launch(int32_t* dst, int32_t delta, int64_t n, cudaStream_t s);
int add_u32_launch(uint32_t* dst, uint32_t delta, cudaStream_t s);
// ctx[i] = pos[i] + 1
int ctx_from_pos_launch(const int32_t* pos, int32_t* ctx, int64_t n, cudaStream_t s);
// Engine bookkeeping per decode step (inference/engine.go:256-319,349-367): append the
// sampled column to the kept tokens of unfinished rows, mark rows that drew a terminal id.
int engine_step_launch(const int32_t* sampled, int32_t* out_tokens, int32_t* out_lengths, int32_t* done, int32_t* n_done, int rows, int max_tokens,
                       int bos, int aend, cudaStream_t s);

// ------------------------------------------------------------- backward glue
struct QkvPostBwd {
  float* dqkv = nullptr;        // [rows, (Hq+2Hkv)*D] in: dq,dk wrt normalised q,k and dv; out: wrt projections (in place)
  const float* qk_rot = nullptr;
  const float* ve_sig = nullptr; const float* ve_table = nullptr; const int32_t* ids = nullptr;
  float* ve_grad = nullptr;     // [Vp, Hkv*D] scatter-add target
  float* dpre = nullptr;        // [rows, Hkv] gradient at the gate pre-activation
  const float* cosv = nullptr; const float* sinv = nullptr;
  int B = 0, T = 0, Hq = 0, Hkv = 0, D = 0, R = 0;
};
int qkv_post_backward_launch(const QkvPostBwd& p, cudaStream_t s);
// dWg[h][c] += sum_r dpre[r,h]*H[r,c] (c < 12) ; dH[r,c] += sum_h dpre[r,h]*Wg[h][c]
int ve_gate_backward_launch(const float* dpre, const float* H, const float* Wg, float* dWg, float* dH, int64_t rows, int Hkv, int d, cudaStream_t s);

// Residual-mix backward (model/train_transformer.go:218-242):
//   *acc_rho += sum dXin*prevX ; *acc_chi += sum dXin*X0 ; dX = rho*dXin ; dX0 (+)= chi*dXin
int mix_backward_launch(const float* dXin, const float* prevX, const float* X0, const float* rho, const float* chi, int layer, float* dX, float* dX0,
                        int first, double* acc_rho, double* acc_chi, int64_t n, cudaStream_t s);
// acc[0] += sign * sum a*b
int dot_accumulate_launch(const float* a, const float* b, int64_t n, double sign, double* acc, cudaStream_t s);
// dst[i] (+)= alpha*src[i]
int axpy_launch(float* dst, const float* src, float alpha, const float* alpha_dev, float alpha_sign, int accumulate, int64_t n, cudaStream_t s);
// grad[index] += (float)acc[i] for the scalar parameters, then clears acc.
int scalar_flush_launch(float* grad, double* acc, int n, cudaStream_t s);

// Smear backward (model/train_transformer.go:269-305).  Xpost is the POST-smear activation:
// the reference's backward reads the tensor that smearAdd modified in place.
int smear_backward_launch(const float* dX, const float* Xpost, const float* E, const float* sig, const float* Ws, const float* lambda, float* dE,
                          float* dWs, double* dlambda_acc, int B, int T, int d, cudaStream_t s);
// draw = rmsnorm_backward(wte[ids], dE) scatter-added into wte_grad[ids]  (layers/linear.go:90-104)
int embed_backward_launch(const int32_t* ids, const float* wte, const float* dE, float* wte_grad, int64_t rows, int d, cudaStream_t s);

double* dummy_unused();

}  // namespace gn
