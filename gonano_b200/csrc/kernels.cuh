// Internal launchers (device pointers, asynchronous on `stream`).  Each returns a
// gn status after checking the launch.
#pragma once
#include "common.cuh"

namespace gn {

// ------------------------------------------------------------- elementwise.cu
enum EwOp { EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_SCALE, EW_ADD_SCALED, EW_NEG, EW_ABS, EW_SQUARE, EW_RELU2, EW_EXP, EW_SIGMOID,
            EW_TANH, EW_RSQRT, EW_SWIGLU };
int ew_launch(int op, float* dst, const float* a, const float* b, float factor, int64_t n, cudaStream_t s);
int swiglu_backward_launch(float* gg, float* ug, const float* gate, const float* up, const float* og, float clamp, int64_t n, cudaStream_t s);
// out (device) receives the result.
int reduce_sum_launch(const float* v, int64_t n, float* out, cudaStream_t s);
int reduce_max_launch(const float* v, int64_t n, float* out, cudaStream_t s);
int reduce_argmax_launch(const float* v, int64_t n, int64_t* out, cudaStream_t s);
int dot_launch(const float* a, const float* b, int64_t n, float* out, cudaStream_t s);
int softmax_rows_launch(float* dst, const float* src, int64_t rows, int cols, cudaStream_t s);
int rmsnorm_rows_launch(float* dst, const float* src, int64_t rows, int cols, float eps, cudaStream_t s);
// dx = dy/r - x*(dy.x)/(n r^3); when `add` != null: dx = add + that.
int rmsnorm_backward_launch(float* dx, const float* x, const float* dy, const float* add, int64_t rows, int cols, float eps, cudaStream_t s);
int fill_launch(float* dst, float value, int64_t n, cudaStream_t s);
int split_matrix_launch(const float* src, float* hi, float* lo, int64_t rows, int cols, int64_t ld, cudaStream_t s);

// --------------------------------------------------------------- optimizer.cu
// In-place updates (optimizer/optimizer.go:143-173, muon.go:23-173, sinkhorn.go:27-95).  `g` is overwritten (it holds the
// update matrix while the step runs).  `step` is AdamW's 1-based count.  Workspaces: *_workspace_bytes.
size_t muon_workspace_bytes(int rows, int cols);
size_t sinkhorn_workspace_bytes(int rows, int cols);
int adamw_launch(float* p, const float* g, float* m, float* v, int64_t n, int step, float lr, float beta1, float beta2, float eps, float wd, cudaStream_t s);
int muon_launch(float* p, float* g, float* mom, float* second, int rows, int cols, float lr, float momentum, int ns_steps, float beta2, float wd,
                void* workspace, int gemm_kind, cudaStream_t s);
int sinkhorn_launch(float* p, float* g, float* mom, int rows, int cols, float lr, float momentum, float gamma, int steps, float tau, float eps,
                    void* workspace, cudaStream_t s);

// --------------------------------------------------------------------- moe.cu
int topk_indices_launch(int32_t* dst, const float* scores, int rows, int count, int k, cudaStream_t s);
int moe_gate_topk_launch(const float* logits, const float* bias, float* probs, int32_t* sel, float* w, int rows, int experts, int k, cudaStream_t s);
int grouped_matmul_t_launch(float* dst, const float* input, const float* weight, const int32_t* counts_dev, int experts, int cols, int inner,
                            int64_t total_rows, cudaStream_t s);
int indexer_scores_launch(float* dst, const float* q, const float* k, const float* w, int rows, int blocks, int heads, int dim, cudaStream_t s);
int indexer_block_max_launch(float* dst, const float* scores, int rows, int blocks, int group, cudaStream_t s);
// dst[row, block] = scale[0] * (q[row] . key[block]), q [rows, dim], key [blocks, dim], scale a device scalar
int dot_scores_launch(float* dst, const float* q, const float* k, const float* scale, int rows, int blocks, int dim, cudaStream_t s);

// --------------------------------------------------------------- attention.cu
// Strided multi-head attention over token-major tensors.
//   q:  element (b, t, hq, d) at q[(b*q_bstride + t*q_tstride) + hq*D + d]
//   k/v: element (b, j, hk, d) at k[b*kv_bstride + j*kv_tstride + hk*kv_hstride + d]
//   out: like q with its own strides; lse [B, Hq, Tq] (nullable)
//   query i of row b sits at absolute position offset[b] (or offset0 when offsets == null) + i.
struct AttnShape {
  int B = 1, Hq = 1, Hkv = 1, D = 0, Tq = 0, Tk = 0;
  int64_t q_bstride = 0, q_tstride = 0;
  int64_t q_hstride = 0, o_hstride = 0;   // 0: heads are D apart inside a token (the usual [token, head, D] layout)
  int64_t kv_bstride = 0, kv_tstride = 0, kv_hstride = 0;
  int64_t o_bstride = 0, o_tstride = 0;
  int window = -1;
  int offset0 = 0;
  int key_ratio = 1;   // > 1: keys are blocks of key_ratio positions; the query at position p sees the blocks before its own, j < p / key_ratio (tensor-core forward only)
  const int32_t* segment_ids = nullptr;  // [Tk] shared by all rows (Tier A only)
  int seg_len = 0;
  int tensor = 0;   // 1: head_dim 128 may run on the tensor cores in 3xTF32 (forward and backward)
  // the last key a query at position pos sees / the first position that sees key j (before the window and the segment mask)
  __host__ __device__ int last_key(int pos) const { return key_ratio == 1 ? pos : pos / key_ratio - 1; }
  __host__ __device__ int first_position(int key) const { return key_ratio == 1 ? key : (key + 1) * key_ratio; }
  __host__ __device__ int64_t q_head(int h) const { return (int64_t)h * (q_hstride ? q_hstride : D); }
  __host__ __device__ int64_t o_head(int h) const { return (int64_t)h * (o_hstride ? o_hstride : D); }
};
// head_dim 128 tensor-core kernels (attention_mma.cu); reached through the two launches below when sh.tensor is set.
bool attention_mma_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4);
int attention_mma_forward(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s);
// compressed attention building blocks (compress.cu)
int compressor_pool_launch(const float* logits, const float* bias, const float* value, int B, int T, int C, int ratio, float* compressed, float* probabilities,
                           cudaStream_t s);
// dlogits and dvalue ([B, T, C], every element written) and the bias gradient (accumulated) from the gradient of the compressed output
int compressor_pool_backward_launch(const float* value, const float* probabilities, const float* compressed, const float* grad_compressed, int B, int T, int C,
                                    int ratio, float* grad_logits, float* grad_value, float* grad_bias, cudaStream_t s);
// compressForward / compressBackward over every kv head: logits [B * T, C] = hidden W^T; key / value [B, H, T, C]; probabilities [B, blocks, ratio, C]
int compress_heads_launch(const float* logits, const float* bias, const float* key, const float* value, int B, int H, int T, int C, int ratio, float* key_c,
                          float* value_c, float* probabilities, cudaStream_t s);
int compress_heads_backward_launch(const float* key, const float* value, const float* probabilities, const float* key_c, const float* value_c,
                                   const float* grad_key_c, const float* grad_value_c, int B, int H, int T, int C, int ratio, float* grad_logits, float* grad_key,
                                   float* grad_value, float* grad_bias, cudaStream_t s);
// selection == nullptr: every block before the query's own; else the token's selected blocks ([B * Hkv, T, topk] with counts [B * Hkv, T])
// (token t stands at position offset + t: offset > 0 is the cached inference form)
int compressed_attention_launch(const float* q, const float* kc, const float* vc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* out, float* lse,
                                const int32_t* selection, const int32_t* counts, int topk, int offset, cudaStream_t s);
// (select_bits: optional scratch of B * Hkv * ceil(blocks / 32) * T words for the selected-block form: the selection as bits per token)
// backward, dense (selection null) or over selected blocks: dq, dkc, dvc are accumulated into; rowcorr nullable (then delta_scratch [B * Hq * T] is used)
int compressed_attention_backward_launch(const float* q, const float* kc, const float* vc, const float* dout, const float* lse, const float* rowcorr,
                                         float* delta_scratch, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* dq, float* dkc, float* dvc,
                                         const int32_t* selection, const int32_t* counts, int topk, cudaStream_t s,
                                         uint32_t* select_bits = nullptr);
int attention_merge_launch(const float* oa, const float* la, const float* ob, const float* lb, int64_t rows, int D, float* out, float* lse, cudaStream_t s);
// score part of the indexer's backward: gq [rows, heads, dim], gk [blocks, heads, dim] overwritten, gw [heads] accumulated; wpart [rows, heads] scratch
// (kpart: optional room for kpart_planes partial copies of gk, used when the blocks are too few to fill the machine)
int indexer_scores_backward_launch(const float* gs, const float* q, const float* key, const float* w, int rows, int blocks, int heads, int dim, float* gq, float* gk,
                                   float* gw, float* wpart, cudaStream_t s, float* kpart = nullptr, int kpart_planes = 0);
// the indexer's distillation: target [B * Hkv, T, blocks] from the main attention logits; grad = (masked softmax(scores) - target) * weight, row r = token r % seq
// (qsum: optional scratch of B * Hkv * T * D + 1 floats: the long-sequence form sums the group's queries first and takes one tiled product per (batch, kv head))
int distillation_target_launch(const float* q, const float* kc, int B, int Hq, int Hkv, int T, int D, int blocks, int ratio, float* target, cudaStream_t s,
                               float* qsum = nullptr);
int distillation_grad_launch(const float* scores, const float* target, const int32_t* candidates, const int32_t* candidate_counts, int cap, int64_t rows, int blocks,
                             int seq, int ratio, float weight, float* grad, cudaStream_t s);
// two-level selection: gmax [tokens, ceil(blocks / pool)] and chosen [tokens, max(1, ceil(budget / pool))] are scratch; candidates [tokens, that * pool]
int select_hierarchical_launch(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int pool, int budget, float* gmax, int32_t* chosen,
                               int32_t* selection, int32_t* counts, int32_t* candidates, int32_t* candidate_counts, cudaStream_t s);
int select_within_pool_launch(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, const int32_t* candidates,
                              const int32_t* candidate_counts, int cap, int32_t* selection, int32_t* counts, cudaStream_t s);
int select_blocks_launch(const float* scores, int tokens, int blocks, int offset, int ratio, int topk, int32_t* selection, int32_t* counts, cudaStream_t s);
// decode attention over the prompt shared by the rows of a group, head_dim 128, on mma.sync (attention_mma.cu): one
// partial-result slot per 32-key tile and (row, head), as attn_decode_prefix_kernel writes them
int attention_mma_decode_prefix(const float* q, int64_t q_rstride, const float* kcache, const float* vcache, int64_t row_stride, int64_t head_stride,
                                const int32_t* ctx_len, int rows, int Hq, int Hkv, int window, int group, int prefix_len, float* part_acc, float* part_ms,
                                int nslots, cudaStream_t s);
// head_dim 128 forward on tcgen05 (attention_tcgen05.cu); preferred over the mma.sync kernel when sh.tensor is set.
bool attention_tc_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3);
int attention_tc_forward(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s);
bool attention_tc_backward_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4);
int attention_tc_backward(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                          float* dq, float* dk, float* dv, int accumulate, cudaStream_t s);
void attention_tc_enable(int on);   // 0: keep head_dim 128 attention on the mma.sync kernels
int attention_mma_backward(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                           float* dq, float* dk, float* dv, int accumulate, cudaStream_t s);
int attention_forward_launch(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s);
// Gradients: dq like q (strides of q), dk/dv like k/v.  accumulate != 0 adds into them.
int attention_backward_launch(const AttnShape& sh, const float* q, const float* k, const float* v, const float* out, const float* dout,
                              const float* lse, const float* row_correction, float* dq, float* dk, float* dv, int accumulate,
                              float* delta_scratch, cudaStream_t s);
int attention_split_launch(const AttnShape& sh, const float* q, const float* k, const float* v, int kstart, int kend, float* acc, float* mx,
                           float* sm, cudaStream_t s);
int attention_combine_launch(const float* acc, const float* mx, const float* sm, int parts, int ql, int hd, float* out, float* lse, cudaStream_t s);
// Decode: one query token per row over the KV cache [row][hk][max_seq][D]; ctx_len[row] keys (device array).
int attention_decode_launch(const float* q, int64_t q_rstride, const float* kcache, const float* vcache, int64_t row_stride, int64_t head_stride,
                            const int32_t* ctx_len, int rows, int Hq, int Hkv, int D, int window, float* out, int64_t o_rstride,
                            float* part_acc, float* part_ms, int splits, cudaStream_t s,
                            float* out_hi = nullptr, float* out_lo = nullptr,    // optional tf32 hi/lo split of the output, same pitch
                            int group = 1, int prefix_len = 0,
                            float* lse_out = nullptr);   // optional [rows, Hq] log-sum-exp; written by the combine pass, so splits must be > 1
// group > 1 and prefix_len > 0: rows come in groups of `group` whose first prefix_len cached positions are identical
// copies (a replicated prompt); those keys are read once per group.  The partial buffers then need
// attention_decode_prefix_splits(...) + splits slots per (row, query head).
int attention_decode_splits(int rows, int Hkv, int max_ctx);
void attention_decode_prefix_mode(int mode);   // -1 automatic, 0 off, 1 on wherever the pass applies
int attention_decode_prefix_splits(int rows, int group, int Hq, int Hkv, int D, int prefix_len);

// ----------------------------------------------------------------- sampler.cu
// Optional bookkeeping of the rollout engine folded into the sampler (one thread per row; all pointers device memory).
// pos != null: the Philox step of row r is pos[r] - pos_base + advance, and afterwards pos[r] += advance,
// ctxlen[r] = pos[r] + 1.  done != null: the engine step (keep the token or finish the row on bos / aend).
struct SampleTail {
  int32_t* pos = nullptr; int32_t* ctxlen = nullptr; int pos_base = 0; int advance = 0;
  int32_t* out_tokens = nullptr; int32_t* out_lengths = nullptr; int32_t* out_masks = nullptr; int32_t* done = nullptr; int32_t* n_done = nullptr;
  int max_tokens = 0, bos = -1, aend = -1;
  // forced-token ring per row (inference/engine.go:262-273): a queued token overrides the sampled one (mask 0)
  int32_t* forced_head = nullptr; int32_t* forced_len = nullptr; int32_t* forced_buf = nullptr; int forced_cap = 0;
  // thinking trace (inference/engine.go:301-314): inside <|think_start|> ... <|think_end|> reasoning tokens are counted
  // and, once `thinking_budget` of them have been emitted, <|think_end|> is queued
  int32_t* in_think = nullptr; int32_t* think_count = nullptr; int thinking = 0, thinking_budget = 0, think_start = -1, think_end = -1;
  int32_t* step_mask = nullptr;   // this step's mask per row (1 sampled, 0 forced)
};
int sample_launch(const float* logits, int rows, int vocab, int logits_row_div, const float* uniforms, const uint64_t* seeds_dev, int group,
                  const uint32_t* step_dev, uint32_t step_host, float temperature, int top_k, int32_t* out, cudaStream_t s,
                  const SampleTail* tail = nullptr);

// -------------------------------------------------------------------- loss.cu
// row_loss: [rows] double scratch; loss_out: device double.  bad_targets: null or a device counter that receives the
// number of targets outside {-1} and [0, vocab) (such rows are treated as ignored, never dereferenced).
int pg_loss_launch(const float* logits, const int32_t* targets, const float* adv, int64_t rows, int vocab, int64_t ld, int seq_len, float norm,
                   float softcap, float* nll, float* dlogits, int64_t ldd, double* row_loss, double* loss_out, int accumulate_loss, cudaStream_t s,
                   int* bad_targets = nullptr, int64_t row_offset = 0);   // row r's advantage is adv[(row_offset + r) / seq_len]
int advantage_launch(const float* rewards, int groups, int group, int mode, float* adv, cudaStream_t s);
int distillation_launch(const float* student, const float* teacher, const int32_t* mask, int64_t rows, int vocab, float temperature, float scale,
                        float* losses, float* grad, double* row_loss, double* loss_sum, cudaStream_t s);

}  // namespace gn
