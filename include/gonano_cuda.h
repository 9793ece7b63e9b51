/*
 * gonano_cuda.h - C ABI of the B200 (sm_100a) CUDA backend for gonano's RL step.
 *
 * The library replaces, for the reinforcement-learning step of gonano
 * (trainer/rl.go driven by cmd/chat_rl), the work that the reference routes
 * through its numeric backend interface `kernels.Backend`
 * (kernels/backend.go:285-297) and through the Go loops around it.
 *
 * Two tiers:
 *
 *   Tier A  one entry point per `kernels.Backend` method, same argument order
 *           and meaning.  Pointers may be host or device memory (detected per
 *           call); host buffers are staged through device memory and the call
 *           returns when the result is back.  This is what a cgo shim that
 *           implements `kernels.Backend` binds.
 *
 *   Tier B  a resident session: the model's parameters, KV cache, activations
 *           and gradients live in device memory, and whole phases of the RL
 *           step run without crossing the host boundary.  This is what
 *           model/, inference/engine.go and trainer/rl.go call when the
 *           selected backend also offers the resident interface.
 *
 * Conventions
 *   - every function returns a status (GN_OK == 0); gn_last_error() gives the
 *     message of the calling thread's last failure.  Nothing aborts or traps.
 *   - matrices are contiguous, row-major float32; token ids are int32
 *     (tensors/tensor.go:10-17, tensors/ids.go:8-11).
 *   - Tier A is safe to call from any number of OS threads (the reference
 *     calls its backend from many goroutines, model/attention.go:311-320);
 *     calls are serialised on one internal lock per process and run on the CUDA device that was
 *     current at the first of them (another current device is refused with GN_ERR_UNSUPPORTED;
 *     other devices are reached through a gn_ctx).
 *   - Tier B objects are single-caller: one thread per gn_ctx at a time.  Every gn_ctx (and
 *     Tier A) owns its scratch memory per (device, stream): contexts on different streams or
 *     devices of one process do not share buffers, so they may run concurrently.
 *   - there is no CPU fallback: without a CUDA device every compute call
 *     fails with GN_ERR_CUDA.
 */
#ifndef GONANO_CUDA_H
#define GONANO_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GN_OK 0
#define GN_ERR_INVALID 1 /* bad argument */
#define GN_ERR_CUDA 2    /* CUDA runtime/driver error, or no device */
#define GN_ERR_COMM 3    /* collective communication error */
#define GN_ERR_TIMEOUT 4 /* a bounded device-side wait ran out */
#define GN_ERR_NOMEM 5
#define GN_ERR_UNSUPPORTED 6 /* valid request outside what this library implements (e.g. training a latent-preset model) */

const char* gn_last_error(void);
/* Library version string. */
const char* gn_version(void);
/* Number of visible CUDA devices (0 when none; never fails). */
int gn_device_count(void);

/* ===================================================================== *
 * Tier A - kernels.Backend                                              *
 * ===================================================================== */

/* Elementwise (kernels/backend.go:21-67).  dst may alias a source. */
int gn_add(float* dst, const float* left, const float* right, int64_t n);
int gn_subtract(float* dst, const float* left, const float* right, int64_t n);
int gn_multiply(float* dst, const float* left, const float* right, int64_t n);
int gn_divide(float* dst, const float* left, const float* right, int64_t n);
int gn_scale(float* dst, const float* src, float factor, int64_t n);
int gn_add_scaled(float* dst, const float* base, const float* scaled, float factor, int64_t n);
int gn_negate(float* dst, const float* src, int64_t n);
int gn_abs(float* dst, const float* src, int64_t n);
int gn_square(float* dst, const float* src, int64_t n);
int gn_relu_squared(float* dst, const float* src, int64_t n);
int gn_swiglu(float* dst, const float* gate, const float* up, float clamp, int64_t n);
/* Overwrites gate_grad and up_grad (kernels/backend.go:54-57). */
int gn_swiglu_backward(float* gate_grad, float* up_grad, const float* gate, const float* up, const float* out_grad,
                       float clamp, int64_t n);
int gn_exp(float* dst, const float* src, int64_t n);
int gn_sigmoid(float* dst, const float* src, int64_t n);
int gn_tanh(float* dst, const float* src, int64_t n);
int gn_rsqrt(float* dst, const float* src, int64_t n);

/* Reductions (kernels/backend.go:70-78); the Go methods return the value, here it
 * comes back through `out` (host memory). Max of an empty slice is 0, ArgMax 0. */
int gn_sum(const float* values, int64_t n, float* out);
int gn_max(const float* values, int64_t n, float* out);
int gn_argmax(const float* values, int64_t n, int64_t* out);

/* Linear algebra (kernels/backend.go:82-93). */
int gn_matmul(float* dst, const float* left, const float* right, int rows, int cols, int inner);
int gn_matmul_transposed(float* dst, const float* left, const float* right, int rows, int cols, int inner);
int gn_dot_product(const float* left, const float* right, int64_t n, float* out);

/* Indexer (kernels/backend.go:103-116). */
int gn_indexer_scores(float* dst, const float* query, const float* key, const float* weight, int rows, int blocks,
                      int heads, int dim);
int gn_indexer_block_max(float* dst, const float* scores, int rows, int blocks, int group_size);
/* The score part of SparseIndexer.Backward (model/indexer.go:107-151) for one key set: grad_query [rows, heads, dim] and
 * grad_key [blocks, heads, dim] are overwritten, grad_weight [heads] is accumulated into.  dim <= 128. */
int gn_indexer_scores_backward(const float* grad_scores, const float* query, const float* key, const float* weight, int rows, int blocks, int heads, int dim,
                               float* grad_query, float* grad_key, float* grad_weight);

/* Building blocks of the compressed ("flash") attention layers, inference forward.  These bypass kernels.Backend in the
 * reference (plain Go loops in model/): ChannelCompressor.Forward (model/compress.go:93-177; hidden [batch, seq, embed],
 * value [batch, seq, channels], logit_weight [channels, embed], bias [ratio, channels] -> compressed [batch,
 * ceil(seq / ratio), channels], probabilities nullable [batch, blocks, ratio, channels]); compressedAttentionForward
 * without a segment mask (model/compress_attention.go:624-673; query [batch, n_head, seq, head_dim], key_c / value_c
 * [batch, n_kv_head, blocks, head_dim]; the queries of block b attend blocks 0 .. b-1, block 0 yields zeros and
 * lse = -inf); mergeAttentionBranches (:440-466); SelectBlocks (model/indexer.go:186-206; selection [tokens, topk]
 * padded with -1, counts [tokens]; descending score, ties toward the smaller block index). */
int gn_compressor_forward(const float* hidden, const float* value, const float* logit_weight, const float* bias, int batch, int seq, int embed,
                          int channels, int ratio, float* compressed, float* probabilities);
/* compressForward / compressBackward (model/compress_attention.go:562-622, 1182-1209), no segment mask: the compressor over the
 * keys and the values of every kv head.  hidden [batch, seq, embed], key / value [batch, n_kv_head, seq, head_dim] ->
 * key_c / value_c [batch, n_kv_head, blocks, head_dim]; the block softmax depends on the hidden state alone, so one logit
 * product and one set of probabilities [batch, blocks, ratio, head_dim] (nullable in the forward) serve every head.  The
 * backward overwrites grad_hidden, grad_key, grad_value and accumulates into grad_weight, grad_bias. */
int gn_compress_forward(const float* hidden, const float* key, const float* value, const float* logit_weight, const float* bias, int batch, int n_kv_head, int seq,
                        int embed, int head_dim, int ratio, float* key_c, float* value_c, float* probabilities);
int gn_compress_backward(const float* hidden, const float* key, const float* value, const float* logit_weight, const float* probabilities, const float* key_c,
                         const float* value_c, const float* grad_key_c, const float* grad_value_c, int batch, int n_kv_head, int seq, int embed, int head_dim,
                         int ratio, float* grad_hidden, float* grad_key, float* grad_value, float* grad_weight, float* grad_bias);
/* ChannelCompressor.Backward (model/compress.go:182-237): probabilities and compressed are gn_compressor_forward's
 * outputs; grad_hidden [batch, seq, embed] and grad_value [batch, seq, channels] are overwritten, grad_weight
 * [channels, embed] and grad_bias [ratio, channels] accumulated. */
int gn_compressor_backward(const float* hidden, const float* value, const float* logit_weight, const float* probabilities, const float* compressed,
                           const float* grad_compressed, int batch, int seq, int embed, int channels, int ratio, float* grad_hidden, float* grad_value,
                           float* grad_weight, float* grad_bias);
int gn_compressed_attention_forward(const float* query, const float* key_c, const float* value_c, int batch, int n_head, int n_kv_head, int seq,
                                    int head_dim, int blocks, int ratio, float* out, float* lse);
/* The same for `seq` new tokens at positions position_offset .. position_offset + seq - 1 over `blocks` cached compressed
 * blocks: the dense global branch of the cached inference path (forwardCompressed, model/compress_attention.go:962-1003);
 * token t takes min((position_offset + t) / ratio, blocks) blocks.  One decode step is seq = 1. */
int gn_compressed_attention_forward_at(const float* query, const float* key_c, const float* value_c, int batch, int n_head, int n_kv_head, int seq, int head_dim,
                                       int blocks, int ratio, int position_offset, float* out, float* lse);
/* compressedAttentionBackward (model/compress_attention.go:735-781): dq, dkc, dvc are accumulated into; row_correction
 * (nullable, [batch, n_head, seq]) is the reference's rowCorrection for a branch whose output was merged with another. */
int gn_compressed_attention_backward(const float* query, const float* key_c, const float* value_c, const float* out_grad, const float* lse,
                                     const float* row_correction, int batch, int n_head, int n_kv_head, int seq, int head_dim, int blocks, int ratio,
                                     float* dq, float* dkc, float* dvc);
/* compressedAttentionForwardSparse (model/compress_attention.go:321-374): selection [batch * n_kv_head, seq, topk] block
 * indices, counts [batch * n_kv_head, seq]; block indices lie in [0, blocks) (an entry outside is ignored). */
int gn_compressed_attention_sparse_forward(const float* query, const float* key_c, const float* value_c, const int32_t* selection, const int32_t* counts,
                                           int batch, int n_head, int n_kv_head, int seq, int head_dim, int blocks, int topk, float* out, float* lse);
/* compressedAttentionBackwardSparse (model/compress_attention.go:376-433): the same over each token's selected blocks. */
int gn_compressed_attention_sparse_backward(const float* query, const float* key_c, const float* value_c, const float* out_grad, const float* lse,
                                            const float* row_correction, const int32_t* selection, const int32_t* counts, int batch, int n_head, int n_kv_head,
                                            int seq, int head_dim, int blocks, int topk, float* dq, float* dkc, float* dvc);
int gn_attention_merge(const float* out_a, const float* lse_a, const float* out_b, const float* lse_b, int64_t rows, int head_dim, float* out,
                       float* lse);
int gn_select_blocks(const float* scores, int tokens, int blocks, int position_offset, int ratio, int topk, int32_t* selection, int32_t* counts);
/* The two-level selection over a score matrix (SparseIndexer.selectFromScoreMatrix / selectRowBlockMax, model/indexer.go:358-381,
 * 442-513): super-blocks of `pool` entries ranked by their maximum over the allowed entries, the best
 * max(1, ceil(candidate_budget / pool)) of them give the candidates [tokens, gn_hierarchical_cap(pool, candidate_budget)]
 * (-1 padded; nullable together with candidate_counts), the selection is the top-k of the candidates.  gn_select_blocks_within_pool
 * is selectWithinPool (model/indexer.go:547-613) over the same score matrix: top-k of a given candidate list, entries outside
 * [0, allowed) dropped. */
/* The indexer's distillation (model/compress_attention.go:120-196, 203-231, 266-303).  Target [batch * n_kv_head, seq, blocks]: per
 * token the softmax over its allowed blocks of the main attention logits averaged over the query heads of the group.  Gradient
 * with respect to the index scores [rows, blocks] (row r is token r % seq): (softmax over the allowed blocks - target) * weight;
 * with candidates [rows, cap] (nullable) scores and target are first restricted to each row's candidate list, the target
 * renormalised inside it. */
int gn_indexer_distillation_target(const float* query, const float* key_c, int batch, int n_head, int n_kv_head, int seq, int head_dim, int blocks, int ratio,
                                   float* target);
int gn_indexer_distillation_grad(const float* scores, const float* target, const int32_t* candidates, const int32_t* candidate_counts, int cap, int64_t rows,
                                 int blocks, int seq, int ratio, float weight, float* grad_scores);
int gn_hierarchical_cap(int pool, int candidate_budget);
int gn_select_blocks_hierarchical(const float* scores, int tokens, int blocks, int position_offset, int ratio, int topk, int pool, int candidate_budget,
                                  int32_t* selection, int32_t* counts, int32_t* candidates, int32_t* candidate_counts);
int gn_select_blocks_within_pool(const float* scores, int tokens, int blocks, int position_offset, int ratio, int topk, const int32_t* candidates,
                                 const int32_t* candidate_counts, int cap, int32_t* selection, int32_t* counts);

/* MoE (kernels/backend.go:119-141).  Indices are exact: descending score, ties
 * toward the smaller index. */
int gn_topk_indices(int32_t* dst, const float* scores, int rows, int count, int k);
int gn_moe_gate_topk(const float* logits, const float* bias, float* probs, int32_t* selected, float* selected_weights,
                     int rows, int experts, int k);
int gn_grouped_matmul_transposed(float* dst, const float* input, const float* weight, const int32_t* token_counts,
                                 int experts, int cols, int inner);

/* Rows (kernels/backend.go:145-153). */
int gn_softmax_last_dim(float* dst, const float* src, int64_t rows, int cols);
int gn_rmsnorm_last_dim(float* dst, const float* src, int64_t rows, int cols, float epsilon);

/* Attention for one (batch, head) (kernels/backend.go:167-283).
 * window < 0: full causal context, else left sliding-window width.
 * segment_ids: NULL or one id per key position (length key_len). */
typedef struct gn_attention_params {
  const float* query;  /* [query_len, head_dim] */
  const float* key;    /* [key_len, head_dim] */
  const float* value;  /* [key_len, head_dim] */
  int32_t query_len, key_len, head_dim, position_offset, window;
  const int32_t* segment_ids;
} gn_attention_params;

/* out [query_len, head_dim]; lse NULL or [query_len]. */
int gn_attention_forward(const gn_attention_params* p, float* out, float* lse);
/* One key shard [key_start, key_end): overwrites acc [query_len, head_dim], max and sum [query_len]. */
int gn_attention_forward_split(const gn_attention_params* p, int key_start, int key_end, float* acc, float* maximum,
                               float* sum);
/* Partials packed shard-major: acc [parts, query_len, head_dim], maximum/sum [parts, query_len]. */
int gn_attention_combine(const float* acc, const float* maximum, const float* sum, int parts, int query_len,
                         int head_dim, float* out, float* lse);
/* ACCUMULATES into dq [query_len, head_dim], dk, dv [key_len, head_dim] (kernels/backend.go:217-220).
 * output is the forward output; row_correction NULL or [query_len] (kernels/backend.go:205-211). */
int gn_attention_backward(const gn_attention_params* p, const float* output, const float* out_grad, const float* lse,
                          const float* row_correction, float* dq, float* dk, float* dv);

/* attentionForwardWindowed / attentionBackwardWindowed (model/compress_attention.go:488-541), no segment mask: the local
 * sliding-window branch of a compressed attention layer for every (batch, query head).  query / out / out_grad / dq
 * [batch, n_head, seq, head_dim], key / value / dk / dv [batch, n_kv_head, seq, head_dim], lse / row_correction
 * [batch, n_head, seq].  The backward accumulates into dq, dk, dv; it takes the (merged) log-sum-exp and either the row
 * correction dO . O of the merged output or, when that is NULL, the forward output. */
int gn_attention_windowed_forward(const float* query, const float* key, const float* value, int batch, int n_head, int n_kv_head, int seq, int head_dim,
                                  int position_offset, int window, float* out, float* lse);
int gn_attention_windowed_backward(const float* query, const float* key, const float* value, const float* output, const float* out_grad, const float* lse,
                                   const float* row_correction, int batch, int n_head, int n_kv_head, int seq, int head_dim, int position_offset, int window,
                                   float* dq, float* dk, float* dv);

/* ===================================================================== *
 * Stand-alone kernels of the RL step (host or device pointers)          *
 * ===================================================================== */

/* inference/sampler.go:16-77 with tensors/random.go:60-80: per row, keep the
 * values >= the top_k-th largest (top_k <= 0 or >= vocab keeps all), add Gumbel
 * noise -log(-log(u)) to value/temperature and take the first maximum;
 * temperature <= 0 is a plain first-maximum argmax.  u comes from `uniforms`
 * ([rows, vocab], one per vocabulary entry, values <= 0 read as 1e-12) or, when
 * uniforms is NULL, from the counter generator Philox-4x32-10 keyed by
 * seeds[row / group] with counter (column/4, row % group, step, 0).
 * Indices are bit-exact against the CPU statement of the same rule. */
int gn_sample_next_token(const float* logits, int rows, int vocab, const float* uniforms, const uint64_t* seeds,
                         int group, uint32_t step, float temperature, int top_k, int32_t* out_ids);

/* cmd/chat_rl/main.go:137-154: advantages of `groups` groups of `group` rewards.
 * mode 0: reward - group mean (the reference).  mode 1: (reward - mean) /
 * (population std + 1e-6). */
int gn_group_advantage(const float* rewards, int groups, int group, int mode, float* advantages);

/* trainer/rl.go:23-56 at given logits [rows, vocab]: per-row
 * nll = logsumexp(row) - row[target] (0 where target == -1),
 * loss = sum nll * adv[row / seq_len] / norm, and
 * dlogits = (softmax - onehot) * adv / norm (0 on ignored rows).  When
 * softcap > 0 the gradient is also multiplied by 1 - (logit / softcap)^2, the
 * backward of the logit softcap (tensors/backward.go:108-116).  dlogits may
 * alias logits (in place) or be NULL (loss only).  nll may be NULL.  loss may be host or
 * device memory.  A target outside {-1} and [0, vocab) is never dereferenced: the call
 * fails with GN_ERR_INVALID (the reference panics on the slice bound). */
int gn_pg_loss_backward(const float* logits, const int32_t* targets, const float* advantages, int64_t rows, int vocab,
                        int seq_len, float norm, float softcap, float* nll, float* dlogits, double* loss);

/* tensors.DistillationLossPerPosition and DistillationGrad (tensors/loss.go:84-213) in one pass: per position the
 * cross-entropy of softmax(teacher / temperature) under softmax(student / temperature) (the teacher's entropy is
 * constant and dropped), and d loss / d student = (softmax(student/T) - softmax(teacher/T)) * scale / T.
 * mask: NULL or one int32 per row, 0 = masked (loss 0, zero gradient).  temperature <= 0 reads as 1.
 * losses [rows], dstudent [rows, vocab], loss_sum (sum over the valid rows) and valid (their count) are optional. */
int gn_distillation_loss_backward(const float* student, const float* teacher, const int32_t* mask, int64_t rows, int vocab,
                                  float temperature, float scale, float* losses, float* dstudent, double* loss_sum, int64_t* valid);

/* gn_pg_loss_backward for callers that must not allocate.  No counterpart in the reference:
 * it exists for hosts that own all device memory themselves (a process whose own arena spans
 * the GPU, a loop that cannot afford cudaMalloc's device-wide synchronisation or a late
 * out-of-memory failure).  The per-row scratch lives in a fixed array inside the library, so
 * the call makes no allocation at all.  Consequences:
 *   - at most GN_STATIC_LOSS_MAX_ROWS rows per call (more is refused with GN_ERR_INVALID);
 *   - logits, targets, advantages, nll and dlogits must be device pointers (no host staging);
 *     loss may be host or device; stream is a cudaStream_t (NULL = default stream); the call
 *     returns after the loss has been written;
 *   - the array is shared by every call on a GPU and keeps the last call's values: what must
 *     start at zero is cleared per call, and calls that overlap on one GPU race - serialise them;
 *   - the first call on each device looks up the array's device address; make that call at
 *     start-up.  The call synchronises the stream before it returns, so it cannot run inside a
 *     stream capture.
 * gn_static_loss_max_rows() returns the row limit the loaded library was built with. */
#define GN_STATIC_LOSS_MAX_ROWS 65536
int gn_static_loss_max_rows(void);
int gn_pg_loss_backward_static(const float* logits, const int32_t* targets, const float* advantages, int64_t rows,
                               int vocab, int seq_len, float norm, float softcap, float* nll, float* dlogits,
                               double* loss, void* stream);

/* ===================================================================== *
 * Tier B - resident session                                             *
 * ===================================================================== */

typedef struct gn_ctx gn_ctx;
typedef struct gn_model gn_model;

/* model.Config fields of the dense preset and of the latent preset (model/config.go:9-124).
 * The last eight are zero for a dense model. */
typedef struct gn_config {
  int32_t sequence_len;  /* SequenceLen: rotary table covers 10x this; window sizes derive from it */
  int32_t vocab_size;    /* VocabSize (padded to a multiple of 64 internally, model/config.go:619-624) */
  int32_t n_layer;       /* NumLayer */
  int32_t n_head;        /* NumHead */
  int32_t n_kv_head;     /* NumKVHead */
  int32_t embed_dim;     /* EmbedDim */
  int32_t rotary_dims;   /* RotaryDims (<= 0: whole head) */
  char window_pattern[16]; /* WindowPattern, e.g. "SSSL" (model/config.go:629-645); empty = "L" */
  /* DeepSeekMoE feed-forward (model/config.go:92-123): n_experts > 0 replaces the dense MLP of every block by a
   * shared SwiGLU expert plus routed experts (model/block.go:23-25).  Inference only in this library. */
  int32_t n_experts;          /* NumExperts */
  int32_t experts_per_token;  /* NumExpertsPerToken (<= 0: 2) */
  int32_t expert_hidden;      /* ExpertHiddenDim (<= 0: embed_dim) */
  int32_t shared_hidden;      /* SharedExpertHiddenDim (<= 0: expert_hidden) */
  float moe_clamp;            /* MoEClamp (0: 10) */
  float moe_scale;            /* MoEScale (0: 1) */
  /* Absorbed multi-head latent attention (model/config.go:80-91): mla_latent > 0 enables it; value embeddings are
   * then off (model/transformer.go:73).  Inference only in this library. */
  int32_t mla_latent;         /* MLALatent */
  int32_t mla_rotary_dims;    /* MLARotaryDims (<= 0: min(head_dim/2, 64), even) */
} gn_config;

/* device: CUDA ordinal.  stream: a cudaStream_t to run on, or NULL for a
 * stream the context creates. */
int gn_ctx_create(int device, void* stream, gn_ctx** out);
int gn_ctx_destroy(gn_ctx* ctx);
int gn_ctx_sync(gn_ctx* ctx);
/* Number of this library's kernels launched through the context so far. */
int gn_ctx_launch_count(gn_ctx* ctx, int64_t* out);
/* Select the GEMM path: 0 = SIMT float32, 1 = tcgen05 3xTF32 (default when built). */
int gn_ctx_set_gemm(gn_ctx* ctx, int kind);

/* Tuning and test switches (no counterpart in the reference).  ctx == NULL addresses the stand-alone
 * (Tier A) calls, after the first of them has run.  Names:
 *   "decode_graph"           1 (default) replays the decode step from a CUDA graph, 0 keeps it eager
 *   "head_chunk_rows"        16384 (default): token rows whose logits exist at once in the training pass
 *   "optimizer_lanes"        4 (default): streams the independent tensors of an optimizer step are spread over (1..4)
 *   "optimizer_graph"        1 (default): from the second step on the optimizer step is replayed from a CUDA graph (all but the
 *                            AdamW scalars, whose bias correction changes every step); 0: launched eagerly every step
 *   "decode_prefix_sharing"  -1 (default) automatic, 0 / 1 shared-prompt attention pass off / on (process-wide)
 *   "attention_tcgen05"      1 (default) head_dim 128 attention forward on tcgen05, 0 on mma.sync (process-wide)
 *   "gemm_persistent_ctas"   -1 (default) one CTA per SM for the tile-walking form, 0 form off, n = n CTAs
 *   "gemm_pdl"               1 (default) products launch with programmatic stream serialization
 *   "gemm_mn_major"          1 (default) operands stored [K, M] / [K, N] are read in place, 0 transposes them
 *   "gemm_mn_3d"             1 (default) one 3-D bulk-tensor copy per such tile instead of one per 32 columns
 *   "gemm_tma_store"         1 (default) one-tile products write plain results with bulk-tensor stores
 *   "gemm_wide_split"        1 (default) 128 x 256 tiles with a K split when 128-wide tiles fill half a wave to a wave
 *   "gemm_few_rows_max"      256 (default): x W^T products with at most this many rows stream the float32 weights
 *                            once and split them on chip (the decode step's form); 0 = off (process-wide)
 *   "gemm_few_rows_min_kblocks"  2 (default): smallest K share (in 32-element blocks) of one CTA of that form
 *   "gemm_few_rows_block"    128 (default): activation rows per CTA of that form (16..256) */
int gn_ctx_set_option(gn_ctx* ctx, const char* name, int value);

/* model.NewTransformer (model/transformer.go:49-83): parameters start at zero. */
int gn_model_create(gn_ctx* ctx, const gn_config* config, gn_model** out);
int gn_model_destroy(gn_model* model);
/* Parameter table, names as in Transformer.NamedParameters (model/params.go:14-74), sorted. */
int gn_model_param_count(gn_model* model, int* out);
int gn_model_param_info(gn_model* model, int index, const char** name, int* rows, int* cols);
int gn_model_upload(gn_model* model, const char* name, const float* host, int64_t n);
int gn_model_download(gn_model* model, const char* name, float* host, int64_t n);
int gn_model_download_grad(gn_model* model, const char* name, float* host, int64_t n);
/* Overwrites one tensor's gradient (Tensor.Grad) from host memory, e.g. gradients reduced elsewhere. */
int gn_model_upload_grad(gn_model* model, const char* name, const float* host, int64_t n);
/* Tensor.ZeroGrad over every parameter (model/params.go:100-104). */
int gn_model_zero_grad(gn_model* model);
/* The flat device buffer that holds every gradient (what the data-parallel
 * all-reduce sums), and the matching parameter buffer. */
int gn_model_grad_buffer(gn_model* model, float** device_ptr, int64_t* n);
int gn_model_param_buffer(gn_model* model, float** device_ptr, int64_t* n);
/* Sum of |gradient| and of |parameter| in float64 (replica checks). */
int gn_model_checksum(gn_model* model, double* param_sum, double* grad_sum);

/* Transformer.Forward without a cache (model/transformer.go:211-342): ids [B,T] (host) ->
 * logits [B,T,vocab] (host).  T > 1. */
int gn_model_forward(gn_model* model, const int32_t* ids, int batch, int seq, float* logits);

/* Engine.GenerateBatchWith for many prompts at once (inference/engine.go:112-369):
 * prefill each prompt, replicate its cache over `group` rows, then sample and
 * decode up to max_tokens steps.  Prompts are [n_prompts, prompt_len] (host).
 * Row p*group+g uses the generator keyed by seeds[p].  A row completes on
 * <|bos|> (vocab-11) or <|assistant_end|> (vocab-7); out_tokens
 * [n_prompts*group, max_tokens] receives the kept tokens (terminal stripped),
 * out_lengths their counts.  step_logits: NULL or host [max_tokens, rows, vocab],
 * the logits each sampling step saw.  steps_run: NULL or the number of sampling steps. */
int gn_generate_batch(gn_model* model, const int32_t* prompts, int n_prompts, int prompt_len, int group,
                      int max_tokens, float temperature, int top_k, const uint64_t* seeds, int32_t* out_tokens,
                      int32_t* out_lengths, float* step_logits, int* steps_run);

/* inference.GenerateOptions (inference/engine.go:24-35) plus tokens queued before the first step.
 * thinking / thinking_budget: the engine tracks <|think_start|> (vocab-2) ... <|think_end|> (vocab-1) and, once
 * thinking_budget reasoning tokens have been emitted, forces <|think_end|> (inference/engine.go:301-314).
 * forced [rows, forced_stride] with forced_counts[row] tokens: what a handled tool call would queue for that row
 * (inference/engine.go:284-300); a queued token overrides the sampled one and gets mask 0.  At most 64 per row. */
typedef struct gn_generate_options {
  int32_t thinking;
  int32_t thinking_budget;
  const int32_t* forced;
  int32_t forced_stride;
  const int32_t* forced_counts;
} gn_generate_options;
/* gn_generate_batch with options (NULL = none) and the masks of Engine.GenerateBatchWith: out_masks NULL or
 * [n_prompts*group, max_tokens], 1 = sampled, 0 = forced, parallel to out_tokens. */
int gn_generate_batch_ex(gn_model* model, const int32_t* prompts, int n_prompts, int prompt_len, int group, int max_tokens,
                         float temperature, int top_k, const uint64_t* seeds, const gn_generate_options* options,
                         int32_t* out_tokens, int32_t* out_lengths, int32_t* out_masks, float* step_logits, int* steps_run);

/* The same engine one step at a time, for hosts that put their own logic between steps: tool calls, which need the
 * tokenizer and a tool registry (inference/engine.go:284-300, inference/tooluse.go), and ensembles, which blend the
 * logits of several models before one token is sampled (inference/ensemble.go:104-243).  Every call returns with
 * the stream idle.
 *   gn_rollout_begin    prefill, replicate the caches over the groups, reset the per-row engine state
 *   gn_rollout_logits   device address of the current logits [logit_rows, vocab]; row r reads row r / row_div
 *                       (row_div = group right after the prefill, then 1)
 *   gn_rollout_sample   one sampling step from logits_device (NULL: the model's own; same shape) through the engine's
 *                       state machine; column / mask (host, [rows], nullable) receive the tokens that are forwarded
 *                       next and their masks; all_done is set when every row has finished
 *   gn_rollout_force    queue tokens for one row (they override the next samples of that row)
 *   gn_rollout_forward  forward the current column (column NULL) or one sampled by another model (an ensemble member
 *                       following the member that sampled)
 *   gn_rollout_end      kept tokens, lengths and masks, as gn_generate_batch_ex returns them */
int gn_rollout_begin(gn_model* model, const int32_t* prompts, int n_prompts, int prompt_len, int group, int max_tokens,
                     const uint64_t* seeds, const gn_generate_options* options);
int gn_rollout_logits(gn_model* model, float** device_ptr, int* logit_rows, int* row_div);
int gn_rollout_sample(gn_model* model, const float* logits_device, float temperature, int top_k, int32_t* column, int32_t* mask,
                      int* all_done);
int gn_rollout_force(gn_model* model, int row, const int32_t* tokens, int n);
int gn_rollout_forward(gn_model* model, const int32_t* column);
int gn_rollout_end(gn_model* model, int32_t* out_tokens, int32_t* out_lengths, int32_t* out_masks);

/* trainer.PolicyGradientStep (trainer/rl.go:14-60): inputs/targets [batch, seq]
 * (host, target -1 = ignore), advantages [batch], norm.  Gradients ACCUMULATE
 * into the model's gradient buffer (tensors/tensor.go:189-194).  Rows are
 * processed in chunks of `rows_per_pass` sequences (0 = library default); the
 * result does not depend on it beyond float32 summation order.
 * Optional host taps: nll [batch*seq], dlogits and logits [batch*seq, vocab]. */
int gn_policy_gradient_step(gn_model* model, const int32_t* inputs, const int32_t* targets, const float* advantages,
                            int batch, int seq, float norm, int rows_per_pass, float* loss, float* nll_tap,
                            float* dlogits_tap, float* logits_tap);

/* The session's KV cache, slice by slice, for the cache wire format of model/kvcache_codec.go (a host routine
 * serialises what these calls return).  All rows share one position, as in the reference (model/kvcache.go:91-94).
 *   kind 0 / 1  keys / values of (layer, row, kv head): positions * head_dim floats (model/kvcache.go:10-28)
 *   kind 2      latent rows of (layer, row): positions * latent floats        (latent attention, model/kvcache.go:224-237)
 *   kind 3      rotary keys of (layer, row): positions * n_kv_head * rope floats
 *   kind 4      the row's previous pre-smear embedding: embed_dim floats (layer, head, positions ignored)
 * gn_model_kv_alloc sizes an empty cache (for writing a deserialised one); gn_generate_batch sizes its own.  After a
 * gn_model_kv_write the rows of a group are no longer assumed to share their prompt's keys and values (the decode
 * attention then reads every row's own copy until the next gn_rollout_begin / gn_generate_batch). */
int gn_model_kv_info(gn_model* model, int* rows, int* max_seq, int* position);
int gn_model_kv_alloc(gn_model* model, int rows, int max_seq, int position);
int gn_model_kv_read(gn_model* model, int layer, int kind, int row, int head, int positions, float* host, int64_t n);
int gn_model_kv_write(gn_model* model, int layer, int kind, int row, int head, int positions, const float* host, int64_t n);

/* Phase timings of the last gn_generate_batch / gn_policy_gradient_step in
 * milliseconds (CUDA events on the context's stream): names are
 * "prefill", "decode", "train_forward", "loss", "train_backward". */
int gn_model_phase_ms(gn_model* model, const char* phase, float* ms);

/* Profiling aid (no counterpart in the reference): times `iters` launches of one kernel of
 * the RL step on synthetic device data with CUDA events on the context's stream, after three
 * warm-up launches, and returns the mean time of one launch in milliseconds.
 *   "gemm_nt" / "gemm_nn" / "gemm_tn"  dims {M, N, K}        C = A B^T / A B / A^T B
 *   "gemm_decode"       dims {rows, N, K, weight copies}      x W^T of the decode step, weights cycled so they come from HBM
 *   "loss"              dims {rows, vocab, valid_percent}    fused loss + dlogits (+ softcap backward)
 *   "sampler"           dims {rows, vocab, top_k}
 *   "decode_attention"  dims {rows, n_head, n_kv_head, head_dim, context}
 *   "attention_fwd" / "attention_bwd"  dims {batch, n_head, n_kv_head, head_dim, seq}   causal training attention
 *   "advantage"         dims {groups, group}
 * Buffers are larger than L2 for the workloads this is used on, so no cache flush is done. */
int gn_profile_kernel(gn_ctx* ctx, const char* kernel, const int64_t* dims, int n_dims, int iters, float* mean_ms);

/* ---------------------------------------------------------------------------
 * Optimizer step (trainer/rl.go:62-67: RLStep = PolicyGradientStep, optimizer.Step, optimizer.ZeroGrad).
 * Stand-alone updates of one tensor, in place; pointers may be host or device memory.  `grad` is
 * overwritten (it serves as the update matrix while the step runs).
 *   gn_adamw_step     optimizer/optimizer.go:143-173; `step` is the 1-based count of this tensor's updates
 *   gn_muon_step      optimizer/muon.go:23-173; second_mom has max(rows, cols) floats
 *   gn_sinkhorn_step  optimizer/sinkhorn.go:27-95; `steps` odd
 */
int gn_adamw_step(float* param, float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, int step, float lr, float beta1, float beta2, float eps,
                  float weight_decay);
int gn_muon_step(float* param, float* grad, float* momentum_state, float* second_mom, int rows, int cols, float lr, float momentum, int ns_steps,
                 float beta2, float weight_decay);
int gn_sinkhorn_step(float* param, float* grad, float* momentum_state, int rows, int cols, float lr, float momentum, float gamma, int steps, float tau,
                     float eps);

/* The optimizer chat_rl builds for the model (model.SetupOptimizer with sinkhorn = true, model/optimizer.go:20-165):
 * Sinkhorn for lm_head, wte and the value embeddings; AdamW for resid_lambdas, x0_lambdas and the smear / backout
 * scalars; Muon for every block matrix.  cmd/chat_rl/main.go:68-72 passes (0.004, 0.2, 0.02, 0.0, 0.5) and multiplies
 * every learning rate by 0.05.  Dense preset only. */
typedef struct gn_optimizer_config {
  float unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr;
  float lr_mult; /* applied to every group's learning rate */
} gn_optimizer_config;
/* Allocates (or resets) the optimizer state of the model: one momentum and one second-moment float per parameter. */
int gn_model_optimizer_init(gn_model* model, const gn_optimizer_config* config);
/* optimizer.Step() then ZeroGrad() on the model's gradient buffer (after the all-reduce in a data-parallel job). */
int gn_model_optimizer_step(gn_model* model);
/* Data-parallel form (the reference has no counterpart: it is single-process).  Every rank calls
 * gn_model_optimizer_step_shard(model, rank, world) after the gradient all-reduce: it updates only the tensors the
 * shard owns (the same deterministic assignment on every rank) and turns the gradient buffer into "my updated tensors,
 * zero elsewhere".  The caller then SUM-all-reduces gn_model_grad_buffer once more and calls gn_model_optimizer_finish,
 * which installs the reduced buffer as the parameters and zeroes the gradients.  The result equals
 * gn_model_optimizer_step bit for bit. */
int gn_model_optimizer_step_shard(gn_model* model, int shard, int shard_count);
int gn_model_optimizer_finish(gn_model* model);

/* ---------------------------------------------------------------------------
 * Data-parallel exchange (no counterpart in the reference, which is single-process, optimizer/optimizer.go:5-7;
 * its nearest analogue is the accumulation into Tensor.Grad, tensors/tensor.go:189-194).  One process per GPU, a
 * full replica each; rollout prompts are sharded by the host.  Rank 0 calls gn_comm_unique_id and hands the
 * GN_COMM_ID_BYTES bytes to the other ranks by its own means; every rank then calls gn_ctx_comm_init (collective:
 * it returns when all ranks have joined).  NCCL (libnccl.so.2) is loaded at the first of these calls.
 *   gn_model_grad_allreduce      SUM of the flat gradient buffer over the ranks, on the context's stream (the
 *                                1/norm factor is already in the gradients, trainer/rl.go:41); phase "allreduce"
 *   gn_ctx_allreduce_max_i64     MAX of one host integer over the ranks (the padded length every rank must use)
 *   gn_model_optimizer_exchange  after gn_model_optimizer_step_shard(model, rank, world) on every rank: each tensor
 *                                is broadcast from the rank that updated it, then the gradients are zeroed
 *                                (optimizer.ZeroGrad); replaces the all-reduce + gn_model_optimizer_finish pair
 * Without a communicator (or with world == 1) the three calls are local no-ops apart from the ZeroGrad. */
#define GN_COMM_ID_BYTES 128
int gn_comm_unique_id(void* id_out);
int gn_ctx_comm_init(gn_ctx* ctx, const void* id, int rank, int world);
int gn_ctx_comm_destroy(gn_ctx* ctx);
int gn_model_grad_allreduce(gn_model* model);
int gn_ctx_allreduce_max_i64(gn_ctx* ctx, int64_t* value);
int gn_model_optimizer_exchange(gn_model* model);

#ifdef __cplusplus
}
#endif
#endif /* GONANO_CUDA_H */
