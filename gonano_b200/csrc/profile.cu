// gn_profile_kernel: per-kernel timing on synthetic device data (CUDA events on the
// context's stream).  The benchmark uses it to put each hot kernel beside its roofline.
#include <algorithm>
#include <string>
#include <vector>

#include "kernels.cuh"
#include "ctx.cuh"

using namespace gn;


namespace {

__global__ void synth_kernel(float* dst, int64_t n, float lo, float hi, uint32_t salt) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint32_t h = (uint32_t)i * 2654435761u + salt;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    dst[i] = lo + (hi - lo) * (float)(h >> 8) * (1.0f / 16777216.0f);
  }
}
__global__ void synth_targets_kernel(int32_t* dst, int64_t n, int vocab, int valid_percent) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t h = (uint32_t)i * 2654435761u + 12345u;
  h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
  dst[i] = ((int)(h % 100u) < valid_percent) ? (int32_t)((h >> 7) % (uint32_t)vocab) : -1;
}

struct Bufs {
  std::vector<void*> p;
  ~Bufs() { for (void* q : p) cudaFree(q); }
  template <typename T>
  int get(T** out, size_t n) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, n * sizeof(T));
    if (e != cudaSuccess) { set_error("profile: cudaMalloc of %zu bytes failed: %s", n * sizeof(T), cudaGetErrorString(e)); return GN_ERR_NOMEM; }
    p.push_back(q);
    *out = (T*)q;
    return GN_OK;
  }
};

int synth(float* dst, int64_t n, float lo, float hi, uint32_t salt, cudaStream_t s) {
  synth_kernel<<<num_sms() * 8, 256, 0, s>>>(dst, n, lo, hi, salt);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

template <typename F>
int time_it(cudaStream_t s, int iters, float* mean_ms, F&& launch) {
  cudaEvent_t a, b;
  GN_CUDA(cudaEventCreate(&a)); GN_CUDA(cudaEventCreate(&b));
  for (int i = 0; i < 3; ++i) GN_TRY(launch());
  GN_CUDA(cudaStreamSynchronize(s));
  GN_CUDA(cudaEventRecord(a, s));
  for (int i = 0; i < iters; ++i) GN_TRY(launch());
  GN_CUDA(cudaEventRecord(b, s));
  GN_CUDA(cudaEventSynchronize(b));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, a, b));
  cudaEventDestroy(a); cudaEventDestroy(b);
  *mean_ms = ms / (float)iters;
  return GN_OK;
}

}  // namespace

extern "C" int gn_profile_kernel(gn_ctx* ctx, const char* kernel, const int64_t* dims, int n_dims, int iters, float* mean_ms) {
  GN_REQUIRE(ctx && kernel && dims && mean_ms && iters > 0, "gn_profile_kernel: bad argument");
  GN_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t s = ctx->stream;
  std::string k(kernel);
  Bufs bufs;
  if (k == "gemm_nt" || k == "gemm_nn" || k == "gemm_tn") {
    GN_REQUIRE(n_dims == 3, "%s wants {M, N, K}", kernel);
    int M = (int)dims[0], N = (int)dims[1], K = (int)dims[2];
    float *A, *B, *C;
    GN_TRY(bufs.get(&A, (size_t)M * K)); GN_TRY(bufs.get(&B, (size_t)N * K)); GN_TRY(bufs.get(&C, (size_t)M * N));
    GN_TRY(synth(A, (int64_t)M * K, -1, 1, 1, s)); GN_TRY(synth(B, (int64_t)N * K, -1, 1, 2, s));
    GemmArgs g; g.A = A; g.B = B; g.C = C; g.M = M; g.N = N; g.K = K; g.ldc = N;
    if (k == "gemm_nt") { g.lda = K; g.ldb = K; g.b_trans = 1; }
    else if (k == "gemm_nn") { g.lda = K; g.ldb = N; g.b_trans = 0; }
    else { g.lda = M; g.a_trans = 1; g.ldb = N; g.b_trans = 0; }
    int kind = ctx->gemm_kind;
    return time_it(s, iters, mean_ms, [&]() { return gemm_dispatch(g, kind, s); });
  }
  if (k == "gemm_decode") {
    // A product of the decode step: few activation rows (already split by their producer) against one of `copies`
    // distinct weight matrices in turn, so that the weights come from HBM as they do in a 12-layer step, the result
    // left as K-split partial tiles for the consumer when the path splits K.
    GN_REQUIRE(n_dims == 4 && dims[3] >= 1, "gemm_decode wants {rows, N, K, weight copies}");
    int M = (int)dims[0], N = (int)dims[1], K = (int)dims[2], copies = (int)dims[3];
    float *A, *Ah, *Al, *B, *C;
    GN_TRY(bufs.get(&A, (size_t)M * K)); GN_TRY(bufs.get(&Ah, (size_t)M * K)); GN_TRY(bufs.get(&Al, (size_t)M * K));
    GN_TRY(bufs.get(&B, (size_t)copies * N * K)); GN_TRY(bufs.get(&C, (size_t)M * N));
    GN_TRY(synth(A, (int64_t)M * K, -1, 1, 1, s)); GN_TRY(synth(B, (int64_t)copies * N * K, -1, 1, 2, s));
    GN_TRY(split_matrix_launch(A, Ah, Al, M, K, K, s));
    int kind = ctx->gemm_kind, turn = 0;
    return time_it(s, iters, mean_ms, [&]() {
      Partials left;
      GemmArgs g; g.A = A; g.a_hi = Ah; g.a_lo = Al; g.lda = K; g.B = B + (size_t)(turn++ % copies) * N * K; g.ldb = K; g.b_trans = 1; g.b_static = 1; g.b_prefetch = 1;
      g.C = C; g.ldc = N; g.M = M; g.N = N; g.K = K; g.leave = &left;
      return gemm_dispatch(g, kind, s);
    });
  }
  if (k == "loss") {
    GN_REQUIRE(n_dims == 3, "loss wants {rows, vocab, valid_percent}");
    int64_t rows = dims[0]; int vocab = (int)dims[1]; int pct = (int)dims[2];
    float *logits, *grad, *adv, *nll; int32_t* tg; double* rl;
    GN_TRY(bufs.get(&logits, (size_t)rows * vocab)); GN_TRY(bufs.get(&grad, (size_t)rows * vocab)); GN_TRY(bufs.get(&adv, (size_t)rows));
    GN_TRY(bufs.get(&nll, (size_t)rows)); GN_TRY(bufs.get(&tg, (size_t)rows)); GN_TRY(bufs.get(&rl, (size_t)rows + 1));
    GN_TRY(synth(logits, rows * vocab, -15, 15, 3, s)); GN_TRY(synth(adv, rows, -1, 1, 4, s));
    synth_targets_kernel<<<ceil_div(rows, 256), 256, 0, s>>>(tg, rows, vocab, pct);
    GN_LAUNCH_CHECK();
    return time_it(s, iters, mean_ms, [&]() { return pg_loss_launch(logits, tg, adv, rows, vocab, vocab, 512, 8192.0f, 15.0f, nll, grad, vocab, rl + 1, rl, 0, s); });
  }
  if (k == "sampler") {
    GN_REQUIRE(n_dims == 3, "sampler wants {rows, vocab, top_k}");
    int rows = (int)dims[0], vocab = (int)dims[1], topk = (int)dims[2];
    float* logits; int32_t* out; uint64_t* seeds;
    GN_TRY(bufs.get(&logits, (size_t)rows * vocab)); GN_TRY(bufs.get(&out, (size_t)rows)); GN_TRY(bufs.get(&seeds, (size_t)rows));
    GN_TRY(synth(logits, (int64_t)rows * vocab, -15, 15, 5, s));
    GN_CUDA(cudaMemsetAsync(seeds, 1, sizeof(uint64_t) * rows, s));
    uint32_t step = 0;
    return time_it(s, iters, mean_ms, [&]() { return sample_launch(logits, rows, vocab, 1, nullptr, seeds, 8, nullptr, step++, 1.0f, topk, out, s); });
  }
  if (k == "decode_attention") {
    GN_REQUIRE(n_dims == 5 || n_dims == 7, "decode_attention wants {rows, n_head, n_kv_head, head_dim, context[, group, shared prefix length]}");
    int rows = (int)dims[0], Hq = (int)dims[1], Hkv = (int)dims[2], D = (int)dims[3], ctxl = (int)dims[4];
    const int group = n_dims == 7 ? (int)dims[5] : 1, prefix = n_dims == 7 ? (int)dims[6] : 0;
    float *q, *kc, *vc, *out, *pa, *pm; int32_t* cl;
    size_t cache = (size_t)rows * Hkv * ctxl * D;
    const int own = attention_decode_splits(rows, Hkv, ctxl);
    int splits = own + attention_decode_prefix_splits(rows, group, Hq, Hkv, D, prefix);
    GN_TRY(bufs.get(&q, (size_t)rows * Hq * D)); GN_TRY(bufs.get(&kc, cache)); GN_TRY(bufs.get(&vc, cache)); GN_TRY(bufs.get(&out, (size_t)rows * Hq * D));
    GN_TRY(bufs.get(&pa, (size_t)rows * Hq * splits * D)); GN_TRY(bufs.get(&pm, (size_t)rows * Hq * splits * 2)); GN_TRY(bufs.get(&cl, (size_t)rows));
    GN_TRY(synth(q, (int64_t)rows * Hq * D, -1, 1, 6, s)); GN_TRY(synth(kc, (int64_t)cache, -1, 1, 7, s)); GN_TRY(synth(vc, (int64_t)cache, -1, 1, 8, s));
    std::vector<int32_t> h(rows, ctxl);
    GN_CUDA(cudaMemcpyAsync(cl, h.data(), sizeof(int32_t) * rows, cudaMemcpyHostToDevice, s));
    GN_CUDA(cudaStreamSynchronize(s));
    return time_it(s, iters, mean_ms, [&]() {
      return attention_decode_launch(q, (int64_t)Hq * D, kc, vc, (int64_t)Hkv * ctxl * D, (int64_t)ctxl * D, cl, rows, Hq, Hkv, D, -1, out, (int64_t)Hq * D, pa, pm, own, s,
                                     nullptr, nullptr, group, prefix);
    });
  }
  if (k == "attention_fwd" || k == "attention_bwd") {
    GN_REQUIRE(n_dims == 5, "%s wants {batch, n_head, n_kv_head, head_dim, seq}", kernel);
    int B = (int)dims[0], Hq = (int)dims[1], Hkv = (int)dims[2], D = (int)dims[3], T = (int)dims[4];
    const int W = (Hq + 2 * Hkv) * D;
    const int64_t rows = (int64_t)B * T;
    float *qkv, *o, *lse, *dqkv, *dout, *delta;
    GN_TRY(bufs.get(&qkv, (size_t)rows * W)); GN_TRY(bufs.get(&o, (size_t)rows * Hq * D)); GN_TRY(bufs.get(&lse, (size_t)B * Hq * T));
    GN_TRY(bufs.get(&dqkv, (size_t)rows * W)); GN_TRY(bufs.get(&dout, (size_t)rows * Hq * D)); GN_TRY(bufs.get(&delta, (size_t)B * Hq * T));
    GN_TRY(synth(qkv, rows * W, -1.2f, 1.2f, 11, s)); GN_TRY(synth(dout, rows * Hq * D, -1, 1, 12, s));
    AttnShape sh;
    sh.B = B; sh.Hq = Hq; sh.Hkv = Hkv; sh.D = D; sh.Tq = T; sh.Tk = T;
    sh.q_bstride = (int64_t)T * W; sh.q_tstride = W; sh.kv_bstride = (int64_t)T * W; sh.kv_tstride = W; sh.kv_hstride = D;
    sh.o_bstride = (int64_t)T * Hq * D; sh.o_tstride = (int64_t)Hq * D; sh.window = -1; sh.offset0 = 0; sh.tensor = ctx->gemm_kind == 1;
    const float* kp = qkv + (int64_t)Hq * D; const float* vp = qkv + (int64_t)(Hq + Hkv) * D;
    GN_TRY(attention_forward_launch(sh, qkv, kp, vp, o, lse, s));
    if (k == "attention_fwd") return time_it(s, iters, mean_ms, [&]() { return attention_forward_launch(sh, qkv, kp, vp, o, lse, s); });
    return time_it(s, iters, mean_ms, [&]() {
      return attention_backward_launch(sh, qkv, kp, vp, o, dout, lse, nullptr, dqkv, dqkv + (int64_t)Hq * D, dqkv + (int64_t)(Hq + Hkv) * D, 0, delta, s);
    });
  }
  if (k == "compressed_attention_fwd" || k == "compressed_attention_bwd" || k == "compressed_attention_sparse_fwd" || k == "compressed_attention_sparse_bwd") {
    // the global branch of a compressed attention layer: {batch, n_head, n_kv_head, head_dim, seq, ratio[, topk]}
    GN_REQUIRE(n_dims >= 6, "%s wants {batch, n_head, n_kv_head, head_dim, seq, ratio[, topk]}", kernel);
    const int B = (int)dims[0], Hq = (int)dims[1], Hkv = (int)dims[2], D = (int)dims[3], T = (int)dims[4], ratio = (int)dims[5];
    const int topk = n_dims > 6 ? (int)dims[6] : 0;
    const bool sparse = k.find("sparse") != std::string::npos;
    GN_REQUIRE(ratio >= 1 && T >= 1 && (!sparse || topk >= 1), "%s: ratio %d, seq %d, topk %d", kernel, ratio, T, topk);
    const int blocks = (T + ratio - 1) / ratio;
    const int64_t nq = (int64_t)B * Hq * T * D, nk = (int64_t)B * Hkv * blocks * D, nt = (int64_t)B * Hq * T;
    float *q, *kc, *vc, *o, *lse, *dout, *dq, *dk, *dv, *delta, *scores = nullptr;
    int32_t *sel = nullptr, *cnt = nullptr;
    GN_TRY(bufs.get(&q, (size_t)nq)); GN_TRY(bufs.get(&kc, (size_t)nk)); GN_TRY(bufs.get(&vc, (size_t)nk)); GN_TRY(bufs.get(&o, (size_t)nq));
    GN_TRY(bufs.get(&lse, (size_t)nt)); GN_TRY(bufs.get(&dout, (size_t)nq)); GN_TRY(bufs.get(&dq, (size_t)nq)); GN_TRY(bufs.get(&dk, (size_t)nk));
    GN_TRY(bufs.get(&dv, (size_t)nk)); GN_TRY(bufs.get(&delta, (size_t)nt));
    GN_TRY(synth(q, nq, -0.6f, 0.6f, 21, s)); GN_TRY(synth(kc, nk, -0.6f, 0.6f, 22, s)); GN_TRY(synth(vc, nk, -1, 1, 23, s)); GN_TRY(synth(dout, nq, -1, 1, 24, s));
    if (sparse) {
      // a selection per (sequence, kv head) from synthetic index scores
      GN_TRY(bufs.get(&scores, (size_t)T * blocks));
      GN_TRY(bufs.get(&sel, (size_t)B * Hkv * T * topk)); GN_TRY(bufs.get(&cnt, (size_t)B * Hkv * T));
      for (int i = 0; i < B * Hkv; ++i) {
        GN_TRY(synth(scores, (int64_t)T * blocks, -1, 1, 30 + i, s));
        GN_TRY(select_blocks_launch(scores, T, blocks, 0, ratio, topk, sel + (int64_t)i * T * topk, cnt + (int64_t)i * T, s));
      }
    }
    GN_TRY(compressed_attention_launch(q, kc, vc, B, Hq, Hkv, T, D, blocks, ratio, o, lse, sel, cnt, topk, 0, s));
    if (k == "compressed_attention_fwd" || k == "compressed_attention_sparse_fwd")
      return time_it(s, iters, mean_ms, [&]() { return compressed_attention_launch(q, kc, vc, B, Hq, Hkv, T, D, blocks, ratio, o, lse, sel, cnt, topk, 0, s); });
    GN_CUDA(cudaMemsetAsync(dq, 0, sizeof(float) * nq, s)); GN_CUDA(cudaMemsetAsync(dk, 0, sizeof(float) * nk, s)); GN_CUDA(cudaMemsetAsync(dv, 0, sizeof(float) * nk, s));
    // as in a layer with a sliding-window branch: the row correction dO . O of the merged output comes with the call
    uint32_t* bits = nullptr; if (sparse) GN_TRY(bufs.get(&bits, (size_t)B * Hkv * T * ((blocks + 31) / 32)));
    float* rowcorr; GN_TRY(bufs.get(&rowcorr, (size_t)nt)); GN_TRY(synth(rowcorr, nt, -1, 1, 25, s));
    return time_it(s, iters, mean_ms, [&]() {
      return compressed_attention_backward_launch(q, kc, vc, dout, lse, rowcorr, delta, B, Hq, Hkv, T, D, blocks, ratio, dq, dk, dv, sel, cnt, topk, s, bits);
    });
  }
  if (k == "indexer_scores") {
    GN_REQUIRE(n_dims == 4, "%s wants {rows, blocks, heads, dim}", kernel);
    const int rows = (int)dims[0], blocks = (int)dims[1], heads = (int)dims[2], dim = (int)dims[3];
    float *q, *kk, *w, *dst;
    GN_TRY(bufs.get(&q, (size_t)rows * heads * dim)); GN_TRY(bufs.get(&kk, (size_t)blocks * heads * dim)); GN_TRY(bufs.get(&w, (size_t)heads));
    GN_TRY(bufs.get(&dst, (size_t)rows * blocks));
    GN_TRY(synth(q, (int64_t)rows * heads * dim, -1, 1, 51, s)); GN_TRY(synth(kk, (int64_t)blocks * heads * dim, -1, 1, 52, s)); GN_TRY(synth(w, heads, 0.5f, 1.5f, 53, s));
    return time_it(s, iters, mean_ms, [&]() { return indexer_scores_launch(dst, q, kk, w, rows, blocks, heads, dim, s); });
  }
  if (k == "distillation_target") {
    GN_REQUIRE(n_dims == 6, "%s wants {batch, n_head, n_kv_head, head_dim, seq, ratio}", kernel);
    const int B = (int)dims[0], Hq = (int)dims[1], Hkv = (int)dims[2], D = (int)dims[3], T = (int)dims[4], ratio = (int)dims[5];
    const int blocks = (T + ratio - 1) / ratio;
    float *q, *kc, *target;
    GN_TRY(bufs.get(&q, (size_t)B * Hq * T * D)); GN_TRY(bufs.get(&kc, (size_t)B * Hkv * blocks * D)); GN_TRY(bufs.get(&target, (size_t)B * Hkv * T * blocks));
    GN_TRY(synth(q, (int64_t)B * Hq * T * D, -0.6f, 0.6f, 71, s)); GN_TRY(synth(kc, (int64_t)B * Hkv * blocks * D, -0.6f, 0.6f, 72, s));
    float* qsum; GN_TRY(bufs.get(&qsum, (size_t)B * Hkv * T * D + 1));
    return time_it(s, iters, mean_ms, [&]() { return distillation_target_launch(q, kc, B, Hq, Hkv, T, D, blocks, ratio, target, s, qsum); });
  }
  if (k == "indexer_scores_bwd") {
    GN_REQUIRE(n_dims == 4, "%s wants {rows, blocks, heads, dim}", kernel);
    const int rows = (int)dims[0], blocks = (int)dims[1], heads = (int)dims[2], dim = (int)dims[3];
    float *q, *kk, *w, *gs, *gq, *gk, *gw, *wpart;
    GN_TRY(bufs.get(&q, (size_t)rows * heads * dim)); GN_TRY(bufs.get(&kk, (size_t)blocks * heads * dim)); GN_TRY(bufs.get(&w, (size_t)heads));
    GN_TRY(bufs.get(&gs, (size_t)rows * blocks)); GN_TRY(bufs.get(&gq, (size_t)rows * heads * dim)); GN_TRY(bufs.get(&gk, (size_t)blocks * heads * dim));
    GN_TRY(bufs.get(&gw, (size_t)heads)); GN_TRY(bufs.get(&wpart, (size_t)rows * heads));
    GN_TRY(synth(q, (int64_t)rows * heads * dim, -1, 1, 51, s)); GN_TRY(synth(kk, (int64_t)blocks * heads * dim, -1, 1, 52, s)); GN_TRY(synth(w, heads, 0.5f, 1.5f, 53, s));
    GN_TRY(synth(gs, (int64_t)rows * blocks, -1, 1, 54, s)); GN_CUDA(cudaMemsetAsync(gw, 0, sizeof(float) * heads, s));
    float* kpart; GN_TRY(bufs.get(&kpart, (size_t)16 * blocks * heads * dim));
    return time_it(s, iters, mean_ms, [&]() { return indexer_scores_backward_launch(gs, q, kk, w, rows, blocks, heads, dim, gq, gk, gw, wpart, s, kpart, 16); });
  }
  if (k == "select_hierarchical" || k == "select_blocks") {
    GN_REQUIRE(n_dims >= 4, "%s wants {tokens, blocks, ratio, topk[, pool, budget]}", kernel);
    const int tokens = (int)dims[0], blocks = (int)dims[1], ratio = (int)dims[2], topk = (int)dims[3];
    const int pool = n_dims > 4 ? std::max(1, (int)dims[4]) : 1, budget = n_dims > 5 ? (int)dims[5] : 0;
    const int per_token = std::max(1, (budget + pool - 1) / pool), cap = per_token * pool;
    float *scores, *gmax; int32_t *sel, *cnt, *cand, *ccnt, *chosen;
    GN_TRY(bufs.get(&scores, (size_t)tokens * blocks)); GN_TRY(bufs.get(&gmax, (size_t)tokens * ((blocks + pool - 1) / pool)));
    GN_TRY(bufs.get(&sel, (size_t)tokens * topk)); GN_TRY(bufs.get(&cnt, (size_t)tokens)); GN_TRY(bufs.get(&cand, (size_t)tokens * cap));
    GN_TRY(bufs.get(&ccnt, (size_t)tokens)); GN_TRY(bufs.get(&chosen, (size_t)tokens * per_token));
    GN_TRY(synth(scores, (int64_t)tokens * blocks, -1, 1, 61, s));
    if (k == "select_blocks") return time_it(s, iters, mean_ms, [&]() { return select_blocks_launch(scores, tokens, blocks, 0, ratio, topk, sel, cnt, s); });
    return time_it(s, iters, mean_ms, [&]() { return select_hierarchical_launch(scores, tokens, blocks, 0, ratio, topk, pool, budget, gmax, chosen, sel, cnt, cand, ccnt, s); });
  }
  if (k == "compressed_attention_decode") {
    // one decode step of the global branch over a cached compressed sequence: {rows, n_head, n_kv_head, head_dim, blocks}
    GN_REQUIRE(n_dims == 5, "%s wants {rows, n_head, n_kv_head, head_dim, blocks}", kernel);
    const int B = (int)dims[0], Hq = (int)dims[1], Hkv = (int)dims[2], D = (int)dims[3], blocks = (int)dims[4];
    float *q, *kc, *vc, *o, *lse;
    GN_TRY(bufs.get(&q, (size_t)B * Hq * D)); GN_TRY(bufs.get(&kc, (size_t)B * Hkv * blocks * D)); GN_TRY(bufs.get(&vc, (size_t)B * Hkv * blocks * D));
    GN_TRY(bufs.get(&o, (size_t)B * Hq * D)); GN_TRY(bufs.get(&lse, (size_t)B * Hq));
    GN_TRY(synth(q, (int64_t)B * Hq * D, -0.6f, 0.6f, 41, s)); GN_TRY(synth(kc, (int64_t)B * Hkv * blocks * D, -0.6f, 0.6f, 42, s));
    GN_TRY(synth(vc, (int64_t)B * Hkv * blocks * D, -1, 1, 43, s));
    // the launch gn_compressed_attention_forward_at makes for one token: the split-context decode kernel over the blocks
    const int splits = std::max(2, attention_decode_splits(B, Hkv, blocks));
    int32_t* cl; float *pa, *pm;
    GN_TRY(bufs.get(&cl, (size_t)B)); GN_TRY(bufs.get(&pa, (size_t)B * Hq * splits * D)); GN_TRY(bufs.get(&pm, (size_t)B * Hq * splits * 2));
    std::vector<int32_t> host((size_t)B, blocks);
    GN_CUDA(cudaMemcpyAsync(cl, host.data(), sizeof(int32_t) * B, cudaMemcpyHostToDevice, s));
    GN_CUDA(cudaStreamSynchronize(s));
    return time_it(s, iters, mean_ms, [&]() {
      return attention_decode_launch(q, (int64_t)Hq * D, kc, vc, (int64_t)Hkv * blocks * D, (int64_t)blocks * D, cl, B, Hq, Hkv, D, -1, o, (int64_t)Hq * D, pa, pm, splits, s,
                                     nullptr, nullptr, 1, 0, lse);
    });
  }
  if (k == "advantage") {
    GN_REQUIRE(n_dims == 2, "advantage wants {groups, group}");
    int groups = (int)dims[0], group = (int)dims[1];
    float *r, *a;
    GN_TRY(bufs.get(&r, (size_t)groups * group)); GN_TRY(bufs.get(&a, (size_t)groups * group));
    GN_TRY(synth(r, (int64_t)groups * group, 0, 1, 9, s));
    return time_it(s, iters, mean_ms, [&]() { return advantage_launch(r, groups, group, 0, a, s); });
  }
  set_error("gn_profile_kernel: unknown kernel '%s'", kernel);
  return GN_ERR_INVALID;
}
