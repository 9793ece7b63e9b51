// Structures shared by the resident-session translation units (model.cu, model_latent.cu).
#pragma once
#include <map>
#include <string>
#include <vector>

#include "kernels.cuh"
#include "model_kernels.cuh"
#include "ctx.cuh"

namespace gnm {
using namespace gn;

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  int ensure(size_t n) {
    if (n <= bytes) return GN_OK;
    if (p) cudaFree(p);
    p = nullptr; bytes = 0;
    cudaError_t e = cudaMalloc(&p, n);
    if (e != cudaSuccess) { set_error("cudaMalloc(%zu bytes) failed: %s", n, cudaGetErrorString(e)); return GN_ERR_NOMEM; }
    bytes = n;
    return GN_OK;
  }
  void release() { if (p) cudaFree(p); p = nullptr; bytes = 0; }
  float* f() const { return (float*)p; }
  int32_t* i() const { return (int32_t*)p; }
};

struct ParamInfo {
  std::string name;
  int rows = 0, cols = 0;
  int64_t offset = 0;
};

// A bump allocator over one DevBuf: buffers of one pass are carved in order.
struct Arena {
  DevBuf buf;
  size_t used = 0;
  size_t planned = 0;
  bool planning = false;
  float* take(size_t floats) {
    size_t bytes = ((floats * sizeof(float) + 255) / 256) * 256;
    if (planning) { planned += bytes; return nullptr; }
    float* r = (float*)((char*)buf.p + used);
    used += bytes;
    return r;
  }
};

struct LayerOffsets {
  int64_t qkv, proj, ve_gate, fc, mproj, ve; bool has_ve;
  // latent attention (model/mla.go:15-37): mla_cat = [q_down; kv_down; q_rope; k_rope], adjacent, all with d columns
  int64_t mla_cat = -1, mla_q_up = -1, mla_k_up = -1, mla_v_up = -1;
  // routed experts (model/moe.go:26-45); with them fc = [c_fc; c_gate] adjacent and mproj = the shared expert's c_proj
  int64_t router = -1, router_bias = -1, exp_gate = -1, exp_up = -1, exp_down = -1;
};

struct LayerSaved {
  float *Xin, *H, *QKV, *QKROT, *O, *LSE, *VESIG, *MID, *M, *U, *HID, *XOUT;
  // tf32 hi/lo splits of H, M and HID written by their producers in the forward pass and read again by the
  // weight-gradient products (tensor-core path; null otherwise)
  float *Hh = nullptr, *Hl = nullptr, *Mh = nullptr, *Ml = nullptr, *Ph = nullptr, *Pl = nullptr;
  // latent preset (model_latent_train.cu): the fused down / rotary projections of latent attention; the shared
  // expert's [up | gate] and hidden rows; the router's softmax, selection, weights, expert-major positions and counts;
  // the experts' gate / up / hidden / output rows
  float *P1 = nullptr, *UG = nullptr, *SHH = nullptr, *SHHh = nullptr, *SHHl = nullptr, *PR = nullptr, *SELW = nullptr;
  int32_t *SEL = nullptr, *POSI = nullptr, *CNT = nullptr;
  float *GG = nullptr, *GU = nullptr, *GH = nullptr, *GHh = nullptr, *GHl = nullptr, *GO = nullptr;
  std::vector<int32_t> host_counts;   // rows per expert, read back once in the forward pass
};

// Scratch of one training pass of the latent preset, shared by all layers.
struct LatentWs {
  float *QC = nullptr, *KC = nullptr, *DQC = nullptr, *DKC = nullptr, *DP1 = nullptr;
  float *SHO = nullptr, *RL = nullptr, *GATH = nullptr, *GATHh = nullptr, *GATHl = nullptr;
  float *DSHH = nullptr, *DUG = nullptr, *DMS = nullptr, *DMR = nullptr, *DGO = nullptr, *DGH = nullptr, *DGG = nullptr, *DGU = nullptr, *DGATH = nullptr;
  double* GPROB = nullptr; float* GLOG = nullptr; int32_t* SEQCNT = nullptr;
  int total_sequences = 0;   // sequences of the whole policy-gradient call (the balance loss is a mean over them)
};
constexpr float kMoEBalanceWeight = 1e-4f;   // defaultMoEBalanceWeight (model/config.go:133-135,176-186)

}  // namespace gnm
using namespace gnm;

namespace gnm {
enum Mode { MODE_PLAIN, MODE_PREFILL, MODE_DECODE, MODE_TRAIN };

struct FwdBufs {
  float *E, *X0, *Xa, *Xb, *H, *QKV, *O, *M, *HID, *BO, *Y, *LOGITS;
  float *S1h, *S1l, *S4h, *S4l;   // producer-written tf32 splits: one [rows, d] pair and one [rows, 4d] pair, reused by every layer
  // train only
  float *SIG, *FP;
  std::vector<LayerSaved> layers;
  LatentWs* lws = nullptr;   // train, latent preset: the pass's scratch
  // latent attention (inference): fused down/rope projections, content queries, absorbed queries, attended latents
  float *P1 = nullptr, *QC = nullptr, *QF = nullptr, *AL = nullptr;
  // routed experts (inference)
  float *UG = nullptr, *SHH = nullptr, *SHO = nullptr, *RL = nullptr, *PR = nullptr, *SELW = nullptr, *GATH = nullptr, *GG = nullptr, *GU = nullptr, *GO = nullptr;
  int32_t *SEL = nullptr, *CNT = nullptr, *POSI = nullptr;
  float *GATHh = nullptr, *GATHl = nullptr, *GHh = nullptr, *GHl = nullptr;   // tf32 splits of the gathered rows and of the experts' hidden rows
};

struct FwdArgs {
  Mode mode;
  const int32_t* ids;      // device [B*T]
  int B, T;
  int cache_rows = 0, cache_row_mul = 1, max_seq = 0;
  int logits_rows = 0;     // rows that get logits (PLAIN/TRAIN: all; PREFILL: B; DECODE: B)
  int group = 1, prefix_len = 0;   // DECODE: rows come in groups sharing their first prefix_len cached positions
  bool skip_head = false;          // TRAIN: stop after the final norm (b.Y); the caller runs lm_head, loss and their backward in row chunks
};

}  // namespace gnm
namespace gnm {
// A rollout in progress (inference/engine.go:112-327): geometry, options and the buffers of its decode steps.
struct Rollout {
  bool active = false;
  int P = 0, plen = 0, G = 0, max_tokens = 0, rows = 0, max_seq = 0;
  int generated = 0;          // sampling steps taken
  int logits_row_div = 1;     // rows that share one row of the current logits (G right after the prefill, then 1)
  bool thinking = false; int thinking_budget = 0;
  int follower_steps = 0;     // forwards of columns sampled elsewhere (ensemble members)
  bool prompt_shared = true;  // the rows of a group still hold identical K/V for the prompt positions (false once the cache was written from outside)
  FwdBufs b;
};
}  // namespace gnm
struct gn_model;
namespace gnm {
// model_latent.cu / model_latent_train.cu
int moe_router_logits(gn_model* m, int l, const float* Mn, float* RL, int64_t rows);
int moe_route_launch(const int32_t* sel, int64_t total, int E, int32_t* counts, int32_t* posi, cudaStream_t s);
size_t latent_saved_layout(const gn_model* m, float* base, LayerSaved* s, int64_t rows);
size_t latent_ws_layout(const gn_model* m, float* base, LatentWs* w, int64_t rows, int B);
int latent_attention_train(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* H, const float* Hh, const float* Hl, int B, int T);
int latent_attention_backward(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* H, const float* DQKV, float* DH, int B, int T);
int moe_ffn_train(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* Mn, const float* Mh, const float* Ml, const float* MID, float* XOUT, int64_t rows);
int moe_ffn_backward(gn_model* m, LayerSaved& sv, LatentWs& w, int l, const float* Mn, const float* DOUT, float* DM, int64_t rows, int seq_len);
}  // namespace gnm

struct gn_model {
  gn_ctx* ctx = nullptr;
  gn_config cfg{};
  int d = 0, L = 0, Hq = 0, Hkv = 0, D = 0, R = 0, V = 0, Vp = 0, W = 0, KV = 0;
  // DeepSeekMoE / latent attention (zero when off)
  int E = 0, topk = 0, eh = 0, sh = 0; float moe_clamp = 0.0f, moe_scale = 0.0f;
  int lat = 0, rope = 0, content = 0;
  bool moe() const { return E > 0; }
  bool mla() const { return lat > 0; }
  std::vector<int> windows;
  std::vector<ParamInfo> params;               // sorted by name
  std::map<std::string, int> index;
  int64_t total = 0;
  DevBuf P, G;
  std::vector<LayerOffsets> lo;
  int64_t off_wte = 0, off_lm = 0, off_rho = 0, off_chi = 0, off_smear_gate = 0, off_smear_lambda = 0, off_backout = 0;
  DevBuf cosb, sinb, sacc;
  // inference state
  DevBuf cache, prev, pos, ctxlen, ids_dev, sampled, seeds, out_tokens, out_lengths, out_masks, engine_state, done, n_done, sel;
  Rollout ro;   // the rollout in progress (gn_generate_batch, gn_rollout_*)
  DevBuf part_acc, part_ms, step_dev;
  // optimizer state (gn_model_optimizer_init): momentum / exp_avg and second moment / exp_avg_sq at the parameter's offset
  DevBuf opt_mom, opt_second, opt_ws;
  // The tensors of an optimizer step are independent: they are updated on kOptLanes streams side by side (lane 0 is the
  // context's stream), each with its own workspace.
  static constexpr int kOptLanes = 4;
  cudaStream_t opt_stream[kOptLanes] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t opt_event[kOptLanes + 1] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  DevBuf opt_ws_lane[kOptLanes];
  gn_optimizer_config opt_cfg{};
  int opt_steps = 0;
  // the captured optimizer step: valid for one (shard, shard_count, lanes, product kind, option generation)
  cudaGraph_t opt_graph = nullptr;
  cudaGraphExec_t opt_graph_exec = nullptr;
  size_t opt_graph_nodes = 0;
  int opt_graph_key[5] = {-1, -1, -1, -1, -1};
  int opt_eager_runs = 0;          // eager steps so far: the first one sizes every scratch buffer
  bool opt_graph_failed = false;   // a capture failed once: stay eager
  bool opt_ready = false;
  DevBuf cache_lat, cache_rope;   // latent attention: [layer][row][max_seq][lat] and [layer][row][max_seq][Hkv*rope]
  Arena infer, train;
  DevBuf tgt_dev, adv_dev, rowloss, loss_dev, in_dev, lat_ws;
  std::map<std::string, float> phase_ms;
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  bool weights_dirty = true;   // cached tensor-core operand splits of the parameters are stale
  int kv_rows = 0, kv_max_seq = 0;   // geometry of the KV cache currently held

  float* p(int64_t off) const { return P.f() + off; }
  float* g(int64_t off) const { return G.f() + off; }
  cudaStream_t s() const { return ctx->stream; }
};

namespace gnm {
using namespace gn;

inline int gemm(gn_model* m, const gn::GemmArgs& a) { return gn::gemm_dispatch(a, m->ctx->gemm_kind, m->s()); }

// Which shard updates which tensor in a sharded optimizer step: a greedy balance of an operation-count estimate,
// identical on every rank (index = position in gn_model::params).
// Cost-balanced assignment of the parameters to `shard_count` bins; with `within`, only the parameters whose entry equals
// `within_value` are assigned (the others stay in bin 0).
std::vector<int> optimizer_owners(gn_model* m, int shard_count, const std::vector<int>* within = nullptr, int within_value = 0);

// model_latent.cu: the two block variants of the latent preset, inference only.
// Attention of layer l from H = norm(x) (with its tf32 split in b.S1h/b.S1l on the tensor-core path):
// writes the head outputs [rows, Hq*D] to O (before c_proj) and appends to the latent cache.
int latent_attention(gn_model* m, FwdBufs& b, const FwdArgs& a, int l, const float* H, float* O);
// Feed-forward of layer l: XOUT = MID + shared_expert(Mn) + routed_experts(Mn).
int moe_ffn(gn_model* m, FwdBufs& b, const FwdArgs& a, int l, const float* Mn, const float* MID, float* XOUT);

}  // namespace gnm
