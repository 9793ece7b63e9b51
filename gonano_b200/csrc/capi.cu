// C entry points of Tier A (one per kernels.Backend method, kernels/backend.go:
// 16-297) and of the stand-alone RL-step kernels.  Pointers may be host or
// device memory: host buffers are staged through device memory and the call
// returns once the results are back, which is what a cgo caller needs (Go
// memory must not be retained after the call returns).  One process-wide lock
// serialises these calls: the reference invokes its backend from many
// goroutines at once (model/attention.go:311-320, tensors/loss.go:30-37).
#include <atomic>
#include <cstdarg>
#include <mutex>
#include <vector>

#include "kernels.cuh"

namespace gn {

static thread_local char g_error[1024] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_error; }

static std::atomic<int64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void count_launches(int64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

int gemm_tcgen05_supported(const GemmArgs& a);
int gemm_tcgen05(const GemmArgs& a, cudaStream_t s);
void gemm_tcgen05_invalidate();
void gemm_tcgen05_mark_stale();
int gemm_tcgen05_check(cudaStream_t s);
void gemm_tcgen05_release(cudaStream_t s);
int gemm_tcgen05_option(cudaStream_t s, const char* name, int value);
void gemm_release_stream(cudaStream_t s) {
#ifdef GN_HAVE_TCGEN05
  gemm_tcgen05_release(s);
#else
  (void)s;
#endif
}
int gemm_set_option(cudaStream_t s, const char* name, int value) {
#ifdef GN_HAVE_TCGEN05
  return gemm_tcgen05_option(s, name, value);
#else
  (void)s; (void)value;
  set_error("unknown option '%s'", name);
  return GN_ERR_INVALID;
#endif
}
int num_sms() {
  static std::atomic<int> cache[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  int v = cache[device].load(std::memory_order_relaxed);
  if (v <= 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) { cudaGetLastError(); v = 148; }
    cache[device].store(v, std::memory_order_relaxed);
  }
  return v;
}
void gemm_invalidate_static() {
#ifdef GN_HAVE_TCGEN05
  gemm_tcgen05_invalidate();
#endif
}
void gemm_mark_static_stale() {
#ifdef GN_HAVE_TCGEN05
  gemm_tcgen05_mark_stale();
#endif
}
int gemm_check_error(cudaStream_t s) {
#ifdef GN_HAVE_TCGEN05
  return gemm_tcgen05_check(s);
#else
  (void)s;
  return GN_OK;
#endif
}
int gemm_default_kind() {
#ifdef GN_HAVE_TCGEN05
  return 1;
#else
  return 0;
#endif
}
int gemm_dispatch(const GemmArgs& a, int kind, cudaStream_t s) {
#ifdef GN_HAVE_TCGEN05
  if (kind == 1 && gemm_tcgen05_supported(a)) return gemm_tcgen05(a, s);
#endif
  (void)kind;
  if (a.leave) *a.leave = Partials{a.C, 1, 0, a.ldc};
  GN_TRY(gemm_simt(a, s));
  // the caller asked for the output's tf32 split (the tensor-core epilogue writes it; here it is a pass of its own)
  if (a.c_hi && a.c_lo) GN_TRY(split_matrix_launch(a.C, a.c_hi, a.c_lo, a.M, a.N, a.ldc, s));
  return GN_OK;
}

int gemm_grouped_dispatch(const GemmArgs& a, int kind, cudaStream_t s) {
#ifdef GN_HAVE_TCGEN05
  if (kind == 1 && a.groups > 0 && gemm_tcgen05_supported(a)) return gemm_tcgen05(a, s);
#endif
  (void)kind;
  GN_REQUIRE(a.lda == a.K && a.ldb == a.K && a.ldc == a.N, "grouped product: the float32 kernel wants packed operands");
  return grouped_matmul_t_launch(a.C, a.A, a.B, a.group_counts, a.groups, a.N, a.K, a.M, s);
}

namespace {

std::mutex g_lock;
cudaStream_t g_stream = nullptr;
int g_stream_device = -1;   // the stand-alone calls run on the device that was current at the first of them

int tier_a_stream(cudaStream_t* out) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) { set_error("no CUDA device available: %s", cudaGetErrorString(e)); return GN_ERR_CUDA; }
  int device = 0;
  GN_CUDA(cudaGetDevice(&device));
  if (!g_stream) { GN_CUDA(cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking)); g_stream_device = device; }
  if (device != g_stream_device) {
    set_error("the stand-alone calls of this process run on device %d (current at their first use); device %d is current now - use a gn_ctx for other devices",
              g_stream_device, device);
    return GN_ERR_UNSUPPORTED;
  }
  *out = g_stream;
  return GN_OK;
}

}  // namespace
cudaStream_t tier_a_stream_or_null() { return g_stream; }
namespace {

bool on_device(const void* p) {
  cudaPointerAttributes at;
  cudaError_t e = cudaPointerGetAttributes(&at, p);
  if (e != cudaSuccess) { cudaGetLastError(); return false; }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

// Stages host buffers for the duration of one call.
struct Stage {
  cudaStream_t s;
  struct Back { void* host; void* dev; size_t bytes; };
  std::vector<void*> owned;
  std::vector<Back> back;
  int status = GN_OK;
  explicit Stage(cudaStream_t st) : s(st) {}
  ~Stage() { for (void* p : owned) cudaFree(p); }
  template <typename T>
  const T* in(const T* p, size_t n) {
    if (!p || n == 0 || on_device(p) || status != GN_OK) return p;
    void* dev = nullptr;
    if (cudaMalloc(&dev, n * sizeof(T)) != cudaSuccess) { set_error("staging: cudaMalloc of %zu bytes failed", n * sizeof(T)); status = GN_ERR_NOMEM; return nullptr; }
    owned.push_back(dev);
    if (cudaMemcpyAsync(dev, p, n * sizeof(T), cudaMemcpyHostToDevice, s) != cudaSuccess) { set_error("staging: host to device copy failed"); status = GN_ERR_CUDA; }
    return (const T*)dev;
  }
  template <typename T>
  T* out(T* p, size_t n, bool read_too = false) {
    if (!p || n == 0 || on_device(p) || status != GN_OK) return p;
    void* dev = nullptr;
    if (cudaMalloc(&dev, n * sizeof(T)) != cudaSuccess) { set_error("staging: cudaMalloc of %zu bytes failed", n * sizeof(T)); status = GN_ERR_NOMEM; return nullptr; }
    owned.push_back(dev);
    if (read_too && cudaMemcpyAsync(dev, p, n * sizeof(T), cudaMemcpyHostToDevice, s) != cudaSuccess) { set_error("staging: host to device copy failed"); status = GN_ERR_CUDA; }
    back.push_back({p, dev, n * sizeof(T)});
    return (T*)dev;
  }
  // device scratch that lives until the call returns
  template <typename T>
  T* temp(size_t n) {
    if (status != GN_OK) return nullptr;
    void* dev = nullptr;
    if (cudaMalloc(&dev, std::max<size_t>(n, 1) * sizeof(T)) != cudaSuccess) { set_error("staging: cudaMalloc of %zu bytes failed", n * sizeof(T)); status = GN_ERR_NOMEM; return nullptr; }
    owned.push_back(dev);
    return (T*)dev;
  }
  int finish() {
    if (status != GN_OK) return status;
    for (auto& b : back) GN_CUDA(cudaMemcpyAsync(b.host, b.dev, b.bytes, cudaMemcpyDeviceToHost, s));
    GN_CUDA(cudaStreamSynchronize(s));
    return GN_OK;
  }
};

#define GN_BEGIN()                               \
  std::lock_guard<std::mutex> guard__(g_lock);   \
  cudaStream_t s = nullptr;                      \
  GN_TRY(tier_a_stream(&s));                     \
  Stage st(s)

#define GN_END()                                 \
  return st.finish()

int ew2(int op, float* dst, const float* a, const float* b, float f, int64_t n) {
  if (n <= 0) return GN_OK;
  GN_REQUIRE(dst && a, "elementwise: null pointer");
  GN_BEGIN();
  const float* da = st.in(a, n); const float* db = b ? st.in(b, n) : nullptr; float* dd = st.out(dst, n);
  if (st.status != GN_OK) return st.status;
  GN_TRY(ew_launch(op, dd, da, db, f, n, s));
  GN_END();
}

}  // namespace
}  // namespace gn

using namespace gn;

extern "C" {

const char* gn_last_error(void) { return get_error(); }
const char* gn_version(void) { return "gonano-cuda 0.1 (sm_100a)"; }
int gn_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return 0; }
  return count;
}

int gn_add(float* d, const float* a, const float* b, int64_t n) { return ew2(EW_ADD, d, a, b, 0, n); }
int gn_subtract(float* d, const float* a, const float* b, int64_t n) { return ew2(EW_SUB, d, a, b, 0, n); }
int gn_multiply(float* d, const float* a, const float* b, int64_t n) { return ew2(EW_MUL, d, a, b, 0, n); }
int gn_divide(float* d, const float* a, const float* b, int64_t n) { return ew2(EW_DIV, d, a, b, 0, n); }
int gn_scale(float* d, const float* a, float f, int64_t n) { return ew2(EW_SCALE, d, a, nullptr, f, n); }
int gn_add_scaled(float* d, const float* base, const float* sc, float f, int64_t n) { return ew2(EW_ADD_SCALED, d, base, sc, f, n); }
int gn_negate(float* d, const float* a, int64_t n) { return ew2(EW_NEG, d, a, nullptr, 0, n); }
int gn_abs(float* d, const float* a, int64_t n) { return ew2(EW_ABS, d, a, nullptr, 0, n); }
int gn_square(float* d, const float* a, int64_t n) { return ew2(EW_SQUARE, d, a, nullptr, 0, n); }
int gn_relu_squared(float* d, const float* a, int64_t n) { return ew2(EW_RELU2, d, a, nullptr, 0, n); }
int gn_swiglu(float* d, const float* gate, const float* up, float clamp, int64_t n) { return ew2(EW_SWIGLU, d, gate, up, clamp, n); }
int gn_exp(float* d, const float* a, int64_t n) { return ew2(EW_EXP, d, a, nullptr, 0, n); }
int gn_sigmoid(float* d, const float* a, int64_t n) { return ew2(EW_SIGMOID, d, a, nullptr, 0, n); }
int gn_tanh(float* d, const float* a, int64_t n) { return ew2(EW_TANH, d, a, nullptr, 0, n); }
int gn_rsqrt(float* d, const float* a, int64_t n) { return ew2(EW_RSQRT, d, a, nullptr, 0, n); }

int gn_swiglu_backward(float* gg, float* ug, const float* gate, const float* up, const float* og, float clamp, int64_t n) {
  if (n <= 0) return GN_OK;
  GN_REQUIRE(gg && ug && gate && up && og, "swiglu_backward: null pointer");
  GN_BEGIN();
  const float* dg = st.in(gate, n); const float* du = st.in(up, n); const float* dog = st.in(og, n);
  float* dgg = st.out(gg, n); float* dug = st.out(ug, n);
  if (st.status != GN_OK) return st.status;
  GN_TRY(swiglu_backward_launch(dgg, dug, dg, du, dog, clamp, n, s));
  GN_END();
}

static int reduce_scalar(int which, const float* v, const float* w, int64_t n, float* out_f, int64_t* out_i) {
  GN_BEGIN();
  const float* dv = st.in(v, n > 0 ? n : 0); const float* dw = w ? st.in(w, n) : nullptr;
  void* res = nullptr;
  GN_CUDA(cudaMalloc(&res, 8));
  st.owned.push_back(res);
  if (st.status != GN_OK) return st.status;
  if (which == 0) GN_TRY(reduce_sum_launch(dv, n, (float*)res, s));
  else if (which == 1) GN_TRY(reduce_max_launch(dv, n, (float*)res, s));
  else if (which == 2) GN_TRY(reduce_argmax_launch(dv, n, (int64_t*)res, s));
  else GN_TRY(dot_launch(dv, dw, n, (float*)res, s));
  if (which == 2) GN_CUDA(cudaMemcpyAsync(out_i, res, 8, cudaMemcpyDeviceToHost, s));
  else GN_CUDA(cudaMemcpyAsync(out_f, res, 4, cudaMemcpyDeviceToHost, s));
  GN_END();
}
int gn_sum(const float* v, int64_t n, float* out) { GN_REQUIRE(out, "sum: null out"); if (n <= 0) { *out = 0; return GN_OK; } return reduce_scalar(0, v, nullptr, n, out, nullptr); }
int gn_max(const float* v, int64_t n, float* out) { GN_REQUIRE(out, "max: null out"); if (n <= 0) { *out = 0; return GN_OK; } return reduce_scalar(1, v, nullptr, n, out, nullptr); }
int gn_argmax(const float* v, int64_t n, int64_t* out) { GN_REQUIRE(out, "argmax: null out"); if (n <= 0) { *out = 0; return GN_OK; } return reduce_scalar(2, v, nullptr, n, nullptr, out); }
int gn_dot_product(const float* a, const float* b, int64_t n, float* out) { GN_REQUIRE(out, "dot: null out"); if (n <= 0) { *out = 0; return GN_OK; } return reduce_scalar(3, a, b, n, out, nullptr); }

static int matmul_any(float* dst, const float* left, const float* right, int rows, int cols, int inner, int b_trans) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  GN_REQUIRE(dst && left && right && inner >= 0, "matmul: bad argument");
  GN_BEGIN();
  GemmArgs g;
  g.A = st.in(left, (size_t)rows * inner); g.B = st.in(right, (size_t)cols * inner); g.C = st.out(dst, (size_t)rows * cols);
  if (st.status != GN_OK) return st.status;
  g.M = rows; g.N = cols; g.K = inner; g.lda = inner; g.ldb = b_trans ? inner : cols; g.ldc = cols; g.b_trans = b_trans;
  GN_TRY(gemm_dispatch(g, gemm_default_kind(), s));
  GN_TRY(st.finish());
  return gemm_check_error(s);
}
int gn_matmul(float* dst, const float* l, const float* r, int rows, int cols, int inner) { return matmul_any(dst, l, r, rows, cols, inner, 0); }
int gn_matmul_transposed(float* dst, const float* l, const float* r, int rows, int cols, int inner) { return matmul_any(dst, l, r, rows, cols, inner, 1); }

int gn_indexer_scores(float* dst, const float* q, const float* k, const float* w, int rows, int blocks, int heads, int dim) {
  if (rows <= 0 || blocks <= 0) return GN_OK;
  GN_BEGIN();
  const float* dq = st.in(q, (size_t)rows * heads * dim); const float* dk = st.in(k, (size_t)blocks * heads * dim); const float* dw = st.in(w, heads);
  float* dd = st.out(dst, (size_t)rows * blocks);
  if (st.status != GN_OK) return st.status;
  GN_TRY(indexer_scores_launch(dd, dq, dk, dw, rows, blocks, heads, dim, s));
  GN_END();
}
int gn_indexer_block_max(float* dst, const float* scores, int rows, int blocks, int group) {
  if (rows <= 0 || blocks <= 0) return GN_OK;
  if (group < 1) group = 1;
  int groups = (blocks + group - 1) / group;
  GN_BEGIN();
  const float* ds = st.in(scores, (size_t)rows * blocks); float* dd = st.out(dst, (size_t)rows * groups);
  if (st.status != GN_OK) return st.status;
  GN_TRY(indexer_block_max_launch(dd, ds, rows, blocks, group, s));
  GN_END();
}

// ChannelCompressor.Forward (model/compress.go:93-177)
int gn_compressor_forward(const float* hidden, const float* value, const float* logit_weight, const float* bias, int batch, int seq, int embed, int channels,
                          int ratio, float* compressed, float* probabilities) {
  if (batch <= 0 || seq <= 0 || channels <= 0) return GN_OK;
  GN_REQUIRE(hidden && value && logit_weight && bias && compressed && ratio >= 1 && embed > 0, "compressor_forward: bad argument");
  const int blocks = (seq + ratio - 1) / ratio;
  GN_BEGIN();
  const size_t rows = (size_t)batch * seq;
  const float* dh = st.in(hidden, rows * embed); const float* dv = st.in(value, rows * channels);
  const float* dw = st.in(logit_weight, (size_t)channels * embed); const float* db = st.in(bias, (size_t)ratio * channels);
  float* dc = st.out(compressed, (size_t)batch * blocks * channels);
  float* dp = probabilities ? st.out(probabilities, (size_t)batch * blocks * ratio * channels) : nullptr;
  float* logits = st.temp<float>(rows * channels);
  if (st.status != GN_OK) return st.status;
  GemmArgs g;
  g.A = dh; g.B = dw; g.C = logits; g.M = (int)rows; g.N = channels; g.K = embed; g.lda = embed; g.ldb = embed; g.ldc = channels; g.b_trans = 1;
  GN_TRY(gemm_dispatch(g, gemm_default_kind(), s));
  GN_TRY(compressor_pool_launch(logits, db, dv, batch, seq, channels, ratio, dc, dp, s));
  GN_TRY(st.finish());
  return gemm_check_error(s);
}
// ChannelCompressor.Backward (model/compress.go:182-237), no segment mask: grad_hidden and grad_value are overwritten,
// grad_weight and grad_bias accumulated (Tensor.AddGrad)
int gn_compressor_backward(const float* hidden, const float* value, const float* logit_weight, const float* probabilities, const float* compressed,
                           const float* grad_compressed, int batch, int seq, int embed, int channels, int ratio, float* grad_hidden, float* grad_value,
                           float* grad_weight, float* grad_bias) {
  if (batch <= 0 || seq <= 0 || channels <= 0) return GN_OK;
  GN_REQUIRE(hidden && value && logit_weight && probabilities && compressed && grad_compressed && grad_hidden && grad_value && grad_weight && grad_bias &&
             ratio >= 1 && embed > 0, "compressor_backward: bad argument");
  const int blocks = (seq + ratio - 1) / ratio;
  GN_BEGIN();
  const size_t rows = (size_t)batch * seq;
  const float* dh = st.in(hidden, rows * embed); const float* dv = st.in(value, rows * channels);
  const float* dw = st.in(logit_weight, (size_t)channels * embed);
  const float* dp = st.in(probabilities, (size_t)batch * blocks * ratio * channels); const float* dc = st.in(compressed, (size_t)batch * blocks * channels);
  const float* dg = st.in(grad_compressed, (size_t)batch * blocks * channels);
  float* gh = st.out(grad_hidden, rows * embed); float* gv = st.out(grad_value, rows * channels);
  float* gw = st.out(grad_weight, (size_t)channels * embed, true); float* gb = st.out(grad_bias, (size_t)ratio * channels, true);
  float* gl = st.temp<float>(rows * channels);
  if (st.status != GN_OK) return st.status;
  // rows of a trailing partial block that do not exist are not written by the kernel: none are left out, every (b, t) belongs to a block
  GN_TRY(compressor_pool_backward_launch(dv, dp, dc, dg, batch, seq, channels, ratio, gl, gv, gb, s));
  { GemmArgs g; g.A = gl; g.lda = channels; g.B = dw; g.ldb = embed; g.b_trans = 0; g.C = gh; g.ldc = embed; g.M = (int)rows; g.N = embed; g.K = channels;
    GN_TRY(gemm_dispatch(g, gemm_default_kind(), s)); }                       // dhidden = dlogits W
  { GemmArgs g; g.A = gl; g.lda = channels; g.a_trans = 1; g.B = dh; g.ldb = embed; g.b_trans = 0; g.C = gw; g.ldc = embed; g.M = channels; g.N = embed; g.K = (int)rows;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm_dispatch(g, gemm_default_kind(), s)); }   // dW += dlogits^T hidden
  GN_TRY(st.finish());
  return gemm_check_error(s);
}
// compressForward (model/compress_attention.go:562-622), no segment mask: one logit product, then the block softmax applied to the keys and values of every kv head
int gn_compress_forward(const float* hidden, const float* key, const float* value, const float* logit_weight, const float* bias, int batch, int n_kv_head, int seq,
                        int embed, int head_dim, int ratio, float* key_c, float* value_c, float* probabilities) {
  if (batch <= 0 || seq <= 0 || head_dim <= 0 || n_kv_head <= 0) return GN_OK;
  GN_REQUIRE(hidden && key && value && logit_weight && bias && key_c && value_c && ratio >= 1 && embed > 0, "compress_forward: bad argument");
  const int blocks = (seq + ratio - 1) / ratio;
  GN_BEGIN();
  const size_t rows = (size_t)batch * seq, nkv = (size_t)batch * n_kv_head * seq * head_dim, nc = (size_t)batch * n_kv_head * blocks * head_dim;
  const float* dh = st.in(hidden, rows * embed); const float* dk = st.in(key, nkv); const float* dv = st.in(value, nkv);
  const float* dw = st.in(logit_weight, (size_t)head_dim * embed); const float* db = st.in(bias, (size_t)ratio * head_dim);
  float* kc = st.out(key_c, nc); float* vc = st.out(value_c, nc);
  const size_t np = (size_t)batch * blocks * ratio * head_dim;
  float* dp = probabilities ? st.out(probabilities, np) : st.temp<float>(np);
  float* logits = st.temp<float>(rows * head_dim);
  if (st.status != GN_OK) return st.status;
  GemmArgs g;
  g.A = dh; g.B = dw; g.C = logits; g.M = (int)rows; g.N = head_dim; g.K = embed; g.lda = embed; g.ldb = embed; g.ldc = head_dim; g.b_trans = 1;
  GN_TRY(gemm_dispatch(g, gemm_default_kind(), s));
  GN_TRY(compress_heads_launch(logits, db, dk, dv, batch, n_kv_head, seq, head_dim, ratio, kc, vc, dp, s));
  GN_TRY(st.finish());
  return gemm_check_error(s);
}
// compressBackward (model/compress_attention.go:1182-1209): grad_hidden, grad_key, grad_value are overwritten, grad_weight and grad_bias accumulated
int gn_compress_backward(const float* hidden, const float* key, const float* value, const float* logit_weight, const float* probabilities, const float* key_c,
                         const float* value_c, const float* grad_key_c, const float* grad_value_c, int batch, int n_kv_head, int seq, int embed, int head_dim,
                         int ratio, float* grad_hidden, float* grad_key, float* grad_value, float* grad_weight, float* grad_bias) {
  if (batch <= 0 || seq <= 0 || head_dim <= 0 || n_kv_head <= 0) return GN_OK;
  GN_REQUIRE(hidden && key && value && logit_weight && probabilities && key_c && value_c && grad_key_c && grad_value_c && grad_hidden && grad_key && grad_value &&
             grad_weight && grad_bias && ratio >= 1 && embed > 0, "compress_backward: bad argument");
  const int blocks = (seq + ratio - 1) / ratio;
  GN_BEGIN();
  const size_t rows = (size_t)batch * seq, nkv = (size_t)batch * n_kv_head * seq * head_dim, nc = (size_t)batch * n_kv_head * blocks * head_dim;
  const float* dh = st.in(hidden, rows * embed); const float* dk = st.in(key, nkv); const float* dv = st.in(value, nkv);
  const float* dw = st.in(logit_weight, (size_t)head_dim * embed);
  const float* dp = st.in(probabilities, (size_t)batch * blocks * ratio * head_dim);
  const float* kc = st.in(key_c, nc); const float* vc = st.in(value_c, nc); const float* gkc = st.in(grad_key_c, nc); const float* gvc = st.in(grad_value_c, nc);
  float* gh = st.out(grad_hidden, rows * embed); float* gk = st.out(grad_key, nkv); float* gv = st.out(grad_value, nkv);
  float* gw = st.out(grad_weight, (size_t)head_dim * embed, true); float* gb = st.out(grad_bias, (size_t)ratio * head_dim, true);
  float* gl = st.temp<float>(rows * head_dim);
  if (st.status != GN_OK) return st.status;
  GN_TRY(compress_heads_backward_launch(dk, dv, dp, kc, vc, gkc, gvc, batch, n_kv_head, seq, head_dim, ratio, gl, gk, gv, gb, s));
  { GemmArgs g; g.A = gl; g.lda = head_dim; g.B = dw; g.ldb = embed; g.b_trans = 0; g.C = gh; g.ldc = embed; g.M = (int)rows; g.N = embed; g.K = head_dim;
    GN_TRY(gemm_dispatch(g, gemm_default_kind(), s)); }                       // dhidden = dlogits W
  { GemmArgs g; g.A = gl; g.lda = head_dim; g.a_trans = 1; g.B = dh; g.ldb = embed; g.b_trans = 0; g.C = gw; g.ldc = embed; g.M = head_dim; g.N = embed; g.K = (int)rows;
    g.epilogue = EPI_ACCUM; GN_TRY(gemm_dispatch(g, gemm_default_kind(), s)); }   // dW += dlogits^T hidden
  GN_TRY(st.finish());
  return gemm_check_error(s);
}
// compressedAttentionForward (model/compress_attention.go:624-673), no segment mask
int gn_compressed_attention_forward(const float* query, const float* key_c, const float* value_c, int batch, int n_head, int n_kv_head, int seq, int head_dim,
                                    int blocks, int ratio, float* out, float* lse) {
  return gn_compressed_attention_forward_at(query, key_c, value_c, batch, n_head, n_kv_head, seq, head_dim, blocks, ratio, 0, out, lse);
}
// the dense loop of forwardCompressed (model/compress_attention.go:962-1003): `seq` new tokens at positions position_offset .. over `blocks` cached blocks
int gn_compressed_attention_forward_at(const float* query, const float* key_c, const float* value_c, int batch, int n_head, int n_kv_head, int seq, int head_dim,
                                       int blocks, int ratio, int position_offset, float* out, float* lse) {
  if (batch <= 0 || seq <= 0) return GN_OK;
  GN_REQUIRE(query && (blocks == 0 || (key_c && value_c)) && out && blocks >= 0 && position_offset >= 0, "compressed_attention_forward: bad argument");
  GN_BEGIN();
  const size_t nq = (size_t)batch * n_head * seq * head_dim, nk = (size_t)batch * n_kv_head * blocks * head_dim;
  const float* dq = st.in(query, nq); const float* dk = st.in(key_c, nk); const float* dv = st.in(value_c, nk);
  float* dout = st.out(out, nq); float* dl = lse ? st.out(lse, (size_t)batch * n_head * seq) : nullptr;
  // One decode step over a long compressed cache: the rows' blocks are a key / value cache of `count` positions, so the
  // split-context decode attention kernel (a CTA per row and kv head and context share, the group's heads served from
  // one read of each row) takes it; the warp-per-token form would walk the blocks one warp per group.
  const int hr = n_kv_head > 0 ? n_head / n_kv_head : 0;
  if (seq == 1 && head_dim == 128 && blocks >= 64 && n_kv_head > 0 && n_head % n_kv_head == 0 && ratio >= 1 &&
      (hr == 1 || hr == 2 || hr == 3 || hr == 4 || hr == 8)) {
    const int count = std::min(position_offset / ratio, blocks);
    const int splits = std::max(2, attention_decode_splits(batch, n_kv_head, blocks));
    std::vector<int32_t> ctx_host((size_t)batch, count);
    const int32_t* ctx_len = st.in(ctx_host.data(), (size_t)batch);
    float* pa = st.temp<float>((size_t)batch * n_head * splits * head_dim); float* pm = st.temp<float>((size_t)batch * n_head * splits * 2);
    float* dl2 = dl ? dl : st.temp<float>((size_t)batch * n_head);
    if (st.status != GN_OK) return st.status;
    GN_TRY(attention_decode_launch(dq, (int64_t)n_head * head_dim, dk, dv, (int64_t)n_kv_head * blocks * head_dim, (int64_t)blocks * head_dim, ctx_len, batch, n_head,
                                   n_kv_head, head_dim, -1, dout, (int64_t)n_head * head_dim, pa, pm, splits, s, nullptr, nullptr, 1, 0, dl2));
    GN_END();
  }
  if (st.status != GN_OK) return st.status;
  GN_TRY(compressed_attention_launch(dq, dk, dv, batch, n_head, n_kv_head, seq, head_dim, blocks, ratio, dout, dl, nullptr, nullptr, 0, position_offset, s));
  GN_END();
}
// compressedAttentionBackward (model/compress_attention.go:735-781), no segment mask; the three gradients accumulate
int gn_compressed_attention_backward(const float* query, const float* key_c, const float* value_c, const float* out_grad, const float* lse,
                                     const float* row_correction, int batch, int n_head, int n_kv_head, int seq, int head_dim, int blocks, int ratio,
                                     float* dq, float* dkc, float* dvc) {
  if (batch <= 0 || seq <= 0 || blocks <= 0) return GN_OK;
  GN_REQUIRE(query && key_c && value_c && out_grad && lse && dq && dkc && dvc, "compressed_attention_backward: bad argument");
  GN_BEGIN();
  const size_t nq = (size_t)batch * n_head * seq * head_dim, nk = (size_t)batch * n_kv_head * blocks * head_dim, nt = (size_t)batch * n_head * seq;
  const float* pq = st.in(query, nq); const float* pk = st.in(key_c, nk); const float* pv = st.in(value_c, nk);
  const float* pg = st.in(out_grad, nq); const float* pl = st.in(lse, nt); const float* pr = row_correction ? st.in(row_correction, nt) : nullptr;
  float* gq = st.out(dq, nq, true); float* gk = st.out(dkc, nk, true); float* gv = st.out(dvc, nk, true);
  float* scratch = st.temp<float>(nt);
  if (st.status != GN_OK) return st.status;
  GN_TRY(compressed_attention_backward_launch(pq, pk, pv, pg, pl, pr, scratch, batch, n_head, n_kv_head, seq, head_dim, blocks, ratio, gq, gk, gv, nullptr, nullptr, 0, s));
  GN_END();
}
// compressedAttentionForwardSparse (model/compress_attention.go:321-374), no segment mask
int gn_compressed_attention_sparse_forward(const float* query, const float* key_c, const float* value_c, const int32_t* selection, const int32_t* counts, int batch,
                                           int n_head, int n_kv_head, int seq, int head_dim, int blocks, int topk, float* out, float* lse) {
  if (batch <= 0 || seq <= 0) return GN_OK;
  GN_REQUIRE(query && key_c && value_c && selection && counts && out && blocks >= 0 && topk >= 1, "compressed_attention_sparse_forward: bad argument");
  GN_BEGIN();
  const size_t nq = (size_t)batch * n_head * seq * head_dim, nk = (size_t)batch * n_kv_head * blocks * head_dim, nt = (size_t)batch * n_kv_head * seq;
  const float* dq = st.in(query, nq); const float* dk = st.in(key_c, nk); const float* dv = st.in(value_c, nk);
  const int32_t* ds = st.in(selection, nt * topk); const int32_t* dc = st.in(counts, nt);
  float* dout = st.out(out, nq); float* dl = lse ? st.out(lse, (size_t)batch * n_head * seq) : nullptr;
  if (st.status != GN_OK) return st.status;
  GN_TRY(compressed_attention_launch(dq, dk, dv, batch, n_head, n_kv_head, seq, head_dim, blocks, 1, dout, dl, ds, dc, topk, 0, s));
  GN_END();
}
// compressedAttentionBackwardSparse (model/compress_attention.go:376-433), no segment mask; the three gradients accumulate
int gn_compressed_attention_sparse_backward(const float* query, const float* key_c, const float* value_c, const float* out_grad, const float* lse,
                                            const float* row_correction, const int32_t* selection, const int32_t* counts, int batch, int n_head, int n_kv_head,
                                            int seq, int head_dim, int blocks, int topk, float* dq, float* dkc, float* dvc) {
  if (batch <= 0 || seq <= 0 || blocks <= 0) return GN_OK;
  GN_REQUIRE(query && key_c && value_c && out_grad && lse && selection && counts && topk >= 1 && dq && dkc && dvc, "compressed_attention_sparse_backward: bad argument");
  GN_BEGIN();
  const size_t nq = (size_t)batch * n_head * seq * head_dim, nk = (size_t)batch * n_kv_head * blocks * head_dim, nt = (size_t)batch * n_head * seq;
  const size_t ns = (size_t)batch * n_kv_head * seq;
  const float* pq = st.in(query, nq); const float* pk = st.in(key_c, nk); const float* pv = st.in(value_c, nk);
  const float* pg = st.in(out_grad, nq); const float* pl = st.in(lse, nt); const float* pr = row_correction ? st.in(row_correction, nt) : nullptr;
  const int32_t* ps = st.in(selection, ns * topk); const int32_t* pc = st.in(counts, ns);
  float* gq = st.out(dq, nq, true); float* gk = st.out(dkc, nk, true); float* gv = st.out(dvc, nk, true);
  float* scratch = st.temp<float>(nt);
  if (st.status != GN_OK) return st.status;
  uint32_t* bits = st.temp<uint32_t>((size_t)batch * n_kv_head * seq * ((blocks + 31) / 32));
  if (st.status != GN_OK) return st.status;
  GN_TRY(compressed_attention_backward_launch(pq, pk, pv, pg, pl, pr, scratch, batch, n_head, n_kv_head, seq, head_dim, blocks, 1, gq, gk, gv, ps, pc, topk, s, bits));
  GN_END();
}
// mergeAttentionBranches (model/compress_attention.go:440-466)
int gn_attention_merge(const float* out_a, const float* lse_a, const float* out_b, const float* lse_b, int64_t rows, int head_dim, float* out, float* lse) {
  if (rows <= 0) return GN_OK;
  GN_REQUIRE(out_a && lse_a && out_b && lse_b && out && head_dim > 0, "attention_merge: bad argument");
  GN_BEGIN();
  const float* da = st.in(out_a, (size_t)rows * head_dim); const float* dla = st.in(lse_a, (size_t)rows);
  const float* db = st.in(out_b, (size_t)rows * head_dim); const float* dlb = st.in(lse_b, (size_t)rows);
  float* dout = st.out(out, (size_t)rows * head_dim); float* dl = lse ? st.out(lse, (size_t)rows) : nullptr;
  if (st.status != GN_OK) return st.status;
  GN_TRY(attention_merge_launch(da, dla, db, dlb, rows, head_dim, dout, dl, s));
  GN_END();
}
// SelectBlocks (model/indexer.go:186-206)
int gn_select_blocks(const float* scores, int tokens, int blocks, int position_offset, int ratio, int topk, int32_t* selection, int32_t* counts) {
  if (tokens <= 0) return GN_OK;
  GN_REQUIRE(scores && counts && blocks > 0 && ratio >= 1 && topk >= 0 && (selection || topk == 0), "select_blocks: bad argument");
  GN_BEGIN();
  const float* ds = st.in(scores, (size_t)tokens * blocks);
  int32_t* dsel = topk > 0 ? st.out(selection, (size_t)tokens * topk) : nullptr; int32_t* dc = st.out(counts, (size_t)tokens);
  if (st.status != GN_OK) return st.status;
  GN_TRY(select_blocks_launch(ds, tokens, blocks, position_offset, ratio, topk, dsel, dc, s));
  GN_END();
}
// the score part of SparseIndexer.Backward (model/indexer.go:107-151) for one key set
int gn_indexer_scores_backward(const float* grad_scores, const float* query, const float* key, const float* weight, int rows, int blocks, int heads, int dim,
                               float* grad_query, float* grad_key, float* grad_weight) {
  if (rows <= 0 || blocks <= 0 || heads <= 0) return GN_OK;
  GN_REQUIRE(grad_scores && query && key && weight && grad_query && grad_key && grad_weight && dim >= 1, "indexer_scores_backward: bad argument");
  GN_BEGIN();
  const float* pg = st.in(grad_scores, (size_t)rows * blocks); const float* pq = st.in(query, (size_t)rows * heads * dim);
  const float* pk = st.in(key, (size_t)blocks * heads * dim); const float* pw = st.in(weight, (size_t)heads);
  float* gq = st.out(grad_query, (size_t)rows * heads * dim); float* gk = st.out(grad_key, (size_t)blocks * heads * dim);
  float* gw = st.out(grad_weight, (size_t)heads, true);
  float* wpart = st.temp<float>((size_t)rows * heads);
  const int kplanes = rows >= 64 && blocks >= 64 ? 16 : 0;
  float* kpart = kplanes ? st.temp<float>((size_t)kplanes * blocks * heads * dim) : nullptr;
  if (st.status != GN_OK) return st.status;
  GN_TRY(indexer_scores_backward_launch(pg, pq, pk, pw, rows, blocks, heads, dim, gq, gk, gw, wpart, s, kpart, kplanes));
  GN_END();
}
// distillationTarget (model/compress_attention.go:155-196) for every (batch, kv head)
int gn_indexer_distillation_target(const float* query, const float* key_c, int batch, int n_head, int n_kv_head, int seq, int head_dim, int blocks, int ratio,
                                   float* target) {
  if (batch <= 0 || seq <= 0 || blocks <= 0) return GN_OK;
  GN_REQUIRE(query && key_c && target && n_kv_head > 0, "indexer_distillation_target: bad argument");
  GN_BEGIN();
  const float* pq = st.in(query, (size_t)batch * n_head * seq * head_dim); const float* pk = st.in(key_c, (size_t)batch * n_kv_head * blocks * head_dim);
  float* pt = st.out(target, (size_t)batch * n_kv_head * seq * blocks);
  if (st.status != GN_OK) return st.status;
  float* qsum = (seq >= 64 && blocks >= 64) ? st.temp<float>((size_t)batch * n_kv_head * seq * head_dim + 1) : nullptr;
  if (st.status != GN_OK) return st.status;
  GN_TRY(distillation_target_launch(pq, pk, batch, n_head, n_kv_head, seq, head_dim, blocks, ratio, pt, s, qsum));
  GN_END();
}
// the score gradient of indexerDistillationGradient (model/compress_attention.go:120-151) with restrictIndexerToPool (:203-231)
int gn_indexer_distillation_grad(const float* scores, const float* target, const int32_t* candidates, const int32_t* candidate_counts, int cap, int64_t rows,
                                 int blocks, int seq, int ratio, float weight, float* grad_scores) {
  if (rows <= 0 || blocks <= 0) return GN_OK;
  GN_REQUIRE(scores && target && grad_scores && (!candidates || candidate_counts), "indexer_distillation_grad: bad argument");
  GN_BEGIN();
  const float* ps = st.in(scores, (size_t)rows * blocks); const float* pt = st.in(target, (size_t)rows * blocks);
  const int32_t* pc = candidates ? st.in(candidates, (size_t)rows * cap) : nullptr; const int32_t* pn = candidates ? st.in(candidate_counts, (size_t)rows) : nullptr;
  float* pg = st.out(grad_scores, (size_t)rows * blocks);
  if (st.status != GN_OK) return st.status;
  GN_TRY(distillation_grad_launch(ps, pt, pc, pn, cap, rows, blocks, seq, ratio, weight, pg, s));
  GN_END();
}
// selectFromScoreMatrix / selectRowBlockMax (model/indexer.go:358-381, 442-513)
int gn_hierarchical_cap(int pool, int candidate_budget) { pool = pool < 1 ? 1 : pool; const int g = (candidate_budget + pool - 1) / pool; return (g < 1 ? 1 : g) * pool; }
int gn_select_blocks_hierarchical(const float* scores, int tokens, int blocks, int position_offset, int ratio, int topk, int pool, int candidate_budget,
                                  int32_t* selection, int32_t* counts, int32_t* candidates, int32_t* candidate_counts) {
  if (tokens <= 0) return GN_OK;
  GN_REQUIRE(scores && counts && blocks > 0 && ratio >= 1 && topk >= 1 && selection && (!candidates || candidate_counts), "select_blocks_hierarchical: bad argument");
  pool = pool < 1 ? 1 : pool;
  const int cap = gn_hierarchical_cap(pool, candidate_budget);
  GN_BEGIN();
  const float* ds = st.in(scores, (size_t)tokens * blocks);
  int32_t* dsel = st.out(selection, (size_t)tokens * topk); int32_t* dc = st.out(counts, (size_t)tokens);
  int32_t* dcand = candidates ? st.out(candidates, (size_t)tokens * cap) : st.temp<int32_t>((size_t)tokens * cap);
  int32_t* dcc = candidates ? st.out(candidate_counts, (size_t)tokens) : st.temp<int32_t>((size_t)tokens);
  float* gmax = st.temp<float>((size_t)tokens * ((blocks + pool - 1) / pool));
  int32_t* chosen = st.temp<int32_t>((size_t)tokens * (cap / pool));
  if (st.status != GN_OK) return st.status;
  GN_TRY(select_hierarchical_launch(ds, tokens, blocks, position_offset, ratio, topk, pool, candidate_budget, gmax, chosen, dsel, dc, dcand, dcc, s));
  GN_END();
}
// selectWithinPool over a score matrix (model/indexer.go:547-613)
int gn_select_blocks_within_pool(const float* scores, int tokens, int blocks, int position_offset, int ratio, int topk, const int32_t* candidates,
                                 const int32_t* candidate_counts, int cap, int32_t* selection, int32_t* counts) {
  if (tokens <= 0) return GN_OK;
  GN_REQUIRE(scores && counts && blocks > 0 && ratio >= 1 && topk >= 1 && selection && candidates && candidate_counts && cap >= 1, "select_blocks_within_pool: bad argument");
  GN_BEGIN();
  const float* ds = st.in(scores, (size_t)tokens * blocks);
  const int32_t* dcand = st.in(candidates, (size_t)tokens * cap); const int32_t* dcc = st.in(candidate_counts, (size_t)tokens);
  int32_t* dsel = st.out(selection, (size_t)tokens * topk); int32_t* dc = st.out(counts, (size_t)tokens);
  if (st.status != GN_OK) return st.status;
  GN_TRY(select_within_pool_launch(ds, tokens, blocks, position_offset, ratio, topk, dcand, dcc, cap, dsel, dc, s));
  GN_END();
}

int gn_topk_indices(int32_t* dst, const float* scores, int rows, int count, int k) {
  if (rows <= 0 || count <= 0 || k <= 0) return GN_OK;
  GN_BEGIN();
  const float* ds = st.in(scores, (size_t)rows * count); int32_t* dd = st.out(dst, (size_t)rows * k, true);
  if (st.status != GN_OK) return st.status;
  GN_TRY(topk_indices_launch(dd, ds, rows, count, k, s));
  GN_END();
}
int gn_moe_gate_topk(const float* logits, const float* bias, float* probs, int32_t* sel, float* w, int rows, int experts, int k) {
  if (rows <= 0 || experts <= 0) return GN_OK;
  GN_REQUIRE(logits && bias && probs && sel && w && k > 0, "moe_gate_topk: bad argument");
  GN_BEGIN();
  const float* dl = st.in(logits, (size_t)rows * experts); const float* db = st.in(bias, experts);
  float* dp = st.out(probs, (size_t)rows * experts); int32_t* dsel = st.out(sel, (size_t)rows * k, true); float* dw = st.out(w, (size_t)rows * k, true);
  if (st.status != GN_OK) return st.status;
  GN_TRY(moe_gate_topk_launch(dl, db, dp, dsel, dw, rows, experts, k, s));
  GN_END();
}
int gn_grouped_matmul_transposed(float* dst, const float* input, const float* weight, const int32_t* counts, int experts, int cols, int inner) {
  GN_REQUIRE(counts && experts >= 0, "grouped_matmul: bad argument");
  GN_BEGIN();
  // The row total is needed on the host to size the launch.
  std::vector<int32_t> hc(experts);
  if (on_device(counts)) { GN_CUDA(cudaMemcpyAsync(hc.data(), counts, sizeof(int32_t) * experts, cudaMemcpyDeviceToHost, s)); GN_CUDA(cudaStreamSynchronize(s)); }
  else std::memcpy(hc.data(), counts, sizeof(int32_t) * experts);
  int64_t total = 0;
  for (int e = 0; e < experts; ++e) { GN_REQUIRE(hc[e] >= 0, "grouped_matmul: negative token count"); total += hc[e]; }
  if (total == 0 || cols <= 0) return GN_OK;
  const float* din = st.in(input, (size_t)total * inner); const float* dw = st.in(weight, (size_t)experts * cols * inner);
  const int32_t* dc = st.in(counts, experts); float* dd = st.out(dst, (size_t)total * cols);
  if (st.status != GN_OK) return st.status;
  { GemmArgs g; g.A = din; g.lda = inner; g.B = dw; g.ldb = inner; g.b_trans = 1; g.C = dd; g.ldc = cols; g.M = (int)total; g.N = cols; g.K = inner;
    g.group_counts = dc; g.groups = experts;
    GN_TRY(gemm_grouped_dispatch(g, gemm_default_kind(), s)); }
  GN_END();
}

int gn_adamw_step(float* param, float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, int step, float lr, float beta1, float beta2, float eps,
                  float weight_decay) {
  GN_REQUIRE(param && grad && exp_avg && exp_avg_sq && n >= 0 && step >= 1, "adamw_step: bad argument");
  if (n == 0) return GN_OK;
  GN_BEGIN();
  float* dp = st.out(param, (size_t)n, true); const float* dg = st.in(grad, (size_t)n);
  float* dm = st.out(exp_avg, (size_t)n, true); float* dv = st.out(exp_avg_sq, (size_t)n, true);
  if (st.status != GN_OK) return st.status;
  GN_TRY(adamw_launch(dp, dg, dm, dv, n, step, lr, beta1, beta2, eps, weight_decay, s));
  GN_END();
}

namespace {
struct Scratch {   // device workspace freed on scope exit
  void* p = nullptr;
  ~Scratch() { if (p) cudaFree(p); }
  int get(size_t bytes) { if (cudaMalloc(&p, bytes) != cudaSuccess) { set_error("optimizer: cannot allocate a %zu-byte workspace", bytes); return GN_ERR_NOMEM; } return GN_OK; }
};
}  // namespace

int gn_muon_step(float* param, float* grad, float* momentum_state, float* second_mom, int rows, int cols, float lr, float momentum, int ns_steps,
                 float beta2, float weight_decay) {
  GN_REQUIRE(param && grad && momentum_state && second_mom && rows > 0 && cols > 0, "muon_step: bad argument");
  GN_BEGIN();
  const size_t n = (size_t)rows * cols, nv = (size_t)std::max(rows, cols);
  float* dp = st.out(param, n, true); float* dg = st.out(grad, n, true);
  float* dm = st.out(momentum_state, n, true); float* dv = st.out(second_mom, nv, true);
  if (st.status != GN_OK) return st.status;
  Scratch ws; GN_TRY(ws.get(muon_workspace_bytes(rows, cols)));
  GN_TRY(muon_launch(dp, dg, dm, dv, rows, cols, lr, momentum, ns_steps, beta2, weight_decay, ws.p, gemm_default_kind(), s));
  int rc = st.finish();
  if (rc == GN_OK) rc = gemm_check_error(s);
  return rc;
}

int gn_sinkhorn_step(float* param, float* grad, float* momentum_state, int rows, int cols, float lr, float momentum, float gamma, int steps, float tau,
                     float eps) {
  GN_REQUIRE(param && grad && momentum_state && rows > 0 && cols > 0, "sinkhorn_step: bad argument");
  GN_BEGIN();
  const size_t n = (size_t)rows * cols;
  float* dp = st.out(param, n, true); float* dg = st.out(grad, n, true); float* dm = st.out(momentum_state, n, true);
  if (st.status != GN_OK) return st.status;
  Scratch ws; GN_TRY(ws.get(sinkhorn_workspace_bytes(rows, cols)));
  GN_TRY(sinkhorn_launch(dp, dg, dm, rows, cols, lr, momentum, gamma, steps, tau, eps, ws.p, s));
  GN_END();
}

int gn_softmax_last_dim(float* dst, const float* src, int64_t rows, int cols) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  GN_BEGIN();
  const float* ds = st.in(src, (size_t)rows * cols); float* dd = st.out(dst, (size_t)rows * cols);
  if (st.status != GN_OK) return st.status;
  GN_TRY(softmax_rows_launch(dd, ds, rows, cols, s));
  GN_END();
}
int gn_rmsnorm_last_dim(float* dst, const float* src, int64_t rows, int cols, float eps) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  GN_BEGIN();
  const float* ds = st.in(src, (size_t)rows * cols); float* dd = st.out(dst, (size_t)rows * cols);
  if (st.status != GN_OK) return st.status;
  GN_TRY(rmsnorm_rows_launch(dd, ds, rows, cols, eps, s));
  GN_END();
}

static int attn_shape(const gn_attention_params* p, AttnShape& sh, Stage& st, const float** q, const float** k, const float** v) {
  GN_REQUIRE(p && p->query && p->key && p->value, "attention: null argument");
  GN_REQUIRE(p->head_dim > 0 && p->head_dim <= 128, "attention: head_dim %d outside (0,128]", p->head_dim);
  GN_REQUIRE(p->query_len >= 0 && p->key_len >= 0, "attention: negative length");
  sh.B = 1; sh.Hq = 1; sh.Hkv = 1; sh.D = p->head_dim; sh.Tq = p->query_len; sh.Tk = p->key_len;
  sh.q_bstride = 0; sh.q_tstride = p->head_dim; sh.kv_bstride = 0; sh.kv_tstride = p->head_dim; sh.kv_hstride = 0;
  sh.o_bstride = 0; sh.o_tstride = p->head_dim; sh.window = p->window; sh.offset0 = p->position_offset; sh.tensor = gemm_default_kind();
  *q = st.in(p->query, (size_t)p->query_len * p->head_dim);
  *k = st.in(p->key, (size_t)p->key_len * p->head_dim);
  *v = st.in(p->value, (size_t)p->key_len * p->head_dim);
  sh.segment_ids = p->segment_ids ? st.in(p->segment_ids, (size_t)p->key_len) : nullptr;
  sh.seg_len = p->segment_ids ? p->key_len : 0;
  return st.status;
}
int gn_attention_forward(const gn_attention_params* p, float* out, float* lse) {
  GN_REQUIRE(p && out, "attention_forward: null argument");
  if (p->query_len <= 0) return GN_OK;
  GN_BEGIN();
  AttnShape sh; const float *q, *k, *v;
  GN_TRY(attn_shape(p, sh, st, &q, &k, &v));
  float* dout = st.out(out, (size_t)p->query_len * p->head_dim); float* dlse = lse ? st.out(lse, p->query_len) : nullptr;
  if (st.status != GN_OK) return st.status;
  GN_TRY(attention_forward_launch(sh, q, k, v, dout, dlse, s));
  GN_END();
}
int gn_attention_forward_split(const gn_attention_params* p, int kstart, int kend, float* acc, float* mx, float* sm) {
  GN_REQUIRE(p && acc && mx && sm, "attention_forward_split: null argument");
  if (p->query_len <= 0) return GN_OK;
  GN_BEGIN();
  AttnShape sh; const float *q, *k, *v;
  GN_TRY(attn_shape(p, sh, st, &q, &k, &v));
  float* dacc = st.out(acc, (size_t)p->query_len * p->head_dim); float* dmx = st.out(mx, p->query_len); float* dsm = st.out(sm, p->query_len);
  if (st.status != GN_OK) return st.status;
  GN_TRY(attention_split_launch(sh, q, k, v, kstart, kend, dacc, dmx, dsm, s));
  GN_END();
}
int gn_attention_combine(const float* acc, const float* mx, const float* sm, int parts, int ql, int hd, float* out, float* lse) {
  GN_REQUIRE(acc && mx && sm && out && parts > 0, "attention_combine: bad argument");
  if (ql <= 0) return GN_OK;
  GN_BEGIN();
  const float* da = st.in(acc, (size_t)parts * ql * hd); const float* dm = st.in(mx, (size_t)parts * ql); const float* ds = st.in(sm, (size_t)parts * ql);
  float* dout = st.out(out, (size_t)ql * hd); float* dlse = lse ? st.out(lse, ql) : nullptr;
  if (st.status != GN_OK) return st.status;
  GN_TRY(attention_combine_launch(da, dm, ds, parts, ql, hd, dout, dlse, s));
  GN_END();
}
int gn_attention_backward(const gn_attention_params* p, const float* output, const float* out_grad, const float* lse, const float* rowcorr,
                          float* dq, float* dk, float* dv) {
  GN_REQUIRE(p && out_grad && lse && dq && dk && dv && (output || rowcorr), "attention_backward: null argument");
  if (p->query_len <= 0) return GN_OK;
  GN_BEGIN();
  AttnShape sh; const float *q, *k, *v;
  GN_TRY(attn_shape(p, sh, st, &q, &k, &v));
  size_t nq = (size_t)p->query_len * p->head_dim, nk = (size_t)p->key_len * p->head_dim;
  const float* dout = st.in(out_grad, nq); const float* dlse = st.in(lse, p->query_len);
  const float* dO = output ? st.in(output, nq) : nullptr;
  const float* drc = rowcorr ? st.in(rowcorr, p->query_len) : nullptr;
  float* ddq = st.out(dq, nq, true); float* ddk = st.out(dk, nk, true); float* ddv = st.out(dv, nk, true);
  float* delta = nullptr;
  GN_CUDA(cudaMalloc((void**)&delta, sizeof(float) * (size_t)std::max(p->query_len, 1)));
  st.owned.push_back(delta);
  if (st.status != GN_OK) return st.status;
  GN_TRY(attention_backward_launch(sh, q, k, v, dO, dout, dlse, drc, ddq, ddk, ddv, 1, delta, s));
  GN_END();
}

// attentionForwardWindowed / attentionBackwardWindowed (model/compress_attention.go:488-541), no segment mask: the local
// sliding-window branch for every (batch, query head) over head-major tensors.  head_dim 128 runs as one batched launch on the
// tensor cores (forward tcgen05, backward mma.sync); other head dims go head by head through the float32 kernels.
static void windowed_shape(AttnShape& sh, int batch, int n_head, int n_kv_head, int seq, int head_dim, int position_offset, int window) {
  sh.B = batch; sh.Hq = n_head; sh.Hkv = n_kv_head; sh.D = head_dim; sh.Tq = seq; sh.Tk = seq;
  sh.q_bstride = (int64_t)n_head * seq * head_dim; sh.q_tstride = head_dim; sh.q_hstride = (int64_t)seq * head_dim;
  sh.kv_bstride = (int64_t)n_kv_head * seq * head_dim; sh.kv_tstride = head_dim; sh.kv_hstride = (int64_t)seq * head_dim;
  sh.o_bstride = sh.q_bstride; sh.o_tstride = head_dim; sh.o_hstride = sh.q_hstride;
  sh.window = window; sh.offset0 = position_offset; sh.tensor = gemm_default_kind();
}
static void one_head_shape(AttnShape& sh, int seq, int head_dim, int position_offset, int window) {
  sh = AttnShape();
  sh.D = head_dim; sh.Tq = seq; sh.Tk = seq; sh.q_tstride = head_dim; sh.kv_tstride = head_dim; sh.o_tstride = head_dim;
  sh.window = window; sh.offset0 = position_offset; sh.tensor = gemm_default_kind();
}
int gn_attention_windowed_forward(const float* query, const float* key, const float* value, int batch, int n_head, int n_kv_head, int seq, int head_dim,
                                  int position_offset, int window, float* out, float* lse) {
  if (batch <= 0 || seq <= 0) return GN_OK;
  GN_REQUIRE(query && key && value && out && n_kv_head > 0 && n_head % n_kv_head == 0 && head_dim > 0 && head_dim <= 128 && position_offset >= 0,
             "attention_windowed_forward: bad argument");
  GN_BEGIN();
  const size_t hd = (size_t)seq * head_dim, nq = (size_t)batch * n_head * hd, nk = (size_t)batch * n_kv_head * hd;
  const float* pq = st.in(query, nq); const float* pk = st.in(key, nk); const float* pv = st.in(value, nk);
  float* po = st.out(out, nq); float* pl = lse ? st.out(lse, (size_t)batch * n_head * seq) : nullptr;
  if (st.status != GN_OK) return st.status;
  AttnShape sh; windowed_shape(sh, batch, n_head, n_kv_head, seq, head_dim, position_offset, window);
#ifdef GN_HAVE_TCGEN05
  if (sh.tensor && attention_tc_ok(sh, pq, pk, pv, po)) { GN_TRY(attention_tc_forward(sh, pq, pk, pv, po, pl, s)); GN_END(); }
#endif
  AttnShape one; one_head_shape(one, seq, head_dim, position_offset, window);
  const int hr = n_head / n_kv_head;
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < n_head; ++h) {
      const size_t qi = (size_t)b * n_head + h, ki = (size_t)b * n_kv_head + h / hr;
      GN_TRY(attention_forward_launch(one, pq + qi * hd, pk + ki * hd, pv + ki * hd, po + qi * hd, pl ? pl + qi * seq : nullptr, s));
    }
  GN_END();
}
__global__ void __launch_bounds__(256) row_dot_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t rows, int width, float* __restrict__ dst) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * 8 + warp;
  if (r >= rows) return;
  float acc = 0.0f;
  for (int c = lane; c < width; c += 32) acc = fmaf(a[r * width + c], b[r * width + c], acc);
  acc = warp_sum(acc);
  if (lane == 0) dst[r] = acc;
}
int gn_attention_windowed_backward(const float* query, const float* key, const float* value, const float* output, const float* out_grad, const float* lse,
                                   const float* row_correction, int batch, int n_head, int n_kv_head, int seq, int head_dim, int position_offset, int window,
                                   float* dq, float* dk, float* dv) {
  if (batch <= 0 || seq <= 0) return GN_OK;
  GN_REQUIRE(query && key && value && out_grad && lse && dq && dk && dv && (output || row_correction) && n_kv_head > 0 && n_head % n_kv_head == 0 &&
             head_dim > 0 && head_dim <= 128 && position_offset >= 0, "attention_windowed_backward: bad argument");
  GN_BEGIN();
  const size_t hd = (size_t)seq * head_dim, nq = (size_t)batch * n_head * hd, nk = (size_t)batch * n_kv_head * hd, nt = (size_t)batch * n_head * seq;
  const float* pq = st.in(query, nq); const float* pk = st.in(key, nk); const float* pv = st.in(value, nk);
  const float* po = output ? st.in(output, nq) : nullptr; const float* pg = st.in(out_grad, nq); const float* pl = st.in(lse, nt);
  const float* pr = row_correction ? st.in(row_correction, nt) : nullptr;
  float* gq = st.out(dq, nq, true); float* gk = st.out(dk, nk, true); float* gv = st.out(dv, nk, true);
  float* delta = st.temp<float>(nt);
  if (st.status != GN_OK) return st.status;
  AttnShape sh; windowed_shape(sh, batch, n_head, n_kv_head, seq, head_dim, position_offset, window);
  if (sh.tensor && attention_mma_ok(sh, pq, pk, pv, pg, gq) && (reinterpret_cast<uintptr_t>(gk) & 15) == 0 && (reinterpret_cast<uintptr_t>(gv) & 15) == 0) {
    const float* dl = pr;
    if (!dl) { row_dot_kernel<<<(unsigned)ceil_div((int64_t)nt, 8), 256, 0, s>>>(pg, po, (int64_t)nt, head_dim, delta); GN_LAUNCH_CHECK(); dl = delta; }
    GN_TRY(attention_mma_backward(sh, pq, pk, pv, pg, pl, dl, gq, gk, gv, 1, s));
    GN_END();
  }
  AttnShape one; one_head_shape(one, seq, head_dim, position_offset, window);
  const int hr = n_head / n_kv_head;
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < n_head; ++h) {
      const size_t qi = (size_t)b * n_head + h, ki = (size_t)b * n_kv_head + h / hr;
      GN_TRY(attention_backward_launch(one, pq + qi * hd, pk + ki * hd, pv + ki * hd, po ? po + qi * hd : nullptr, pg + qi * hd, pl + qi * seq,
                                       pr ? pr + qi * seq : nullptr, gq + qi * hd, gk + ki * hd, gv + ki * hd, 1, delta + qi * seq, s));
    }
  GN_END();
}

int gn_sample_next_token(const float* logits, int rows, int vocab, const float* uniforms, const uint64_t* seeds, int group, uint32_t step,
                         float temperature, int top_k, int32_t* out) {
  GN_REQUIRE(logits && out, "sample_next_token: null argument");
  if (rows <= 0) return GN_OK;
  if (group < 1) group = 1;
  GN_BEGIN();
  const float* dl = st.in(logits, (size_t)rows * vocab); const float* du = uniforms ? st.in(uniforms, (size_t)rows * vocab) : nullptr;
  const uint64_t* dsd = seeds ? st.in(seeds, (size_t)((rows + group - 1) / group)) : nullptr;
  int32_t* dd = st.out(out, rows);
  if (st.status != GN_OK) return st.status;
  GN_TRY(sample_launch(dl, rows, vocab, 1, du, dsd, group, nullptr, step, temperature, top_k, dd, s));
  GN_END();
}
int gn_group_advantage(const float* rewards, int groups, int group, int mode, float* adv) {
  GN_REQUIRE(rewards && adv && group > 0, "group_advantage: bad argument");
  if (groups <= 0) return GN_OK;
  GN_BEGIN();
  const float* dr = st.in(rewards, (size_t)groups * group); float* da = st.out(adv, (size_t)groups * group);
  if (st.status != GN_OK) return st.status;
  GN_TRY(advantage_launch(dr, groups, group, mode, da, s));
  GN_END();
}
int gn_pg_loss_backward(const float* logits, const int32_t* targets, const float* adv, int64_t rows, int vocab, int seq_len, float norm, float softcap,
                        float* nll, float* dlogits, double* loss) {
  GN_REQUIRE(logits && targets && adv && loss && vocab > 0 && seq_len > 0 && rows >= 0, "pg_loss_backward: bad argument");
  GN_BEGIN();
  size_t n = (size_t)rows * vocab;
  const bool in_place = dlogits == logits;
  const float* dl; float* dd = nullptr;
  if (in_place) { dd = st.out(dlogits, n, true); dl = dd; }
  else { dl = st.in(logits, n); dd = dlogits ? st.out(dlogits, n) : nullptr; }
  const int32_t* dt = st.in(targets, rows); const float* da = st.in(adv, (size_t)((rows + seq_len - 1) / seq_len));
  float* dn = nll ? st.out(nll, rows) : nullptr;
  // scratch: cell 0 the loss total, cell 1 the count of out-of-range targets, cells 2.. one term per row
  double* scratch = nullptr;
  GN_CUDA(cudaMalloc((void**)&scratch, sizeof(double) * (size_t)(rows + 2)));
  st.owned.push_back(scratch);
  if (st.status != GN_OK) return st.status;
  GN_CUDA(cudaMemsetAsync(scratch, 0, 2 * sizeof(double), s));
  GN_TRY(pg_loss_launch(dl, dt, da, rows, vocab, vocab, seq_len, norm, softcap, dn, dd, vocab, scratch + 2, scratch, 0, s, reinterpret_cast<int*>(scratch + 1)));
  int bad = 0;
  GN_CUDA(cudaMemcpyAsync(&bad, scratch + 1, sizeof(int), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaMemcpyAsync(loss, scratch, sizeof(double), cudaMemcpyDefault, s));   // loss may be host or device memory
  GN_CUDA(cudaStreamSynchronize(s));
  if (bad) { set_error("pg_loss_backward: %d targets outside {-1} and [0, %d)", bad, vocab); return GN_ERR_INVALID; }
  GN_END();
}

// tensors.DistillationLossPerPosition + DistillationGrad (tensors/loss.go:84-213)
int gn_distillation_loss_backward(const float* student, const float* teacher, const int32_t* mask, int64_t rows, int vocab, float temperature, float scale,
                                  float* losses, float* dstudent, double* loss_sum, int64_t* valid) {
  GN_REQUIRE(student && teacher && vocab > 0 && rows >= 0, "distillation_loss_backward: bad argument");
  GN_BEGIN();
  const size_t n = (size_t)rows * vocab;
  const float* ds = st.in(student, n); const float* dt = st.in(teacher, n);
  const int32_t* dm = mask ? st.in(mask, rows) : nullptr;
  float* dl = losses ? st.out(losses, rows) : nullptr; float* dg = dstudent ? st.out(dstudent, n) : nullptr;
  double* scratch = nullptr;
  GN_CUDA(cudaMalloc((void**)&scratch, sizeof(double) * (size_t)(rows + 1)));
  st.owned.push_back(scratch);
  if (st.status != GN_OK) return st.status;
  GN_TRY(distillation_launch(ds, dt, dm, rows, vocab, temperature, scale, dl, dg, scratch + 1, scratch, s));
  if (loss_sum) GN_CUDA(cudaMemcpyAsync(loss_sum, scratch, sizeof(double), cudaMemcpyDefault, s));
  if (valid) {   // the mask is small: count it on the host side of the call
    int64_t count = rows;
    if (mask) {
      std::vector<int32_t> hm((size_t)rows);
      GN_CUDA(cudaMemcpyAsync(hm.data(), dm, sizeof(int32_t) * rows, cudaMemcpyDeviceToHost, s));
      GN_CUDA(cudaStreamSynchronize(s));
      count = 0; for (int32_t v : hm) count += v != 0;
    }
    *valid = count;
  }
  GN_END();
}

}  // extern "C"
