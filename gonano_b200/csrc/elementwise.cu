// Elementwise, reduction and per-row kernels of the backend contract
// (kernels/backend.go:21-78,145-153) plus the RMSNorm backward
// (tensors/backward.go:81-104).  All HBM-bound: float4 accesses where the
// pointers allow it, grids sized in multiples of the SM count.
#include "kernels.cuh"

namespace gn {

__device__ __forceinline__ float ew_apply(int op, float a, float b, float f) {
  switch (op) {
    case EW_ADD: return a + b;
    case EW_SUB: return a - b;
    case EW_MUL: return a * b;
    case EW_DIV: return a / b;
    case EW_SCALE: return a * f;
    case EW_ADD_SCALED: return a + f * b;
    case EW_NEG: return -a;
    case EW_ABS: return fabsf(a);
    case EW_SQUARE: return a * a;
    case EW_RELU2: { float v = a < 0.0f ? 0.0f : a; return v * v; }
    case EW_EXP: return (float)exp((double)a);
    case EW_SIGMOID: return (float)(1.0 / (1.0 + exp((double)(-a))));
    case EW_TANH: return (float)tanh((double)a);
    case EW_RSQRT: return (float)(1.0 / sqrt((double)a));
    case EW_SWIGLU: {
      // kernels/scalar/elementwise.go:105-134: gate clamped above, up clamped both sides.
      float g = (f > 0.0f && a >= f) ? f : a;
      float u = b;
      if (f > 0.0f) { if (u > f) u = f; else if (u < -f) u = -f; }
      float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
      return g * sg * u;
    }
  }
  return 0.0f;
}

template <int OP>
__global__ void __launch_bounds__(256) ew_kernel(float* __restrict__ dst, const float* a, const float* b, float f, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float av = a[i];
    float bv = b ? b[i] : 0.0f;
    dst[i] = ew_apply(OP, av, bv, f);
  }
}

template <int OP>
static int ew_go(float* dst, const float* a, const float* b, float f, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 16);
  ew_kernel<OP><<<blocks, 256, 0, s>>>(dst, a, b, f, n);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int ew_launch(int op, float* dst, const float* a, const float* b, float f, int64_t n, cudaStream_t s) {
  switch (op) {
    case EW_ADD: return ew_go<EW_ADD>(dst, a, b, f, n, s);
    case EW_SUB: return ew_go<EW_SUB>(dst, a, b, f, n, s);
    case EW_MUL: return ew_go<EW_MUL>(dst, a, b, f, n, s);
    case EW_DIV: return ew_go<EW_DIV>(dst, a, b, f, n, s);
    case EW_SCALE: return ew_go<EW_SCALE>(dst, a, b, f, n, s);
    case EW_ADD_SCALED: return ew_go<EW_ADD_SCALED>(dst, a, b, f, n, s);
    case EW_NEG: return ew_go<EW_NEG>(dst, a, b, f, n, s);
    case EW_ABS: return ew_go<EW_ABS>(dst, a, b, f, n, s);
    case EW_SQUARE: return ew_go<EW_SQUARE>(dst, a, b, f, n, s);
    case EW_RELU2: return ew_go<EW_RELU2>(dst, a, b, f, n, s);
    case EW_EXP: return ew_go<EW_EXP>(dst, a, b, f, n, s);
    case EW_SIGMOID: return ew_go<EW_SIGMOID>(dst, a, b, f, n, s);
    case EW_TANH: return ew_go<EW_TANH>(dst, a, b, f, n, s);
    case EW_RSQRT: return ew_go<EW_RSQRT>(dst, a, b, f, n, s);
    case EW_SWIGLU: return ew_go<EW_SWIGLU>(dst, a, b, f, n, s);
  }
  set_error("unknown elementwise op %d", op);
  return GN_ERR_INVALID;
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(float* gg, float* ug, const float* gate, const float* up, const float* og, float c, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    // kernels/scalar/elementwise.go:94-103
    float g = gate[i], u = up[i], d = og[i];
    float gm = 1.0f, um = 1.0f;
    if (c > 0.0f && g >= c) { g = c; gm = 0.0f; }
    if (c > 0.0f) { if (u > c) { u = c; um = 0.0f; } else if (u < -c) { u = -c; um = 0.0f; } }
    float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
    float silu = g * sg;
    float sgrad = sg * (1.0f + g * (1.0f - sg));
    gg[i] = d * u * sgrad * gm;
    ug[i] = d * silu * um;
  }
}
int swiglu_backward_launch(float* gg, float* ug, const float* gate, const float* up, const float* og, float clamp, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 16);
  swiglu_bwd_kernel<<<blocks, 256, 0, s>>>(gg, ug, gate, up, og, clamp, n);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// hi/lo tf32 split of a pitched matrix (the form the tensor-core products read), for producers that ran on the float32 path
__global__ void __launch_bounds__(256) split_matrix_kernel(const float* src, float* hi, float* lo, int64_t rows, int cols, int64_t ld) {
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols; const int c = (int)(i % cols);
    float h, l; split_tf32(src[r * ld + c], h, l);
    hi[r * ld + c] = h; lo[r * ld + c] = l;
  }
}
int split_matrix_launch(const float* src, float* hi, float* lo, int64_t rows, int cols, int64_t ld, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  const int blocks = (int)std::min<int64_t>((rows * cols + 255) / 256, (int64_t)num_sms() * 16);
  split_matrix_kernel<<<blocks, 256, 0, s>>>(src, hi, lo, rows, cols, ld);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(256) fill_kernel(float* dst, float v, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = v;
}
int fill_launch(float* dst, float value, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 16);
  fill_kernel<<<blocks, 256, 0, s>>>(dst, value, n);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ------------------------------------------------------------------ reductions
// Single-block reductions: these entry points exist for conformance with the
// contract; the RL step never reduces to a host scalar on its hot path.
__global__ void __launch_bounds__(1024) sum_kernel(const float* v, int64_t n, float* out) {
  __shared__ double sh[32];
  double acc = 0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) acc += (double)v[i];
  acc = block_sum_d(acc, sh);
  if (threadIdx.x == 0) *out = (float)acc;
}
__global__ void __launch_bounds__(1024) dot_kernel(const float* a, const float* b, int64_t n, float* out) {
  __shared__ double sh[32];
  double acc = 0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) acc += (double)a[i] * (double)b[i];
  acc = block_sum_d(acc, sh);
  if (threadIdx.x == 0) *out = (float)acc;
}
__global__ void __launch_bounds__(1024) max_kernel(const float* v, int64_t n, float* out) {
  __shared__ float sh[32];
  float m = -INFINITY;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, v[i]);
  m = block_max(m, sh);
  if (threadIdx.x == 0) *out = (n == 0) ? 0.0f : m;
}
__global__ void __launch_bounds__(1024) argmax_kernel(const float* v, int64_t n, int64_t* out) {
  __shared__ float shv[32];
  __shared__ long long shi[32];
  float best = -INFINITY; long long bi = 0x7fffffffffffffffLL;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float x = v[i];
    if (x > best || (x == best && (long long)i < bi)) { best = x; bi = i; }
  }
  // first maximum wins (kernels/scalar/reduce.go:26-36): larger value, then smaller index
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { shv[warp] = best; shi[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? shv[lane] : -INFINITY; bi = lane < nw ? shi[lane] : 0x7fffffffffffffffLL;
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) *out = (n == 0 || bi == 0x7fffffffffffffffLL) ? 0 : bi;
  }
}
int reduce_sum_launch(const float* v, int64_t n, float* out, cudaStream_t s) { sum_kernel<<<1, 1024, 0, s>>>(v, n, out); GN_LAUNCH_CHECK(); return GN_OK; }
int reduce_max_launch(const float* v, int64_t n, float* out, cudaStream_t s) { max_kernel<<<1, 1024, 0, s>>>(v, n, out); GN_LAUNCH_CHECK(); return GN_OK; }
int reduce_argmax_launch(const float* v, int64_t n, int64_t* out, cudaStream_t s) { argmax_kernel<<<1, 1024, 0, s>>>(v, n, out); GN_LAUNCH_CHECK(); return GN_OK; }
int dot_launch(const float* a, const float* b, int64_t n, float* out, cudaStream_t s) { dot_kernel<<<1, 1024, 0, s>>>(a, b, n, out); GN_LAUNCH_CHECK(); return GN_OK; }

// ------------------------------------------------------------------------ rows
// One warp per row for narrow rows, one block per row for wide ones.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) softmax_rows_kernel(float* dst, const float* src, int64_t rows, int cols) {
  __shared__ float sh[32];
  int64_t row = blockIdx.x;
  const float* s = src + row * cols;
  float* d = dst + row * cols;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += THREADS) m = fmaxf(m, s[c]);
  m = block_max(m, sh);
  float sum = 0;
  for (int c = threadIdx.x; c < cols; c += THREADS) sum += expf(s[c] - m);
  sum = block_sum(sum, sh);
  float inv = 1.0f / sum;
  for (int c = threadIdx.x; c < cols; c += THREADS) d[c] = expf(s[c] - m) * inv;
}
int softmax_rows_launch(float* dst, const float* src, int64_t rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  if (cols <= 256) softmax_rows_kernel<32><<<(unsigned)rows, 32, 0, s>>>(dst, src, rows, cols);
  else softmax_rows_kernel<256><<<(unsigned)rows, 256, 0, s>>>(dst, src, rows, cols);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// kernels/scalar/norm.go:26-40: mean square, cast to f32, 1/sqrt(ms + eps).
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(float* dst, const float* src, int64_t rows, int cols, float eps) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const float* s = src + row * cols;
  float* d = dst + row * cols;
  float ss = 0;
  for (int c = lane; c < cols; c += 32) { float x = s[c]; ss = fmaf(x, x, ss); }
  ss = warp_sum(ss);
  float ms = ss / (float)cols;
  float inv = (float)(1.0 / sqrt((double)ms + (double)eps));
  for (int c = lane; c < cols; c += 32) d[c] = s[c] * inv;
}
int rmsnorm_rows_launch(float* dst, const float* src, int64_t rows, int cols, float eps, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  int blocks = ceil_div(rows, 8);
  rmsnorm_rows_kernel<<<blocks, 256, 0, s>>>(dst, src, rows, cols, eps);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(float* dx, const float* x, const float* dy, const float* add, int64_t rows, int cols, float eps) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const float* xr = x + row * cols; const float* gr = dy + row * cols; float* o = dx + row * cols;
  const float* ar = add ? add + row * cols : nullptr;
  float ss = 0, dp = 0;
  for (int c = lane; c < cols; c += 32) { float xv = xr[c]; ss = fmaf(xv, xv, ss); dp = fmaf(gr[c], xv, dp); }
  ss = warp_sum(ss); dp = warp_sum(dp);
  double ms = (double)ss / (double)cols;
  double rms = sqrt(ms + (double)eps);
  float inv = (float)(1.0 / rms);
  float coef = (float)((double)dp / ((double)cols * rms * rms * rms));
  for (int c = lane; c < cols; c += 32) {
    float v = gr[c] * inv - coef * xr[c];
    o[c] = ar ? ar[c] + v : v;
  }
}
int rmsnorm_backward_launch(float* dx, const float* x, const float* dy, const float* add, int64_t rows, int cols, float eps, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return GN_OK;
  int blocks = ceil_div(rows, 8);
  rmsnorm_bwd_kernel<<<blocks, 256, 0, s>>>(dx, x, dy, add, rows, cols, eps);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
