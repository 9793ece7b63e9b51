// The optimizer step of the RL step (trainer/rl.go:62-67: optimizer.Step then ZeroGrad), on the device:
//   AdamW     optimizer/optimizer.go:143-173   scalar groups (a few dozen floats)
//   Muon      optimizer/muon.go:23-173         every block matrix: Nesterov momentum, row equilibration,
//                                              5 Polar-Express iterations (three products each, on the GEMM path),
//                                              Muon+ renormalisation, NorMuon variance reduction, cautious decay
//   Sinkhorn  optimizer/sinkhorn.go:27-95      lm_head, wte, value embeddings: Nesterov momentum, near-zero row
//                                              mask, 11 alternating row / column L2 normalisations, unit-RMS update
// and the routing chat_rl uses (model/optimizer.go:20-165 with sinkhorn = true, cmd/chat_rl/main.go:68-72).
//
// The update matrix is built in place in the gradient buffer (the step ends with ZeroGrad anyway).  Sums that the
// reference takes in float64 are taken in float64 here too, by fixed-shape block reductions (deterministic; the
// order differs from the reference's sequential loops at the 1e-16 level).  Scalars that steer later kernels
// (norms, thresholds) stay in device memory: the step never synchronises with the host.
// The Sinkhorn passes are HBM-bound: 1 + 5 x (column sums read, row step read + write) over the matrix.
#include <algorithm>
#include <cmath>

#include "model_internal.cuh"

namespace gn {

namespace {

constexpr int RT = 256;   // threads of the one-block-per-row kernels

// ------------------------------------------------------------------ AdamW
__global__ void adamw_kernel(float* p, const float* g, float* m, float* v, int64_t n, double b1, double b2, double eps, double decay, double step_size,
                             double bias2) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float pv = p[i] * (float)decay;
  const double gi = (double)g[i];
  const float mi = (float)(b1 * (double)m[i] + (1 - b1) * gi);
  const float vi = (float)(b2 * (double)v[i] + (1 - b2) * gi * gi);
  m[i] = mi; v[i] = vi;
  const double denom = sqrt((double)vi / bias2) + eps;
  pv -= (float)(step_size * (double)mi / denom);
  p[i] = pv;
}

// ------------------------------------------------------------------ shared small kernels
// out[0] = sum of v[0..n) in float64 (one block, fixed order); when root != 0 the square root of it.
__global__ void __launch_bounds__(1024) sum_d_kernel(const double* v, int64_t n, double* out, int root, int root_each) {
  __shared__ double scratch[33];
  double s = 0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += root_each ? sqrt(v[i]) : v[i];
  s = block_sum_d(s, scratch);
  if (threadIdx.x == 0) out[0] = root ? sqrt(s) : s;
}
// x *= (float) f(scal)   kinds: 0 = 1 / (norm * 1.01 + 1e-6)   (optimizer/muon.go:57-61)
//                               1 = sqrt(min_dim) / max(norm, 1e-6), also leaves per-row sums of squares of the result
__global__ void __launch_bounds__(RT) scale_rows_kernel(float* x, int cols, const double* scal, int kind, float target, double* rowss) {
  __shared__ double scratch[33];
  const int64_t r = blockIdx.x;
  const float norm = (float)scal[0];
  float sc;
  if (kind == 0) sc = (float)(1.0 / ((double)norm * 1.01 + 1e-6));
  else { float cur = norm < 1e-6f ? 1e-6f : norm; sc = target / cur; }
  double ss = 0;
  for (int c = threadIdx.x; c < cols; c += RT) { const float v = x[r * cols + c] * sc; x[r * cols + c] = v; ss += (double)v * (double)v; }
  if (rowss) { ss = block_sum_d(ss, scratch); if (threadIdx.x == 0) rowss[r] = ss; }
}

// rowss[r] = sum of squares of row r (float64)
__global__ void __launch_bounds__(RT) rowss_kernel(const float* x, int cols, double* rowss) {
  __shared__ double scratch[33];
  const int64_t r = blockIdx.x;
  double ss = 0;
  for (int c = threadIdx.x; c < cols; c += RT) { const double v = x[r * cols + c]; ss += v * v; }
  ss = block_sum_d(ss, scratch);
  if (threadIdx.x == 0) rowss[r] = ss;
}

// ------------------------------------------------------------------ Muon
// mom = momentum*mom + (1-momentum)*g ; u = (1-momentum)*g + momentum*mom (float32, u overwrites g); rowss[r] = sum u^2
__global__ void __launch_bounds__(RT) muon_momentum_kernel(float* g, float* mom, int cols, float momentum, double* rowss) {
  __shared__ double scratch[33];
  const int64_t r = blockIdx.x;
  const float om = 1.0f - momentum;
  double ss = 0;
  for (int c = threadIdx.x; c < cols; c += RT) {
    const int64_t i = r * cols + c;
    const float gi = g[i];
    const float mi = __fadd_rn(__fmul_rn(momentum, mom[i]), __fmul_rn(om, gi));
    mom[i] = mi;
    const float u = __fadd_rn(__fmul_rn(om, gi), __fmul_rn(momentum, mi));
    g[i] = u; ss += (double)u * (double)u;
  }
  ss = block_sum_d(ss, scratch);
  if (threadIdx.x == 0) rowss[r] = ss;
}
// row equilibration (optimizer/muon.go:43-54): scal[0] = Frobenius norm; leaves the new row sums of squares
__global__ void __launch_bounds__(RT) muon_equilibrate_kernel(float* u, int rows, int cols, const double* scal, double* rowss) {
  __shared__ double scratch[33];
  const int64_t r = blockIdx.x;
  const float target = (float)scal[0] / (float)sqrt((double)rows);
  float rn = (float)sqrt(rowss[r]);
  if (rn < 1e-6f) rn = 1e-6f;
  const float sc = target / rn;
  double ss = 0;
  for (int c = threadIdx.x; c < cols; c += RT) { const float v = u[r * cols + c] * sc; u[r * cols + c] = v; ss += (double)v * (double)v; }
  ss = block_sum_d(ss, scratch);
  if (threadIdx.x == 0) rowss[r] = ss;
}
// poly = gram*b + gram2*c
__global__ void poly_kernel(float* poly, const float* gram, const float* gram2, int64_t n, float b, float c) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) poly[i] = __fadd_rn(__fmul_rn(gram[i], b), __fmul_rn(gram2[i], c));
}
// u = u*a + prod
__global__ void axpby_kernel(float* u, const float* prod, int64_t n, float a) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) u[i] = __fadd_rn(__fmul_rn(u[i], a), prod[i]);
}
// column sums of squares in float64: thread = column, rows walked in order
__global__ void colss_kernel(const float* u, int rows, int cols, double* colss) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  double s = 0;
  for (int r = 0; r < rows; ++r) { const double v = u[(int64_t)r * cols + c]; s += v * v; }
  colss[c] = s;
}
// NorMuon variance reduction (optimizer/muon.go:88-149), one block: ss[i] = sum of squares of row / column i of the
// renormalised update; updates second_mom and writes the final per-row / per-column scale.
__global__ void __launch_bounds__(1024) muon_variance_kernel(const double* ss, int nv, int reduce, float beta2, float* second_mom, float* fin) {
  __shared__ double scratch[33];
  double a = 0, b = 0;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const float vm = (float)(ss[i] / (double)reduce);
    a += (double)vm;
    const float smn = __fadd_rn(__fmul_rn(beta2, second_mom[i]), __fmul_rn(1.0f - beta2, vm));
    second_mom[i] = smn;
    const float smc = smn < 1e-10f ? 1e-10f : smn;
    const float st = (float)(1.0 / sqrt((double)smc));
    fin[i] = st;
    b += (double)vm * (double)reduce * (double)st * (double)st;
  }
  a = block_sum_d(a, scratch);
  b = block_sum_d(b, scratch);
  const float vnorm = (float)sqrt(a * (double)reduce);
  float nvn = (float)sqrt(b);
  if (nvn < 1e-10f) nvn = 1e-10f;
  const float ratio = vnorm / nvn;
  __syncthreads();
  for (int i = threadIdx.x; i < nv; i += blockDim.x) fin[i] = fin[i] * ratio;
}
// u *= fin[row or col]; cautious weight decay; parameter update (optimizer/muon.go:151-173)
__global__ void muon_apply_kernel(float* p, const float* u, const float* fin, int rows, int cols, int per_row, float lr, float wd) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)rows * cols) return;
  const float uv = u[i] * fin[per_row ? i / cols : i % cols];
  const float pv = p[i];
  const float mask = (uv * pv >= 0.0f) ? 1.0f : 0.0f;
  p[i] = pv - __fadd_rn(__fmul_rn(lr, uv), __fmul_rn(__fmul_rn(__fmul_rn(lr, wd), pv), mask));
}

// ------------------------------------------------------------------ Sinkhorn
// momentum and Nesterov update in float64 (optimizer/sinkhorn.go:35-40); u overwrites g; rowss[r] = sum u^2
__global__ void __launch_bounds__(RT) sk_momentum_kernel(float* g, float* mom, int cols, double beta, double* rowss) {
  __shared__ double scratch[33];
  const int64_t r = blockIdx.x;
  double ss = 0;
  for (int c = threadIdx.x; c < cols; c += RT) {
    const int64_t i = r * cols + c;
    const double gi = (double)g[i];
    const double mv = beta * (double)mom[i] + (1 - beta) * gi;
    mom[i] = (float)mv;
    const float u = (float)(beta * mv + (1 - beta) * gi);
    g[i] = u; ss += (double)u * (double)u;
  }
  ss = block_sum_d(ss, scratch);
  if (threadIdx.x == 0) rowss[r] = ss;
}
// One row normalisation (odd steps).  first: rows whose norm is <= tau * mean row norm are zeroed before it
// (scal[0] = sum of the row norms).  colscale: the pending column normalisation of the previous even step is
// applied on the way in.  last: the parameter update replaces the store (optimizer/sinkhorn.go:88-94).
__global__ void __launch_bounds__(RT) sk_row_step_kernel(float* u, float* p, int rows, int cols, const double* rowss, const double* scal, double tau,
                                                         const double* colscale, double eps, int first, int last, double lrf) {
  __shared__ double scratch[33];
  const int64_t r = blockIdx.x;
  bool zero = false;
  if (first) { const double thr = tau * scal[0] / (double)rows; zero = sqrt(rowss[r]) <= thr; }
  double ss = 0;
  for (int c = threadIdx.x; c < cols; c += RT) {
    float v = zero ? 0.0f : u[r * cols + c];
    if (colscale) v = (float)((double)v * colscale[c]);
    ss += (double)v * (double)v;
  }
  ss = block_sum_d(ss, scratch);
  const double sc = 1.0 / (sqrt(ss) + eps);
  for (int c = threadIdx.x; c < cols; c += RT) {
    float v = zero ? 0.0f : u[r * cols + c];
    if (colscale) v = (float)((double)v * colscale[c]);
    const float o = (float)((double)v * sc);
    if (last) p[r * cols + c] -= (float)(lrf * (double)o);
    else u[r * cols + c] = o;
  }
}
// column sums of squares in two fixed-order levels: partial[chunk][col] over a chunk of rows, then over the chunks
__global__ void __launch_bounds__(128) sk_colss_partial_kernel(const float* u, int rows, int cols, int chunk_rows, double* partial) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= cols) return;
  const int r0 = blockIdx.y * chunk_rows, r1 = min(rows, r0 + chunk_rows);
  double s = 0;
  for (int r = r0; r < r1; ++r) { const double v = u[(int64_t)r * cols + c]; s += v * v; }
  partial[(int64_t)blockIdx.y * cols + c] = s;
}
__global__ void sk_colscale_kernel(const double* partial, int chunks, int cols, double eps, double* colscale) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  double s = 0;
  for (int k = 0; k < chunks; ++k) s += partial[(int64_t)k * cols + c];
  colscale[c] = 1.0 / (sqrt(s) + eps);
}

int blocks_for(int64_t n) { return (int)((n + 255) / 256); }

}  // namespace

// Device workspace one update needs (doubles first, then floats).
size_t muon_workspace_bytes(int rows, int cols) {
  const size_t g = (size_t)std::min(rows, cols);
  return sizeof(double) * (16 + (size_t)rows + cols) + 256 + sizeof(float) * (3 * g * g + (size_t)rows * cols + (size_t)std::max(rows, cols));
}
size_t sinkhorn_workspace_bytes(int rows, int cols) { return sizeof(double) * (16 + (size_t)rows + cols + (size_t)128 * cols); }

int adamw_launch(float* p, const float* g, float* m, float* v, int64_t n, int step, float lr, float beta1, float beta2, float eps, float wd, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  const double b1 = beta1, b2 = beta2, l = lr;
  const double bias1 = 1 - std::pow(b1, (double)step), bias2 = 1 - std::pow(b2, (double)step);
  adamw_kernel<<<blocks_for(n), 256, 0, s>>>(p, g, m, v, n, b1, b2, (double)eps, 1 - l * (double)wd, l / bias1, bias2);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int muon_launch(float* p, float* g, float* mom, float* second, int rows, int cols, float lr, float momentum, int ns_steps, float beta2, float wd,
                void* workspace, int gemm_kind, cudaStream_t s) {
  GN_REQUIRE(rows > 0 && cols > 0 && ns_steps >= 0 && ns_steps <= 5, "muon: bad shape or step count");
  const int64_t n = (int64_t)rows * cols;
  const bool tall = rows > cols;
  const int gd = tall ? cols : rows;
  double* scal = (double*)workspace;                 // [16]
  double* rowss = scal + 16;                          // [rows]
  double* colss = rowss + rows;                       // [cols]
  float* gram = (float*)(colss + cols);
  gram = (float*)(((uintptr_t)gram + 255) & ~(uintptr_t)255);
  float* gram2 = gram + (size_t)gd * gd; float* poly = gram2 + (size_t)gd * gd; float* prod = poly + (size_t)gd * gd;
  float* fin = prod + n;
  float* u = g;
  muon_momentum_kernel<<<rows, RT, 0, s>>>(u, mom, cols, momentum, rowss); GN_LAUNCH_CHECK();
  sum_d_kernel<<<1, 1024, 0, s>>>(rowss, rows, scal, 1, 0); GN_LAUNCH_CHECK();
  muon_equilibrate_kernel<<<rows, RT, 0, s>>>(u, rows, cols, scal, rowss); GN_LAUNCH_CHECK();
  sum_d_kernel<<<1, 1024, 0, s>>>(rowss, rows, scal, 1, 0); GN_LAUNCH_CHECK();
  scale_rows_kernel<<<rows, RT, 0, s>>>(u, cols, scal, 0, 0.0f, nullptr); GN_LAUNCH_CHECK();
  static const double coeff[5][3] = {
      {8.156554524902461, -22.48329292557795, 15.878769915207462}, {4.042929935166739, -2.808917465908714, 0.5000178451051316},
      {3.8916678022926607, -2.772484153217685, 0.5060648178503393}, {3.285753657755655, -2.3681294933425376, 0.46449024233003106},
      {2.3465413258596377, -1.7097828382687081, 0.42323551169305323}};   // optimizer/muon.go:11-17
  for (int st = 0; st < ns_steps; ++st) {
    const float a = (float)coeff[st][0], b = (float)coeff[st][1], c = (float)coeff[st][2];
    { GemmArgs ga; ga.C = gram; ga.ldc = gd; ga.M = gd; ga.N = gd;
      if (tall) { ga.A = u; ga.lda = cols; ga.a_trans = 1; ga.B = u; ga.ldb = cols; ga.b_trans = 0; ga.K = rows; }       // U^T U
      else { ga.A = u; ga.lda = cols; ga.a_trans = 0; ga.B = u; ga.ldb = cols; ga.b_trans = 1; ga.K = cols; }            // U U^T
      GN_TRY(gemm_dispatch(ga, gemm_kind, s)); }
    { GemmArgs ga; ga.A = gram; ga.lda = gd; ga.B = gram; ga.ldb = gd; ga.b_trans = 0; ga.C = gram2; ga.ldc = gd; ga.M = gd; ga.N = gd; ga.K = gd;
      GN_TRY(gemm_dispatch(ga, gemm_kind, s)); }
    poly_kernel<<<blocks_for((int64_t)gd * gd), 256, 0, s>>>(poly, gram, gram2, (int64_t)gd * gd, b, c); GN_LAUNCH_CHECK();
    { GemmArgs ga; ga.C = prod; ga.ldc = cols; ga.M = rows; ga.N = cols;
      if (tall) { ga.A = u; ga.lda = cols; ga.B = poly; ga.ldb = gd; ga.b_trans = 0; ga.K = cols; }                     // U poly
      else { ga.A = poly; ga.lda = gd; ga.B = u; ga.ldb = cols; ga.b_trans = 0; ga.K = rows; }                          // poly U
      GN_TRY(gemm_dispatch(ga, gemm_kind, s)); }
    axpby_kernel<<<blocks_for(n), 256, 0, s>>>(u, prod, n, a); GN_LAUNCH_CHECK();
  }
  // Muon+ renormalisation to sqrt(min(rows, cols)), then the row / column mean squares of the result
  rowss_kernel<<<rows, RT, 0, s>>>(u, cols, rowss); GN_LAUNCH_CHECK();
  sum_d_kernel<<<1, 1024, 0, s>>>(rowss, rows, scal, 1, 0); GN_LAUNCH_CHECK();
  scale_rows_kernel<<<rows, RT, 0, s>>>(u, cols, scal, 1, (float)std::sqrt((double)std::min(rows, cols)), rowss); GN_LAUNCH_CHECK();
  const bool per_row = rows >= cols;
  const int nv = per_row ? rows : cols, reduce = per_row ? cols : rows;
  const double* ss = rowss;
  if (!per_row) { colss_kernel<<<blocks_for(cols), 256, 0, s>>>(u, rows, cols, colss); GN_LAUNCH_CHECK(); ss = colss; }
  muon_variance_kernel<<<1, 1024, 0, s>>>(ss, nv, reduce, beta2, second, fin); GN_LAUNCH_CHECK();
  muon_apply_kernel<<<blocks_for(n), 256, 0, s>>>(p, u, fin, rows, cols, per_row ? 1 : 0, lr, wd); GN_LAUNCH_CHECK();
  return GN_OK;
}

int sinkhorn_launch(float* p, float* g, float* mom, int rows, int cols, float lr, float momentum, float gamma, int steps, float tau, float eps,
                    void* workspace, cudaStream_t s) {
  GN_REQUIRE(rows > 0 && cols > 0 && steps >= 1 && steps % 2 == 1, "sinkhorn: needs an odd positive number of normalisations (got %d)", steps);
  const int chunks = std::min(128, std::max(1, rows / 64));
  const int chunk_rows = (rows + chunks - 1) / chunks;
  double* scal = (double*)workspace;
  double* rowss = scal + 16;
  double* colscale = rowss + rows;
  double* partial = colscale + cols;
  float* u = g;
  const double lrf = (double)gamma * (double)lr * std::sqrt((double)cols);
  sk_momentum_kernel<<<rows, RT, 0, s>>>(u, mom, cols, (double)momentum, rowss); GN_LAUNCH_CHECK();
  sum_d_kernel<<<1, 1024, 0, s>>>(rowss, rows, scal, 0, 1); GN_LAUNCH_CHECK();                 // sum of the row norms
  sk_row_step_kernel<<<rows, RT, 0, s>>>(u, p, rows, cols, rowss, scal, (double)tau, nullptr, (double)eps, 1, steps == 1 ? 1 : 0, lrf); GN_LAUNCH_CHECK();
  for (int st = 2; st <= steps; st += 2) {
    dim3 grid((cols + 127) / 128, chunks);
    sk_colss_partial_kernel<<<grid, 128, 0, s>>>(u, rows, cols, chunk_rows, partial); GN_LAUNCH_CHECK();
    sk_colscale_kernel<<<blocks_for(cols), 256, 0, s>>>(partial, chunks, cols, (double)eps, colscale); GN_LAUNCH_CHECK();
    sk_row_step_kernel<<<rows, RT, 0, s>>>(u, p, rows, cols, rowss, scal, 0.0, colscale, (double)eps, 0, st + 1 == steps ? 1 : 0, lrf); GN_LAUNCH_CHECK();
  }
  return GN_OK;
}

}  // namespace gn
