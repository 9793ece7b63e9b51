// Fused policy-gradient loss and its backward at the logits
// (trainer/rl.go:23-56 with tensors/loss.go:16-46; the softcap backward of
// tensors/backward.go:108-116 can be folded in), and the group-relative
// advantage of cmd/chat_rl/main.go:137-154.
//
// The reference makes three passes over the [rows, vocab] matrix (log-sum-exp,
// a second softmax over ALL rows, then a single-threaded gradient loop) and a
// fourth for the softcap backward.  Here one CTA owns a row: the row is read
// from HBM once into registers (the part beyond 32768 columns is re-read, from
// L2), reduced to (max, sum) on chip, and the gradient is written once.
// Ignored rows (target == -1) are never read: their gradient row is zeroed.
// HBM traffic per call = 4*vocab*(2*valid + masked) bytes + O(rows).
#include "kernels.cuh"

namespace gn {

constexpr int LT = 1024;       // threads per row
constexpr int LIPT = 32;       // values per thread held in registers

__device__ __forceinline__ void ms_merge(float& m, float& s, float om, float os) {
  float mn = fmaxf(m, om);
  float a = (m == -INFINITY) ? 0.0f : __expf(m - mn);
  float b = (om == -INFINITY) ? 0.0f : __expf(om - mn);
  s = s * a + os * b;
  m = mn;
}

template <bool VEC>
__global__ void __launch_bounds__(LT) pg_loss_kernel(const float* __restrict__ logits, const int32_t* __restrict__ targets, const float* __restrict__ adv,
                                                     int64_t rows, int vocab, int64_t ld, int seq_len, float norm, float softcap, float* __restrict__ nll,
                                                     float* dlogits, int64_t ldd, double* __restrict__ row_loss, int* __restrict__ bad_targets,
                                                     int64_t row_offset) {
  __shared__ float sh_m[32], sh_s[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int32_t target = targets[row];
    float* drow = dlogits ? dlogits + row * ldd : nullptr;
    // A target outside {-1} and [0, vocab) would index outside the row: the row is treated as ignored and counted,
    // and the host turns a non-zero count into GN_ERR_INVALID (the reference panics on Go's bounds check instead).
    if (target < -1 || target >= vocab) { if (tid == 0 && bad_targets) atomicAdd(bad_targets, 1); }
    if (target < 0 || target >= vocab) {
      if (drow) {
        if (VEC) { float4 z = make_float4(0, 0, 0, 0); for (int c = tid * 4; c < vocab; c += LT * 4) *reinterpret_cast<float4*>(drow + c) = z; }
        else { for (int c = tid; c < vocab; c += LT) drow[c] = 0.0f; }
      }
      if (tid == 0) { if (nll) nll[row] = 0.0f; row_loss[row] = 0.0; }
      continue;
    }
    const float* xrow = logits + row * ld;
    const float x_target = xrow[target];  // read before any in-place write of this row
    float x[LIPT];
    float m = -INFINITY, s = 0.0f;
    // ---- pass 1: registers hold the first LIPT*LT columns
    if (VEC) {
#pragma unroll
      for (int it = 0; it < LIPT / 4; ++it) {
        int c = (it * LT + tid) * 4;
        float4 v = (c < vocab) ? *reinterpret_cast<const float4*>(xrow + c) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        x[it * 4 + 0] = v.x; x[it * 4 + 1] = v.y; x[it * 4 + 2] = v.z; x[it * 4 + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int it = 0; it < LIPT; ++it) { int c = it * LT + tid; x[it] = c < vocab ? xrow[c] : -INFINITY; }
    }
#pragma unroll
    for (int it = 0; it < LIPT / 4; ++it) {
      float m4 = fmaxf(fmaxf(x[it * 4], x[it * 4 + 1]), fmaxf(x[it * 4 + 2], x[it * 4 + 3]));
      if (m4 > -INFINITY) {
        float mn = fmaxf(m, m4);
        float a = (m == -INFINITY) ? 0.0f : __expf(m - mn);
        s = s * a + __expf(x[it * 4] - mn) + __expf(x[it * 4 + 1] - mn) + __expf(x[it * 4 + 2] - mn) + __expf(x[it * 4 + 3] - mn);
        m = mn;
      }
    }
    for (int c = LIPT * LT + tid; c < vocab; c += LT) {  // columns beyond the register window
      float v = xrow[c];
      float mn = fmaxf(m, v);
      float a = (m == -INFINITY) ? 0.0f : __expf(m - mn);
      s = s * a + __expf(v - mn);
      m = mn;
    }
    // ---- block (max, sum)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      ms_merge(m, s, om, os);
    }
    __syncthreads();  // previous row's readers of sh_* are done
    if (lane == 0) { sh_m[warp] = m; sh_s[warp] = s; }
    __syncthreads();
    m = sh_m[lane]; s = sh_s[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      ms_merge(m, s, om, os);
    }
    const float a_over_n = adv[(row_offset + row) / seq_len] / norm;   // rows may be a slice of the batch: row_offset is its first row
    if (tid == 0) {
      float l = m + logf(s) - x_target;
      if (nll) nll[row] = l;
      row_loss[row] = (double)l * (double)adv[(row_offset + row) / seq_len] / (double)norm;
    }
    if (!drow) continue;
    // ---- pass 2: gradient
    const float inv_s = 1.0f / s;
    const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;
    if (VEC) {
#pragma unroll
      for (int it = 0; it < LIPT / 4; ++it) {
        int c = (it * LT + tid) * 4;
        if (c < vocab) {
          float g[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float xv = x[it * 4 + e];
            float p = __expf(xv - m) * inv_s;
            if (c + e == target) p -= 1.0f;
            float gv = p * a_over_n;
            if (softcap > 0.0f) { float t = xv * inv_cap; gv *= (1.0f - t * t); }
            g[e] = gv;
          }
          *reinterpret_cast<float4*>(drow + c) = make_float4(g[0], g[1], g[2], g[3]);
        }
      }
    } else {
#pragma unroll
      for (int it = 0; it < LIPT; ++it) {
        int c = it * LT + tid;
        if (c < vocab) {
          float xv = x[it];
          float p = __expf(xv - m) * inv_s;
          if (c == target) p -= 1.0f;
          float gv = p * a_over_n;
          if (softcap > 0.0f) { float t = xv * inv_cap; gv *= (1.0f - t * t); }
          drow[c] = gv;
        }
      }
    }
    for (int c = LIPT * LT + tid; c < vocab; c += LT) {
      float xv = xrow[c];
      float p = __expf(xv - m) * inv_s;
      if (c == target) p -= 1.0f;
      float gv = p * a_over_n;
      if (softcap > 0.0f) { float t = xv * inv_cap; gv *= (1.0f - t * t); }
      drow[c] = gv;
    }
  }
}

// Fixed-order float64 sum of the per-row terms: the loss is bit-reproducible.
__global__ void __launch_bounds__(1024) loss_sum_kernel(const double* row_loss, int64_t rows, double* out, int accumulate) {
  __shared__ double sh[32];
  double acc = 0;
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) acc += row_loss[i];
  acc = block_sum_d(acc, sh);
  if (threadIdx.x == 0) { if (accumulate) *out += acc; else *out = acc; }
}

int pg_loss_launch(const float* logits, const int32_t* targets, const float* adv, int64_t rows, int vocab, int64_t ld, int seq_len, float norm,
                   float softcap, float* nll, float* dlogits, int64_t ldd, double* row_loss, double* loss_out, int accumulate_loss, cudaStream_t s,
                   int* bad_targets, int64_t row_offset) {
  GN_REQUIRE(vocab > 0 && seq_len > 0, "loss: vocab %d / seq_len %d must be positive", vocab, seq_len);
  if (rows > 0) {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    bool vec = al(logits) && (!dlogits || al(dlogits)) && vocab % 4 == 0 && ld % 4 == 0 && ldd % 4 == 0;
    // In the vector path the register window covers LIPT*LT columns as float4 groups.
    int grid = (int)std::min<int64_t>(rows, (int64_t)num_sms() * 8);
    if (vec) pg_loss_kernel<true><<<grid, LT, 0, s>>>(logits, targets, adv, rows, vocab, ld, seq_len, norm, softcap, nll, dlogits, ldd, row_loss, bad_targets, row_offset);
    else pg_loss_kernel<false><<<grid, LT, 0, s>>>(logits, targets, adv, rows, vocab, ld, seq_len, norm, softcap, nll, dlogits, ldd, row_loss, bad_targets, row_offset);
    GN_LAUNCH_CHECK();
  }
  if (accumulate_loss != 2 && loss_out) {  // 0: overwrite, 1: add, 2: leave the total alone
    loss_sum_kernel<<<1, 1024, 0, s>>>(row_loss, rows, loss_out, accumulate_loss);
    GN_LAUNCH_CHECK();
  }
  return GN_OK;
}

// On-policy distillation loss (tensors/loss.go:84-213): per position the cross-entropy of softmax(teacher / tau)
// under softmax(student / tau), and its gradient (softmax(student/tau) - softmax(teacher/tau)) * scale / tau.
// One CTA per row: a first pass over both rows finds the two maxima, a second the two sums and the teacher-weighted
// student logits, a third writes the gradient; the second and third passes re-read the rows from L2 (a row pair is
// at most 512 KB).  HBM traffic per valid row: 2 rows read + 1 written.  Masked rows are never read.
__global__ void __launch_bounds__(LT) distill_kernel(const float* __restrict__ student, const float* __restrict__ teacher, const int32_t* __restrict__ mask,
                                                     int64_t rows, int vocab, float inv_tau, float grad_scale, float* __restrict__ losses,
                                                     float* __restrict__ grad, double* __restrict__ row_loss) {
  __shared__ float sh[33];
  __shared__ double shd[33];
  const int tid = threadIdx.x;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float* grow = grad ? grad + row * vocab : nullptr;
    if (mask && mask[row] == 0) {
      if (grow) for (int c = tid; c < vocab; c += LT) grow[c] = 0.0f;
      if (tid == 0) { if (losses) losses[row] = 0.0f; row_loss[row] = 0.0; }
      continue;
    }
    const float* s = student + row * vocab; const float* t = teacher + row * vocab;
    float smax = -INFINITY, tmax = -INFINITY;
    for (int c = tid; c < vocab; c += LT) { smax = fmaxf(smax, s[c] * inv_tau); tmax = fmaxf(tmax, t[c] * inv_tau); }
    smax = block_max(smax, sh); tmax = block_max(tmax, sh);
    double ssum = 0.0, tsum = 0.0, weighted = 0.0;
    for (int c = tid; c < vocab; c += LT) {
      const float sv = s[c] * inv_tau;
      const float sw = __expf(sv - smax), tw = __expf(t[c] * inv_tau - tmax);
      ssum += (double)sw; tsum += (double)tw; weighted += (double)tw * (double)sv;
    }
    ssum = block_sum_d(ssum, shd); tsum = block_sum_d(tsum, shd); weighted = block_sum_d(weighted, shd);
    if (tid == 0) {
      const double l = (double)smax + log(ssum) - weighted / tsum;
      if (losses) losses[row] = (float)l;
      row_loss[row] = l;
    }
    if (!grow) continue;
    const float is = (float)(1.0 / ssum), it = (float)(1.0 / tsum);
    for (int c = tid; c < vocab; c += LT)
      grow[c] = (__expf(s[c] * inv_tau - smax) * is - __expf(t[c] * inv_tau - tmax) * it) * grad_scale;
  }
}
// losses / grad nullable; row_loss: [rows] double scratch; loss_sum: device double receiving the sum of the valid rows' losses.
int distillation_launch(const float* student, const float* teacher, const int32_t* mask, int64_t rows, int vocab, float temperature, float scale,
                        float* losses, float* grad, double* row_loss, double* loss_sum, cudaStream_t s) {
  GN_REQUIRE(vocab > 0, "distillation: vocab must be positive");
  const float tau = temperature <= 0.0f ? 1.0f : temperature;   // tensors/loss.go:151-157
  if (rows > 0) {
    const int grid = (int)std::min<int64_t>(rows, (int64_t)num_sms() * 8);
    distill_kernel<<<grid, LT, 0, s>>>(student, teacher, mask, rows, vocab, 1.0f / tau, scale / tau, losses, grad, row_loss);
    GN_LAUNCH_CHECK();
  }
  loss_sum_kernel<<<1, 1024, 0, s>>>(row_loss, rows, loss_sum, 0);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// cmd/chat_rl/main.go:137-154; float32 arithmetic in the reference's order.
__global__ void __launch_bounds__(128) advantage_kernel(const float* rewards, int groups, int group, int mode, float* adv) {
  int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const float* r = rewards + (int64_t)g * group;
  float* a = adv + (int64_t)g * group;
  float mean = 0.0f;
  for (int i = 0; i < group; ++i) mean = __fadd_rn(mean, r[i]);
  mean = __fdiv_rn(mean, (float)group);
  if (mode == 0) { for (int i = 0; i < group; ++i) a[i] = __fsub_rn(r[i], mean); return; }
  float var = 0.0f;
  for (int i = 0; i < group; ++i) { float d = __fsub_rn(r[i], mean); var = __fadd_rn(var, __fmul_rn(d, d)); }
  var = __fdiv_rn(var, (float)group);
  float sd = __fsqrt_rn(var);
  for (int i = 0; i < group; ++i) a[i] = __fdiv_rn(__fsub_rn(r[i], mean), __fadd_rn(sd, 1e-6f));
}
int advantage_launch(const float* rewards, int groups, int group, int mode, float* adv, cudaStream_t s) {
  if (groups <= 0) return GN_OK;
  GN_REQUIRE(group > 0, "advantage: group size must be positive");
  advantage_kernel<<<ceil_div(groups, 128), 128, 0, s>>>(rewards, groups, group, mode, adv);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
