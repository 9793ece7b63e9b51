// Fused glue kernels of the dense transformer (see model_kernels.cuh).  All of
// them are HBM-bound row kernels: one warp per token row (or per (row, head)),
// coalesced row reads, no intermediate tensors.
#include "model_kernels.cuh"

namespace gn {

constexpr int WPB = 8;  // warps per block

__device__ __forceinline__ float row_inv_rms(float ss, int cols) {
  // kernels/scalar/norm.go:26-40: mean square rounded to float32, then 1/sqrt(ms + eps).
  float ms = ss / (float)cols;
  return (float)(1.0 / sqrt((double)ms + (double)kNormEps));
}

// ---------------------------------------------------------------- embedding
__global__ void __launch_bounds__(WPB * 32) embed_norm_kernel(const int32_t* ids, const float* wte, float* E, int64_t rows, int d) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r >= rows) return;
  const float* src = wte + (int64_t)ids[r] * d;
  float ss = 0;
  for (int c = lane; c < d; c += 32) { float x = src[c]; ss = fmaf(x, x, ss); }
  ss = warp_sum(ss);
  float inv = row_inv_rms(ss, d);
  for (int c = lane; c < d; c += 32) E[r * d + c] = src[c] * inv;
}
int embed_norm_launch(const int32_t* ids, const float* wte, float* E, int64_t rows, int d, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  embed_norm_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(ids, wte, E, rows, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// -------------------------------------------------------------------- smear
__global__ void __launch_bounds__(WPB * 32) smear_kernel(const float* E, float* X, const float* prev_in, float* prev_out, int prev_mul, float* sig_out,
                                                         const float* Ws, const float* lambda, int B, int T, int d) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r >= (int64_t)B * T) return;
  int b = (int)(r / T), t = (int)(r % T);
  const float* e = E + r * d;
  const float* pv = nullptr;
  if (t >= 1) pv = e - d;
  else if (prev_in) pv = prev_in + (int64_t)b * prev_mul * d;
  float gate = 0.0f;
  if (pv) {
    float pre = (lane < kSmearChannels) ? e[lane] * Ws[lane] : 0.0f;
    pre = warp_sum(pre);
    float sg = sigmoid_exact(pre);
    if (sig_out && t >= 1 && lane == 0) sig_out[(int64_t)b * (T - 1) + (t - 1)] = sg;
    gate = sg * lambda[0];
  }
  for (int c = lane; c < d; c += 32) {
    float v = e[c];
    if (pv) v += gate * pv[c];
    X[r * d + c] = v;
  }
  if (prev_out && t == T - 1)
    for (int c = lane; c < d; c += 32) prev_out[(int64_t)b * prev_mul * d + c] = e[c];
}
int smear_launch(const float* E, float* X, const float* prev_in, float* prev_out, int prev_mul, float* sig_out, const float* Ws,
                 const float* lambda, int B, int T, int d, cudaStream_t s) {
  int64_t rows = (int64_t)B * T;
  if (rows <= 0) return GN_OK;
  smear_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(E, X, prev_in, prev_out, prev_mul, sig_out, Ws, lambda, B, T, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ---------------------------------------------------------- mix / norm / backout
__global__ void __launch_bounds__(WPB * 32) mix_norm_kernel(const float* X, const float* X0, const float* rho, const float* chi, int layer, float* Xin,
                                                            float* H, float* Hh, float* Hl, int64_t rows, int d) {
  pdl_trigger();
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r >= rows) return;
  float rw = rho[layer], xw = chi[layer];
  float ss = 0;
  for (int c = lane; c < d; c += 32) {
    // combineResidual: rw*x + xw*x0 with two roundings of the products (model/transformer.go:544-551)
    float v = __fadd_rn(__fmul_rn(rw, X[r * d + c]), __fmul_rn(xw, X0[r * d + c]));
    Xin[r * d + c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  float inv = row_inv_rms(ss, d);
  for (int c = lane; c < d; c += 32) {
    float v = Xin[r * d + c] * inv;
    H[r * d + c] = v;
    if (Hh) { float h, l; split_tf32(v, h, l); Hh[r * d + c] = h; Hl[r * d + c] = l; }
  }
}
int mix_norm_launch(const float* X, const float* X0, const float* rho, const float* chi, int layer, float* Xin, float* H, float* Hh, float* Hl,
                    int64_t rows, int d, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  mix_norm_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(X, X0, rho, chi, layer, Xin, H, Hh, Hl, rows, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(WPB * 32) backout_norm_kernel(const float* X, const float* BO, const float* lambda_b, const int32_t* sel, float* FP,
                                                                float* Y, float* Yh, float* Yl, int64_t rows, int d) {
  pdl_trigger();
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r >= rows) return;
  int64_t src = sel ? sel[r] : r;
  float lam = BO ? -lambda_b[0] : 0.0f;
  float ss = 0;
  // values are recomputed in the second loop instead of being staged
  for (int c = lane; c < d; c += 32) {
    float v = X[src * d + c];
    if (BO) v = v + lam * BO[src * d + c];
    if (FP) FP[r * d + c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  float inv = row_inv_rms(ss, d);
  for (int c = lane; c < d; c += 32) {
    float v = X[src * d + c];
    if (BO) v = v + lam * BO[src * d + c];
    v = v * inv;
    Y[r * d + c] = v;
    if (Yh) { float h, l; split_tf32(v, h, l); Yh[r * d + c] = h; Yl[r * d + c] = l; }
  }
}
int backout_norm_launch(const float* X, const float* BO, const float* lambda_b, const int32_t* sel, float* FP, float* Y, float* Yh, float* Yl,
                        int64_t rows, int d, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  backout_norm_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(X, BO, lambda_b, sel, FP, Y, Yh, Yl, rows, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}
int norm_launch(const float* X, float* Y, float* Yh, float* Yl, int64_t rows, int d, cudaStream_t s) {
  return backout_norm_launch(X, nullptr, nullptr, nullptr, nullptr, Y, Yh, Yl, rows, d, s);
}

// One block per row, one float4 per thread.
__global__ void __launch_bounds__(1024) sum_norm_kernel(SumNorm p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[33];
  const int64_t r = blockIdx.x;
  const int64_t src = p.sel ? p.sel[r] : r;
  const int c = threadIdx.x * 4;
  const bool live = c < p.d;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    v = *reinterpret_cast<const float4*>(p.R + src * p.d + c);
    if (p.part.on()) { const float4 q = p.part.at4(src, c); v.x = __fadd_rn(q.x, v.x); v.y = __fadd_rn(q.y, v.y); v.z = __fadd_rn(q.z, v.z); v.w = __fadd_rn(q.w, v.w); }
    if (p.Xsum) *reinterpret_cast<float4*>(p.Xsum + r * p.d + c) = v;
    if (p.X0) {
      // combineResidual: two rounded products, then the sum (model/transformer.go:544-551)
      const float rw = p.rho[p.layer], xw = p.chi[p.layer];
      const float4 x0 = *reinterpret_cast<const float4*>(p.X0 + r * p.d + c);
      v.x = __fadd_rn(__fmul_rn(rw, v.x), __fmul_rn(xw, x0.x)); v.y = __fadd_rn(__fmul_rn(rw, v.y), __fmul_rn(xw, x0.y));
      v.z = __fadd_rn(__fmul_rn(rw, v.z), __fmul_rn(xw, x0.z)); v.w = __fadd_rn(__fmul_rn(rw, v.w), __fmul_rn(xw, x0.w));
    }
    if (p.BO) {
      const float lam = -p.lambda_b[0];
      const float4 bo = *reinterpret_cast<const float4*>(p.BO + src * p.d + c);
      v.x = v.x + lam * bo.x; v.y = v.y + lam * bo.y; v.z = v.z + lam * bo.z; v.w = v.w + lam * bo.w;
    }
    if (p.V) *reinterpret_cast<float4*>(p.V + r * p.d + c) = v;
  }
  float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
  ss = block_sum(ss, scratch);
  const float inv = row_inv_rms(ss, p.d);
  if (live) {
    const float4 y = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
    *reinterpret_cast<float4*>(p.Y + r * p.d + c) = y;
    if (p.Yh) {
      float4 h, l;
      split_tf32(y.x, h.x, l.x); split_tf32(y.y, h.y, l.y); split_tf32(y.z, h.z, l.z); split_tf32(y.w, h.w, l.w);
      *reinterpret_cast<float4*>(p.Yh + r * p.d + c) = h;
      *reinterpret_cast<float4*>(p.Yl + r * p.d + c) = l;
    }
  }
}
int sum_norm_launch(const SumNorm& p, cudaStream_t s) {
  if (p.rows <= 0) return GN_OK;
  GN_REQUIRE(sum_norm_supported(p.d), "sum_norm: width %d unsupported", p.d);
  const int threads = (p.d / 4 + 31) / 32 * 32;
  GN_CUDA(launch_pdl(sum_norm_kernel, dim3((unsigned)p.rows), dim3(threads), 0, s, p));
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ------------------------------------------------------------ decode front
// The first three kernels of a decode step in one: e = norm(wte[id]); x0 = e + lambda * sigmoid(Ws . e[0:24]) * prev;
// prev <- e (model/transformer.go:255-301,520-530); then layer 0's residual mix and norm (model/transformer.go:312,
// model/block.go:39) with the tf32 split of the result.  One block per row, one float4 per thread.
__global__ void __launch_bounds__(1024) decode_front_kernel(const int32_t* __restrict__ ids, const float* __restrict__ wte, float* __restrict__ prev,
                                                            const float* __restrict__ Ws, const float* __restrict__ lambda, const float* __restrict__ rho,
                                                            const float* __restrict__ chi, float* __restrict__ X0, float* __restrict__ Xin,
                                                            float* __restrict__ H, float* __restrict__ Hh, float* __restrict__ Hl, int d) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[33];
  __shared__ float gate_sh;
  const int64_t r = blockIdx.x;
  const int c = threadIdx.x * 4;
  const bool live = c < d;
  float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) e = *reinterpret_cast<const float4*>(wte + (int64_t)ids[r] * d + c);
  float ss = fmaf(e.x, e.x, fmaf(e.y, e.y, fmaf(e.z, e.z, e.w * e.w)));
  ss = block_sum(ss, scratch);
  float inv = row_inv_rms(ss, d);
  e.x *= inv; e.y *= inv; e.z *= inv; e.w *= inv;
  // gate from the first kSmearChannels channels of the normalised embedding (they sit in the first warp)
  if (threadIdx.x < 32) {
    float pre = 0.0f;
    const float ev[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) if (c + j < kSmearChannels) pre = fmaf(ev[j], Ws[c + j], pre);
    pre = warp_sum(pre);
    if (threadIdx.x == 0) gate_sh = sigmoid_exact(pre) * lambda[0];
  }
  __syncthreads();
  const float gate = gate_sh;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const float4 pv = *reinterpret_cast<const float4*>(prev + r * d + c);
    *reinterpret_cast<float4*>(prev + r * d + c) = e;
    float4 x0 = make_float4(e.x + gate * pv.x, e.y + gate * pv.y, e.z + gate * pv.z, e.w + gate * pv.w);
    *reinterpret_cast<float4*>(X0 + r * d + c) = x0;
    const float rw = rho[0], xw = chi[0];
    v.x = __fadd_rn(__fmul_rn(rw, x0.x), __fmul_rn(xw, x0.x)); v.y = __fadd_rn(__fmul_rn(rw, x0.y), __fmul_rn(xw, x0.y));
    v.z = __fadd_rn(__fmul_rn(rw, x0.z), __fmul_rn(xw, x0.z)); v.w = __fadd_rn(__fmul_rn(rw, x0.w), __fmul_rn(xw, x0.w));
    *reinterpret_cast<float4*>(Xin + r * d + c) = v;
  }
  float s2 = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
  s2 = block_sum(s2, scratch);
  const float inv2 = row_inv_rms(s2, d);
  if (live) {
    const float4 y = make_float4(v.x * inv2, v.y * inv2, v.z * inv2, v.w * inv2);
    *reinterpret_cast<float4*>(H + r * d + c) = y;
    if (Hh) {
      float4 h, l;
      split_tf32(y.x, h.x, l.x); split_tf32(y.y, h.y, l.y); split_tf32(y.z, h.z, l.z); split_tf32(y.w, h.w, l.w);
      *reinterpret_cast<float4*>(Hh + r * d + c) = h;
      *reinterpret_cast<float4*>(Hl + r * d + c) = l;
    }
  }
}
int decode_front_launch(const int32_t* ids, const float* wte, float* prev, const float* Ws, const float* lambda, const float* rho, const float* chi,
                        float* X0, float* Xin, float* H, float* Hh, float* Hl, int64_t rows, int d, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  GN_REQUIRE(sum_norm_supported(d) && d >= 4 * 32 && kSmearChannels <= 128, "decode_front: width %d unsupported", d);
  const int threads = (d / 4 + 31) / 32 * 32;
  GN_CUDA(launch_pdl(decode_front_kernel, dim3((unsigned)rows), dim3(threads), 0, s, ids, wte, prev, Ws, lambda, rho, chi, X0, Xin, H, Hh, Hl, d));
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ----------------------------------------------------------------- qkv post
// One warp per (token row, head slot); slots = Hq query heads, Hkv key heads, Hkv value heads.
__global__ void __launch_bounds__(WPB * 32) qkv_post_kernel(QkvPost p) {
  __shared__ __align__(16) float sh[WPB][128];
  pdl_trigger();
  pdl_wait();
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.Hq + 2 * p.Hkv;
  int64_t idx = (int64_t)blockIdx.x * WPB + warp;
  int64_t rows = (int64_t)p.B * p.T;
  if (idx >= rows * slots) return;
  int64_t r = idx / slots; int slot = (int)(idx % slots);
  int b = (int)(r / p.T), t = (int)(r % p.T);
  const int D = p.D, W = slots * D;
  float* x = p.qkv + r * W + (int64_t)slot * D;
  float* buf = sh[warp];
  const int crow = b * p.cache_row_mul;
  const int pos = (p.pos ? p.pos[crow] : 0) + t;

  if (slot < p.Hq + p.Hkv) {
    // ---- rotary on the trailing R channels, pairs (first half, second half)  (model/rotary.go:43-75)
    if (p.part.on()) {
      for (int c = lane * 4; c < D; c += 128) *reinterpret_cast<float4*>(buf + c) = p.part.at4(r, (int64_t)slot * D + c);
    } else {
      for (int c = lane; c < D; c += 32) buf[c] = x[c];
    }
    __syncwarp();
    const int half = p.R / 2, off = D - p.R;
    const float* cw = p.cosv + (int64_t)pos * half; const float* sw = p.sinv + (int64_t)pos * half;
    float y1[2], y2[2];
    int nj = 0;
    for (int j = lane; j < half; j += 32, ++nj) {
      float a = buf[off + j], c2 = buf[off + half + j];
      y1[nj] = __fadd_rn(__fmul_rn(a, cw[j]), __fmul_rn(c2, sw[j]));
      y2[nj] = __fadd_rn(__fmul_rn(-a, sw[j]), __fmul_rn(c2, cw[j]));
    }
    __syncwarp();
    nj = 0;
    for (int j = lane; j < half; j += 32, ++nj) { buf[off + j] = y1[nj]; buf[off + half + j] = y2[nj]; }
    __syncwarp();
    if (p.qk_rot) {
      float* rot = p.qk_rot + r * (int64_t)((p.Hq + p.Hkv) * D) + (int64_t)slot * D;
      for (int c = lane; c < D; c += 32) rot[c] = buf[c];
    }
    // ---- QK norm and the 1.2 scale (model/attention.go:255-256)
    float ss = 0;
    for (int c = lane; c < D; c += 32) ss = fmaf(buf[c], buf[c], ss);
    ss = warp_sum(ss);
    float inv = row_inv_rms(ss, D);
    if (slot < p.Hq) {
      for (int c = lane; c < D; c += 32) x[c] = (buf[c] * inv) * kQKScale;
    } else {
      int hk = slot - p.Hq;
      float* kc = p.kcache ? p.kcache + (((int64_t)crow * p.Hkv + hk) * p.max_seq + pos) * D : nullptr;
      for (int c = lane; c < D; c += 32) {
        float v = (buf[c] * inv) * kQKScale;
        x[c] = v;
        if (kc) kc[c] = v;
      }
    }
  } else {
    // ---- value (+ gated value embedding, model/attention.go:245-250,392-405)
    int hk = slot - p.Hq - p.Hkv;
    float gate = 0.0f;
    const float* ve = nullptr;
    if (p.ve_table) {
      const float* h = p.H + r * p.d;
      float pre = (lane < kVeGateChannels) ? h[lane] * p.ve_gate[hk * kVeGateChannels + lane] : 0.0f;
      pre = warp_sum(pre);
      float sg = sigmoid_exact(pre);
      if (p.ve_sig && lane == 0) p.ve_sig[r * p.Hkv + hk] = sg;
      gate = sg * kVeGateScale;
      ve = p.ve_table + (int64_t)p.ids[r] * (p.Hkv * D) + (int64_t)hk * D;
    }
    float* vc = p.vcache ? p.vcache + (((int64_t)crow * p.Hkv + hk) * p.max_seq + pos) * D : nullptr;
    if (p.part.on()) {
      for (int c = lane * 4; c < D; c += 128) *reinterpret_cast<float4*>(buf + c) = p.part.at4(r, (int64_t)slot * D + c);
      __syncwarp();
    }
    for (int c = lane; c < D; c += 32) {
      float v = p.part.on() ? buf[c] : x[c];
      if (ve) v += gate * ve[c];
      x[c] = v;
      if (vc) vc[c] = v;
    }
  }
}
// head_dim 128 form: a lane holds four consecutive channels (one 16-byte access per tensor), the rotary partner of a
// channel sits half / 4 lanes away, nothing passes through shared memory.  Same arithmetic as the kernel above except
// for the order in which the 128 squares of the norm are added.
__global__ void __launch_bounds__(WPB * 32) qkv_post_vec_kernel(QkvPost p) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.Hq + 2 * p.Hkv;
  const int64_t idx = (int64_t)blockIdx.x * WPB + warp;
  const int64_t rows = (int64_t)p.B * p.T;
  if (idx >= rows * slots) return;
  const int64_t r = idx / slots; const int slot = (int)(idx % slots);
  const int b = (int)(r / p.T), t = (int)(r % p.T);
  constexpr int D = 128;
  const int W = slots * D, c = lane * 4;
  float* x = p.qkv + r * W + (int64_t)slot * D;
  const int crow = b * p.cache_row_mul;
  const int pos = (p.pos ? p.pos[crow] : 0) + t;
  float4 v = p.part.on() ? p.part.at4(r, (int64_t)slot * D + c) : *reinterpret_cast<const float4*>(x + c);
  if (slot < p.Hq + p.Hkv) {
    // ---- rotary on the trailing R channels, pairs (first half, second half)  (model/rotary.go:43-75)
    const int half = p.R / 2, off = D - p.R, hl = half / 4;
    float4 o4;
    o4.x = __shfl_xor_sync(0xffffffffu, v.x, hl); o4.y = __shfl_xor_sync(0xffffffffu, v.y, hl);
    o4.z = __shfl_xor_sync(0xffffffffu, v.z, hl); o4.w = __shfl_xor_sync(0xffffffffu, v.w, hl);
    if (c >= off) {
      const bool first = c < off + half;
      const int j = first ? c - off : c - off - half;
      const float4 cw = *reinterpret_cast<const float4*>(p.cosv + (int64_t)pos * half + j);
      const float4 sw = *reinterpret_cast<const float4*>(p.sinv + (int64_t)pos * half + j);
      if (first) {   // a = this channel, b = its partner in the second half
        v.x = __fadd_rn(__fmul_rn(v.x, cw.x), __fmul_rn(o4.x, sw.x)); v.y = __fadd_rn(__fmul_rn(v.y, cw.y), __fmul_rn(o4.y, sw.y));
        v.z = __fadd_rn(__fmul_rn(v.z, cw.z), __fmul_rn(o4.z, sw.z)); v.w = __fadd_rn(__fmul_rn(v.w, cw.w), __fmul_rn(o4.w, sw.w));
      } else {       // a = the partner in the first half, b = this channel
        v.x = __fadd_rn(__fmul_rn(-o4.x, sw.x), __fmul_rn(v.x, cw.x)); v.y = __fadd_rn(__fmul_rn(-o4.y, sw.y), __fmul_rn(v.y, cw.y));
        v.z = __fadd_rn(__fmul_rn(-o4.z, sw.z), __fmul_rn(v.z, cw.z)); v.w = __fadd_rn(__fmul_rn(-o4.w, sw.w), __fmul_rn(v.w, cw.w));
      }
    }
    if (p.qk_rot) *reinterpret_cast<float4*>(p.qk_rot + r * (int64_t)((p.Hq + p.Hkv) * D) + (int64_t)slot * D + c) = v;
    // ---- QK norm and the 1.2 scale (model/attention.go:255-256)
    float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
    ss = warp_sum(ss);
    const float inv = row_inv_rms(ss, D);
    const float4 y = make_float4((v.x * inv) * kQKScale, (v.y * inv) * kQKScale, (v.z * inv) * kQKScale, (v.w * inv) * kQKScale);
    *reinterpret_cast<float4*>(x + c) = y;
    if (slot >= p.Hq && p.kcache) {
      const int hk = slot - p.Hq;
      *reinterpret_cast<float4*>(p.kcache + (((int64_t)crow * p.Hkv + hk) * p.max_seq + pos) * D + c) = y;
    }
  } else {
    // ---- value (+ gated value embedding, model/attention.go:245-250,392-405)
    const int hk = slot - p.Hq - p.Hkv;
    if (p.ve_table) {
      const float* h = p.H + r * p.d;
      float pre = (lane < kVeGateChannels) ? h[lane] * p.ve_gate[hk * kVeGateChannels + lane] : 0.0f;
      pre = warp_sum(pre);
      const float sg = sigmoid_exact(pre);
      if (p.ve_sig && lane == 0) p.ve_sig[r * p.Hkv + hk] = sg;
      const float gate = sg * kVeGateScale;
      const float4 ve = *reinterpret_cast<const float4*>(p.ve_table + (int64_t)p.ids[r] * (p.Hkv * D) + (int64_t)hk * D + c);
      v.x += gate * ve.x; v.y += gate * ve.y; v.z += gate * ve.z; v.w += gate * ve.w;
    }
    *reinterpret_cast<float4*>(x + c) = v;
    if (p.vcache) *reinterpret_cast<float4*>(p.vcache + (((int64_t)crow * p.Hkv + hk) * p.max_seq + pos) * D + c) = v;
  }
}

int qkv_post_launch(const QkvPost& p, cudaStream_t s) {
  int64_t n = (int64_t)p.B * p.T * (p.Hq + 2 * p.Hkv);
  if (n <= 0) return GN_OK;
  GN_REQUIRE(p.D <= 128 && p.R <= p.D && p.R % 2 == 0 && p.R / 2 <= 64, "qkv_post: head_dim %d / rotary %d unsupported", p.D, p.R);
  GN_REQUIRE(!p.part.on() || p.D % 4 == 0, "qkv_post: unreduced input needs head_dim %% 4 == 0 (got %d)", p.D);
  const int half = p.R / 2;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = p.D == 128 && half >= 4 && half % 4 == 0 && ((half / 4) & (half / 4 - 1)) == 0 && (128 - p.R) % 4 == 0 && al16(p.qkv) && al16(p.cosv) && al16(p.sinv) &&
                   al16(p.qk_rot) && al16(p.kcache) && al16(p.vcache) && al16(p.ve_table);
  if (vec) { GN_CUDA(launch_pdl(qkv_post_vec_kernel, dim3(ceil_div(n, WPB)), dim3(WPB * 32), 0, s, p)); }
  else GN_CUDA(launch_pdl(qkv_post_kernel, dim3(ceil_div(n, WPB)), dim3(WPB * 32), 0, s, p));
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ----------------------------------------------------------------- KV cache
// cache layout: [layer*2 (k,v)][row][head][max_seq][D]; copies positions [0,len) of row p*group
// to the other rows of its group.
__global__ void __launch_bounds__(256) kv_replicate_kernel(float* cache, int64_t layer_stride, int64_t row_stride, int64_t head_stride, int Hkv, int D,
                                                           int group, int len) {
  // grid: x = chunk of (head, pos, D) floats, y = prompt, z = layer*2
  int p = blockIdx.y;
  float* base = cache + (int64_t)blockIdx.z * layer_stride + (int64_t)p * group * row_stride;
  int64_t per_head = (int64_t)len * D;
  int64_t total = per_head * Hkv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int h = (int)(i / per_head); int64_t o = i % per_head;
    float v = base[(int64_t)h * head_stride + o];
    for (int g = 1; g < group; ++g) base[(int64_t)g * row_stride + (int64_t)h * head_stride + o] = v;
  }
}
__global__ void __launch_bounds__(256) prev_replicate_kernel(float* prev, int d, int32_t* pos, int n_prompts, int group) {
  int p = blockIdx.x;
  for (int g = 1; g < group; ++g) {
    for (int c = threadIdx.x; c < d; c += blockDim.x) prev[((int64_t)p * group + g) * d + c] = prev[(int64_t)p * group * d + c];
    if (threadIdx.x == 0 && pos) pos[p * group + g] = pos[p * group];
  }
}
int kv_replicate_launch(float* cache, int64_t layer_stride, int n_layer2, int64_t row_stride, int64_t head_stride, int Hkv, int D, int n_prompts,
                        int group, int len, float* prev, int d, int32_t* pos, cudaStream_t s) {
  if (n_prompts <= 0 || group <= 1) return GN_OK;
  int64_t total = (int64_t)len * D * Hkv;
  dim3 grid(std::max(1, std::min(ceil_div(total, 256), 64)), n_prompts, n_layer2);
  kv_replicate_kernel<<<grid, 256, 0, s>>>(cache, layer_stride, row_stride, head_stride, Hkv, D, group, len);
  GN_LAUNCH_CHECK();
  if (prev) {
    prev_replicate_kernel<<<n_prompts, 256, 0, s>>>(prev, d, pos, n_prompts, group);
    GN_LAUNCH_CHECK();
  }
  return GN_OK;
}

__global__ void fill_i32_kernel(int32_t* dst, int32_t v, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = v;
}
__global__ void add_i32_kernel(int32_t* dst, int32_t v, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] += v;
}
__global__ void ctx_from_pos_kernel(const int32_t* pos, int32_t* ctx, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ctx[i] = pos[i] + 1;
}
int fill_i32_launch(int32_t* dst, int32_t value, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  fill_i32_kernel<<<ceil_div(n, 256), 256, 0, s>>>(dst, value, n); GN_LAUNCH_CHECK(); return GN_OK;
}
int add_i32_launch(int32_t* dst, int32_t delta, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  add_i32_kernel<<<ceil_div(n, 256), 256, 0, s>>>(dst, delta, n); GN_LAUNCH_CHECK(); return GN_OK;
}
__global__ void add_u32_kernel(uint32_t* dst, uint32_t v) { *dst += v; }
int add_u32_launch(uint32_t* dst, uint32_t delta, cudaStream_t s) { add_u32_kernel<<<1, 1, 0, s>>>(dst, delta); GN_LAUNCH_CHECK(); return GN_OK; }
int ctx_from_pos_launch(const int32_t* pos, int32_t* ctx, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  ctx_from_pos_kernel<<<ceil_div(n, 256), 256, 0, s>>>(pos, ctx, n); GN_LAUNCH_CHECK(); return GN_OK;
}

__global__ void engine_step_kernel(const int32_t* sampled, int32_t* out_tokens, int32_t* out_lengths, int32_t* done, int32_t* n_done, int rows,
                                   int max_tokens, int bos, int aend) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows || done[r]) return;
  int t = sampled[r];
  if (t == aend || t == bos) { done[r] = 1; atomicAdd(n_done, 1); }
  else { int n = out_lengths[r]; if (n < max_tokens) { out_tokens[(int64_t)r * max_tokens + n] = t; out_lengths[r] = n + 1; } }
}
int engine_step_launch(const int32_t* sampled, int32_t* out_tokens, int32_t* out_lengths, int32_t* done, int32_t* n_done, int rows, int max_tokens,
                       int bos, int aend, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  engine_step_kernel<<<ceil_div(rows, 256), 256, 0, s>>>(sampled, out_tokens, out_lengths, done, n_done, rows, max_tokens, bos, aend);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ============================================================== backward glue
__global__ void __launch_bounds__(WPB * 32) qkv_post_bwd_kernel(QkvPostBwd p) {
  __shared__ float sh[WPB][128];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.Hq + 2 * p.Hkv;
  int64_t idx = (int64_t)blockIdx.x * WPB + warp;
  int64_t rows = (int64_t)p.B * p.T;
  if (idx >= rows * slots) return;
  int64_t r = idx / slots; int slot = (int)(idx % slots);
  int t = (int)(r % p.T);
  const int D = p.D, W = slots * D;
  float* g = p.dqkv + r * W + (int64_t)slot * D;
  float* buf = sh[warp];
  if (slot < p.Hq + p.Hkv) {
    // model/train.go:334-343: scale by 1.2, RMSNorm backward on the saved post-rotary
    // value, then the rotation transposed (negated sine).
    const float* x = p.qk_rot + r * (int64_t)((p.Hq + p.Hkv) * D) + (int64_t)slot * D;
    float ss = 0, dp = 0;
    for (int c = lane; c < D; c += 32) { float xv = x[c]; float gv = g[c] * kQKScale; ss = fmaf(xv, xv, ss); dp = fmaf(gv, xv, dp); }
    ss = warp_sum(ss); dp = warp_sum(dp);
    double ms = (double)ss / (double)D;
    double rms = sqrt(ms + (double)kNormEps);
    float inv = (float)(1.0 / rms);
    float coef = (float)((double)dp / ((double)D * rms * rms * rms));
    for (int c = lane; c < D; c += 32) buf[c] = (g[c] * kQKScale) * inv - coef * x[c];
    __syncwarp();
    const int half = p.R / 2, off = D - p.R;
    const float* cw = p.cosv + (int64_t)t * half; const float* sw = p.sinv + (int64_t)t * half;
    float y1[2], y2[2];
    int nj = 0;
    for (int j = lane; j < half; j += 32, ++nj) {
      float a = buf[off + j], c2 = buf[off + half + j];
      float sn = -sw[j];
      y1[nj] = __fadd_rn(__fmul_rn(a, cw[j]), __fmul_rn(c2, sn));
      y2[nj] = __fadd_rn(__fmul_rn(-a, sn), __fmul_rn(c2, cw[j]));
    }
    __syncwarp();
    nj = 0;
    for (int j = lane; j < half; j += 32, ++nj) { buf[off + j] = y1[nj]; buf[off + half + j] = y2[nj]; }
    __syncwarp();
    for (int c = lane; c < D; c += 32) g[c] = buf[c];
  } else if (p.ve_table) {
    // model/train.go:375-397
    int hk = slot - p.Hq - p.Hkv;
    float sg = p.ve_sig[r * p.Hkv + hk];
    float scale = sg * kVeGateScale;
    int64_t id = p.ids[r];
    const float* ve = p.ve_table + id * (p.Hkv * D) + (int64_t)hk * D;
    float* vg = p.ve_grad + id * (p.Hkv * D) + (int64_t)hk * D;
    float dot = 0;
    for (int c = lane; c < D; c += 32) {
      float dv = g[c];
      dot = fmaf(dv, ve[c], dot);
      atomicAdd(vg + c, dv * scale);
    }
    dot = warp_sum(dot);
    if (lane == 0) {
      float dsig = dot * kVeGateScale;
      p.dpre[r * p.Hkv + hk] = dsig * sg * (1.0f - sg);
    }
  }
}
int qkv_post_backward_launch(const QkvPostBwd& p, cudaStream_t s) {
  int64_t n = (int64_t)p.B * p.T * (p.Hq + 2 * p.Hkv);
  if (n <= 0) return GN_OK;
  qkv_post_bwd_kernel<<<ceil_div(n, WPB), WPB * 32, 0, s>>>(p);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// dWg[h][c] += sum_r dpre[r,h]*H[r,c]: one block per (h, c), fixed-order tree -> reproducible.
__global__ void __launch_bounds__(256) ve_gate_wgrad_kernel(const float* dpre, const float* H, float* dWg, int64_t rows, int Hkv, int d) {
  __shared__ double sh[32];
  int h = blockIdx.x / kVeGateChannels, c = blockIdx.x % kVeGateChannels;
  double acc = 0;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) acc += (double)dpre[r * Hkv + h] * (double)H[r * d + c];
  acc = block_sum_d(acc, sh);
  if (threadIdx.x == 0) dWg[h * kVeGateChannels + c] += (float)acc;
}
__global__ void __launch_bounds__(256) ve_gate_dh_kernel(const float* dpre, const float* Wg, float* dH, int64_t rows, int Hkv, int d) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * kVeGateChannels) return;
  int64_t r = i / kVeGateChannels; int c = (int)(i % kVeGateChannels);
  float acc = 0;
  for (int h = 0; h < Hkv; ++h) acc = fmaf(dpre[r * Hkv + h], Wg[h * kVeGateChannels + c], acc);
  dH[r * d + c] += acc;
}
int ve_gate_backward_launch(const float* dpre, const float* H, const float* Wg, float* dWg, float* dH, int64_t rows, int Hkv, int d, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  ve_gate_wgrad_kernel<<<Hkv * kVeGateChannels, 256, 0, s>>>(dpre, H, dWg, rows, Hkv, d);
  GN_LAUNCH_CHECK();
  ve_gate_dh_kernel<<<ceil_div(rows * kVeGateChannels, 256), 256, 0, s>>>(dpre, Wg, dH, rows, Hkv, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(256) mix_bwd_kernel(const float* dXin, const float* prevX, const float* X0, const float* rho, const float* chi, int layer,
                                                      float* dX, float* dX0, int first, double* acc_rho, double* acc_chi, int64_t n) {
  __shared__ double sh[32];
  float rw = rho[layer], xw = chi[layer];
  double a0 = 0, a1 = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float g = dXin[i];
    a0 += (double)g * (double)prevX[i];
    a1 += (double)g * (double)X0[i];
    dX[i] = g * rw;
    dX0[i] = first ? xw * g : dX0[i] + xw * g;
  }
  a0 = block_sum_d(a0, sh);
  a1 = block_sum_d(a1, sh);
  if (threadIdx.x == 0) { atomicAdd(acc_rho, a0); atomicAdd(acc_chi, a1); }
}
int mix_backward_launch(const float* dXin, const float* prevX, const float* X0, const float* rho, const float* chi, int layer, float* dX, float* dX0,
                        int first, double* acc_rho, double* acc_chi, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 8);
  mix_bwd_kernel<<<blocks, 256, 0, s>>>(dXin, prevX, X0, rho, chi, layer, dX, dX0, first, acc_rho, acc_chi, n);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(256) dot_acc_kernel(const float* a, const float* b, int64_t n, double sign, double* acc) {
  __shared__ double sh[32];
  double t = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) t += (double)a[i] * (double)b[i];
  t = block_sum_d(t, sh);
  if (threadIdx.x == 0) atomicAdd(acc, sign * t);
}
int dot_accumulate_launch(const float* a, const float* b, int64_t n, double sign, double* acc, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 8);
  dot_acc_kernel<<<blocks, 256, 0, s>>>(a, b, n, sign, acc);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(256) axpy_kernel(float* dst, const float* src, float alpha, const float* alpha_dev, float alpha_sign, int accumulate, int64_t n) {
  float a = alpha_dev ? alpha_sign * alpha_dev[0] : alpha;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = accumulate ? dst[i] + a * src[i] : a * src[i];
}
int axpy_launch(float* dst, const float* src, float alpha, const float* alpha_dev, float alpha_sign, int accumulate, int64_t n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 8);
  axpy_kernel<<<blocks, 256, 0, s>>>(dst, src, alpha, alpha_dev, alpha_sign, accumulate, n);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void scalar_flush_kernel(float* grad, double* acc, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { grad[i] += (float)acc[i]; acc[i] = 0.0; }
}
int scalar_flush_launch(float* grad, double* acc, int n, cudaStream_t s) {
  if (n <= 0) return GN_OK;
  scalar_flush_kernel<<<ceil_div(n, 64), 64, 0, s>>>(grad, acc, n);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// Smear backward, gather form: one warp per (b, t).
__global__ void __launch_bounds__(WPB * 32) smear_bwd_kernel(const float* dX, const float* Xpost, const float* E, const float* sig, const float* Ws,
                                                             const float* lambda, float* dE, float* dWs, double* dlambda_acc, int B, int T, int d) {
  __shared__ float wacc[kSmearChannels];
  __shared__ double lacc;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < kSmearChannels) wacc[threadIdx.x] = 0.0f;
  if (threadIdx.x == 0) lacc = 0.0;
  __syncthreads();
  int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r < (int64_t)B * T) {
    int b = (int)(r / T), t = (int)(r % T);
    const float lam = lambda[0];
    const float* g = dX + r * d;
    float dgate = 0.0f;
    if (t >= 1) {
      const float* xp = Xpost + (r - 1) * d;
      double gs = 0;
      for (int c = lane; c < d; c += 32) gs += (double)g[c] * (double)xp[c];
      gs = warp_sum_d(gs);
      float sg = sig[(int64_t)b * (T - 1) + (t - 1)];
      dgate = (float)(gs * (double)lam) * sg * (1.0f - sg);
      if (lane == 0) atomicAdd(&lacc, gs * (double)sg);
      if (lane < kSmearChannels) atomicAdd(&wacc[lane], dgate * E[r * d + lane]);
    }
    float gnext = 0.0f;
    if (t + 1 < T) gnext = lam * sig[(int64_t)b * (T - 1) + t];
    for (int c = lane; c < d; c += 32) {
      float v = g[c];
      if (t + 1 < T) v += g[d + c] * gnext;
      if (t >= 1 && c < kSmearChannels) v += dgate * Ws[c];
      dE[r * d + c] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < kSmearChannels) atomicAdd(dWs + threadIdx.x, wacc[threadIdx.x]);
  if (threadIdx.x == 0) atomicAdd(dlambda_acc, lacc);
}
int smear_backward_launch(const float* dX, const float* Xpost, const float* E, const float* sig, const float* Ws, const float* lambda, float* dE,
                          float* dWs, double* dlambda_acc, int B, int T, int d, cudaStream_t s) {
  int64_t rows = (int64_t)B * T;
  if (rows <= 0) return GN_OK;
  smear_bwd_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(dX, Xpost, E, sig, Ws, lambda, dE, dWs, dlambda_acc, B, T, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

__global__ void __launch_bounds__(WPB * 32) embed_bwd_kernel(const int32_t* ids, const float* wte, const float* dE, float* wte_grad, int64_t rows, int d) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r >= rows) return;
  int64_t id = ids[r];
  const float* x = wte + id * d; const float* g = dE + r * d; float* out = wte_grad + id * d;
  float ss = 0, dp = 0;
  for (int c = lane; c < d; c += 32) { float xv = x[c]; ss = fmaf(xv, xv, ss); dp = fmaf(g[c], xv, dp); }
  ss = warp_sum(ss); dp = warp_sum(dp);
  double ms = (double)ss / (double)d;
  double rms = sqrt(ms + (double)kNormEps);
  float inv = (float)(1.0 / rms);
  float coef = (float)((double)dp / ((double)d * rms * rms * rms));
  for (int c = lane; c < d; c += 32) atomicAdd(out + c, g[c] * inv - coef * x[c]);
}
int embed_backward_launch(const int32_t* ids, const float* wte, const float* dE, float* wte_grad, int64_t rows, int d, cudaStream_t s) {
  if (rows <= 0) return GN_OK;
  embed_bwd_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(ids, wte, dE, wte_grad, rows, d);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

double* dummy_unused() { return nullptr; }

}  // namespace gn
