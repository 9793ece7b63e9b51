// The two block variants of the latent preset, inference only:
//   latent_attention  absorbed multi-head latent attention (model/mla.go:185-279): the cache holds one
//                     latent row and one rotary key row per token; the content-key up-projection is
//                     folded into the query and the value up-projection is applied to the attended
//                     latent, so no per-position key or value is ever materialised.
//   moe_ffn           DeepSeekMoE feed-forward (model/block.go:39-46, model/moe.go:118-169): a shared
//                     SwiGLU expert plus top-k routed experts; routing, the stable expert-major
//                     permutation and the weighted un-permutation run on the device.
//
// Data layout
//   latent cache  [layer][row][max_seq][latent]           (model/kvcache.go:224-237)
//   rotary cache  [layer][row][max_seq][Hkv * rope]
//   routed rows   expert-major [rows * k, width], position = offset[expert] + arrival order in
//                 (row, slot) order, exactly the gather of model/moe.go:130-153.
#include "model_internal.cuh"

namespace gnm {

namespace {

constexpr int WPB = 8;   // warps per block in the row kernels

// ------------------------------------------------------------------ latent attention glue
// One warp per (token row, head slot); slots = Hq rotary queries, Hkv rotary keys, 1 latent copy.
//   query slot: rotate P1's q_rope head (model/rotary.go:43-75, every channel rotates) into QF[r, hq, lat:]
//   key slot:   rotate P1's k_rope head into the rotary cache at the token's position
//   last slot:  copy the kv latent into the latent cache
struct MlaPost {
  const float* P1; int64_t n1;       // [rows, n1] = [q_lat | kv_lat | q_rope (Hq*rope) | k_rope (Hkv*rope)]
  float* QF;                          // [rows, Hq, lat + rope]
  float* lat_cache; float* rope_cache;  // this layer's slices
  const float* cosv; const float* sinv;
  const int32_t* pos; int cache_row_mul, max_seq;
  int B, T, Hq, Hkv, lat, rope;
};
__global__ void __launch_bounds__(WPB * 32) mla_post_kernel(MlaPost p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = p.Hq + p.Hkv + 1;
  const int64_t idx = (int64_t)blockIdx.x * WPB + warp;
  const int64_t rows = (int64_t)p.B * p.T;
  if (idx >= rows * slots) return;
  const int64_t r = idx / slots; const int slot = (int)(idx % slots);
  const int b = (int)(r / p.T), t = (int)(r % p.T);
  const int crow = b * p.cache_row_mul;
  const int pos = p.pos[crow] + t;
  const float* row = p.P1 + r * p.n1;
  const int half = p.rope / 2;
  if (slot == p.Hq + p.Hkv) {
    float* dst = p.lat_cache + ((int64_t)crow * p.max_seq + pos) * p.lat;
    for (int c = lane; c < p.lat; c += 32) dst[c] = row[p.lat + c];
    return;
  }
  const float* src; float* dst;
  if (slot < p.Hq) { src = row + 2 * p.lat + (int64_t)slot * p.rope; dst = p.QF + (r * p.Hq + slot) * (int64_t)(p.lat + p.rope) + p.lat; }
  else { const int hk = slot - p.Hq; src = row + 2 * p.lat + (int64_t)(p.Hq + hk) * p.rope; dst = p.rope_cache + (((int64_t)crow * p.max_seq + pos) * p.Hkv + hk) * p.rope; }
  const float* cw = p.cosv + (int64_t)pos * half; const float* sw = p.sinv + (int64_t)pos * half;
  for (int j = lane; j < half; j += 32) {
    const float a = src[j], c = src[half + j];
    dst[j] = __fadd_rn(__fmul_rn(a, cw[j]), __fmul_rn(c, sw[j]));
    dst[half + j] = __fadd_rn(__fmul_rn(-a, sw[j]), __fmul_rn(c, cw[j]));
  }
}

// One warp per (token row, query head): online softmax over the cached positions with
// score = q_abs . latent[j] + q_rope . k_rope[j, hk]; the output is the attended latent.
// Lane e-th element = channel 32 e + lane; latent <= 512, rope <= 64.
struct MlaAttn {
  const float* QF; const float* lat_cache; const float* rope_cache; float* AL;
  const int32_t* pos; int cache_row_mul, max_seq;
  int B, T, Hq, Hkv, lat, rope, window;
};
__global__ void __launch_bounds__(128) mla_attention_kernel(MlaAttn p) {
  constexpr int ME = 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t idx = (int64_t)blockIdx.x * 4 + warp;
  const int64_t rows = (int64_t)p.B * p.T;
  if (idx >= rows * p.Hq) return;
  const int64_t r = idx / p.Hq; const int hq = (int)(idx % p.Hq), hk = hq / (p.Hq / p.Hkv);
  const int b = (int)(r / p.T), t = (int)(r % p.T);
  const int crow = b * p.cache_row_mul;
  const int qpos = p.pos[crow] + t;
  const int hd = p.lat + p.rope;
  const float* q = p.QF + (r * p.Hq + hq) * (int64_t)hd;
  float qa[ME], acc[ME], qr[2];
#pragma unroll
  for (int e = 0; e < ME; ++e) { const int c = e * 32 + lane; qa[e] = c < p.lat ? q[c] : 0.0f; acc[e] = 0.0f; }
#pragma unroll
  for (int e = 0; e < 2; ++e) { const int c = e * 32 + lane; qr[e] = c < p.rope ? q[p.lat + c] : 0.0f; }
  const float* lc = p.lat_cache + (int64_t)crow * p.max_seq * p.lat;
  const float* rc = p.rope_cache + (int64_t)crow * p.max_seq * p.Hkv * p.rope + (int64_t)hk * p.rope;
  int j0 = 0;
  if (p.window >= 0) j0 = max(0, qpos - p.window);   // kernels/scalar/attention.go: masked when qpos - j > window
  float mrun = -INFINITY, lrun = 0.0f;
  for (int j = j0; j <= qpos; ++j) {
    const float* lj = lc + (int64_t)j * p.lat;
    const float* rj = rc + (int64_t)j * p.Hkv * p.rope;
    float lv[ME];
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < ME; ++e) { const int c = e * 32 + lane; lv[e] = (e * 32 < p.lat && c < p.lat) ? lj[c] : 0.0f; s = fmaf(qa[e], lv[e], s); }
#pragma unroll
    for (int e = 0; e < 2; ++e) { const int c = e * 32 + lane; if (c < p.rope) s = fmaf(qr[e], rj[c], s); }
    s = warp_sum(s);
    const float mn = fmaxf(mrun, s);
    const float alpha = (mrun == -INFINITY) ? 0.0f : __expf(mrun - mn);
    const float pj = __expf(s - mn);
    lrun = lrun * alpha + pj;
#pragma unroll
    for (int e = 0; e < ME; ++e) acc[e] = acc[e] * alpha + pj * lv[e];
    mrun = mn;
  }
  const float inv = lrun > 0.0f ? 1.0f / lrun : 0.0f;
  float* out = p.AL + (r * p.Hq + hq) * (int64_t)p.lat;
#pragma unroll
  for (int e = 0; e < ME; ++e) { const int c = e * 32 + lane; if (c < p.lat) out[c] = acc[e] * inv; }
}

// Tiled form of the same attention: one CTA per query row serves ALL query heads, because they all read the
// same latent rows (the latent is shared by every head; only the small rotary key differs per kv head).
// Tiles of 32 cached positions are staged in shared memory; scores: a warp owns heads w, w + 8, ...,
// lane = position; online softmax per head across tiles; P.V: thread = channel pair for every head.
// Needs latent % 4 == 0, rope % 4 == 0, latent <= 512, Hq <= 16.
constexpr int kMlaTile = 32, kMlaMaxHeads = 16;
__global__ void __launch_bounds__(256) mla_attention_tiled_kernel(MlaAttn p) {
  extern __shared__ __align__(16) float msm[];
  const int lat = p.lat, rope = p.rope, hd = lat + rope, rw = p.Hkv * rope;
  const int LDL = lat + 4, LDR = rw + 4;
  float* Ls = msm;                       // [32][LDL]   latent tile
  float* Rs = Ls + kMlaTile * LDL;       // [32][LDR]   rotary keys of every kv head
  float* Qs = Rs + kMlaTile * LDR;       // [Hq][hd]
  float* Ps = Qs + p.Hq * hd;            // [Hq][32]
  __shared__ float m_run[kMlaMaxHeads], l_run[kMlaMaxHeads], alpha_s[kMlaMaxHeads];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t r = blockIdx.x;
  const int b = (int)(r / p.T), t = (int)(r % p.T);
  const int crow = b * p.cache_row_mul;
  const int qpos = p.pos[crow] + t;
  const int ratio = p.Hq / p.Hkv;
  for (int idx = tid; idx < p.Hq * hd / 4; idx += 256) *reinterpret_cast<float4*>(Qs + idx * 4) = *reinterpret_cast<const float4*>(p.QF + r * p.Hq * (int64_t)hd + idx * 4);
  if (tid < kMlaMaxHeads) { m_run[tid] = -INFINITY; l_run[tid] = 0.0f; }
  const float* lc = p.lat_cache + (int64_t)crow * p.max_seq * lat;
  const float* rc = p.rope_cache + (int64_t)crow * p.max_seq * rw;
  int jmin = 0;
  if (p.window >= 0) jmin = max(0, qpos - p.window);
  const int cp = tid * 2;                // this thread's channel pair in the P.V phase
  float acc[kMlaMaxHeads][2];
#pragma unroll
  for (int h = 0; h < kMlaMaxHeads; ++h) { acc[h][0] = 0.0f; acc[h][1] = 0.0f; }
  for (int j0 = (jmin / kMlaTile) * kMlaTile; j0 <= qpos; j0 += kMlaTile) {
    __syncthreads();
    for (int idx = tid; idx < kMlaTile * (lat / 4); idx += 256) {
      const int jr = idx / (lat / 4), c = (idx % (lat / 4)) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j0 + jr <= qpos) v = *reinterpret_cast<const float4*>(lc + (int64_t)(j0 + jr) * lat + c);
      *reinterpret_cast<float4*>(Ls + jr * LDL + c) = v;
    }
    for (int idx = tid; idx < kMlaTile * (rw / 4); idx += 256) {
      const int jr = idx / (rw / 4), c = (idx % (rw / 4)) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j0 + jr <= qpos) v = *reinterpret_cast<const float4*>(rc + (int64_t)(j0 + jr) * rw + c);
      *reinterpret_cast<float4*>(Rs + jr * LDR + c) = v;
    }
    __syncthreads();
    for (int h = warp; h < p.Hq; h += 8) {
      const int hk = h / ratio;
      const float* q = Qs + h * hd;
      const float* lrow = Ls + lane * LDL;
      const float* rrow = Rs + lane * LDR + hk * rope;
      float d0 = 0.0f, d1 = 0.0f;
      for (int c = 0; c < lat; c += 8) {
        const float4 k0 = *reinterpret_cast<const float4*>(lrow + c), k1 = *reinterpret_cast<const float4*>(lrow + c + 4);
        const float4 q0 = *reinterpret_cast<const float4*>(q + c), q1 = *reinterpret_cast<const float4*>(q + c + 4);
        d0 = fmaf(q0.x, k0.x, d0); d0 = fmaf(q0.y, k0.y, d0); d0 = fmaf(q0.z, k0.z, d0); d0 = fmaf(q0.w, k0.w, d0);
        d1 = fmaf(q1.x, k1.x, d1); d1 = fmaf(q1.y, k1.y, d1); d1 = fmaf(q1.z, k1.z, d1); d1 = fmaf(q1.w, k1.w, d1);
      }
      for (int c = 0; c < rope; c += 4) {
        const float4 k0 = *reinterpret_cast<const float4*>(rrow + c), q0 = *reinterpret_cast<const float4*>(q + lat + c);
        d0 = fmaf(q0.x, k0.x, d0); d0 = fmaf(q0.y, k0.y, d0); d0 = fmaf(q0.z, k0.z, d0); d0 = fmaf(q0.w, k0.w, d0);
      }
      const int j = j0 + lane;
      const bool live = j <= qpos && j >= jmin;
      const float sc = live ? d0 + d1 : -INFINITY;
      float mx = sc;
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
      const float mo = m_run[h], mn = fmaxf(mo, mx);
      const float pj = live ? __expf(sc - mn) : 0.0f;
      const float tot = warp_sum(pj);
      Ps[h * kMlaTile + lane] = pj;
      __syncwarp();
      if (lane == 0) {
        const float al = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
        alpha_s[h] = al; l_run[h] = l_run[h] * al + tot; m_run[h] = mn;
      }
    }
    __syncthreads();
    if (cp < lat) {
#pragma unroll
      for (int h = 0; h < kMlaMaxHeads; ++h) if (h < p.Hq) { const float al = alpha_s[h]; acc[h][0] *= al; acc[h][1] *= al; }
      for (int jb = 0; jb < kMlaTile; jb += 4) {
        float2 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float2*>(Ls + (jb + u) * LDL + cp);
#pragma unroll
        for (int h = 0; h < kMlaMaxHeads; ++h) if (h < p.Hq) {
          const float4 p4 = *reinterpret_cast<const float4*>(Ps + h * kMlaTile + jb);
          acc[h][0] = fmaf(p4.x, v[0].x, acc[h][0]); acc[h][1] = fmaf(p4.x, v[0].y, acc[h][1]);
          acc[h][0] = fmaf(p4.y, v[1].x, acc[h][0]); acc[h][1] = fmaf(p4.y, v[1].y, acc[h][1]);
          acc[h][0] = fmaf(p4.z, v[2].x, acc[h][0]); acc[h][1] = fmaf(p4.z, v[2].y, acc[h][1]);
          acc[h][0] = fmaf(p4.w, v[3].x, acc[h][0]); acc[h][1] = fmaf(p4.w, v[3].y, acc[h][1]);
        }
      }
    }
  }
  __syncthreads();
  if (cp < lat) {
#pragma unroll
    for (int h = 0; h < kMlaMaxHeads; ++h) if (h < p.Hq) {
      const float inv = l_run[h] > 0.0f ? 1.0f / l_run[h] : 0.0f;
      *reinterpret_cast<float2*>(p.AL + (r * p.Hq + h) * (int64_t)lat + cp) = make_float2(acc[h][0] * inv, acc[h][1] * inv);
    }
  }
}
size_t mla_tiled_smem(int Hq, int Hkv, int lat, int rope) {
  return sizeof(float) * ((size_t)kMlaTile * (lat + 4) + (size_t)kMlaTile * (Hkv * rope + 4) + (size_t)Hq * (lat + rope) + (size_t)Hq * kMlaTile);
}

// ------------------------------------------------------------------ routed experts glue
// hidden[r, c] = silu(clamp_above(gate)) * clamp(up) with UG = [up | gate] per row (kernels/scalar/elementwise.go:105-134).
__global__ void __launch_bounds__(256) swiglu_rows_kernel(float* dst, const float* ug, int64_t rows, int width, float clampv) {
  const int64_t total = rows * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width; const int c = (int)(i % width);
    float u = ug[r * 2 * width + c], g = ug[r * 2 * width + width + c];
    if (clampv > 0.0f && g >= clampv) g = clampv;
    if (clampv > 0.0f) { if (u > clampv) u = clampv; else if (u < -clampv) u = -clampv; }
    const float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
    dst[i] = g * sg * u;
  }
}

// Router affinities (model/moe.go:123): logits[r, e] = x[r] . W[e]; one warp per row, the row stays in registers
// (d <= 4096) while the E weight rows stream from L1/L2.  float32 accumulation, fixed order.
__global__ void __launch_bounds__(WPB * 32) router_logits_kernel(float* logits, const float* x, const float* w, int64_t rows, int d, int E) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * WPB + warp;
  if (r >= rows) return;
  constexpr int MAXV = 32;   // float4 per lane: d <= 4096
  float4 xv[MAXV];
  const int nv = d / 128;    // d % 128 == 0 on this path
#pragma unroll
  for (int i = 0; i < MAXV; ++i) if (i < nv) xv[i] = *reinterpret_cast<const float4*>(x + r * d + (i * 32 + lane) * 4);
  for (int e = 0; e < E; ++e) {
    const float* we = w + (int64_t)e * d;
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) if (i < nv) {
      const float4 wv = *reinterpret_cast<const float4*>(we + (i * 32 + lane) * 4);
      acc = fmaf(xv[i].x, wv.x, acc); acc = fmaf(xv[i].y, wv.y, acc); acc = fmaf(xv[i].z, wv.z, acc); acc = fmaf(xv[i].w, wv.w, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) logits[r * E + e] = acc;
  }
}

// One CTA: counts per expert, then the stable expert-major position of every (row, slot) entry in
// entry order (model/moe.go:127-153).  Shared memory holds the per-expert counters and, per chunk of
// blockDim entries, the per-warp tallies that turn warp-local ranks into global ones.
constexpr int kMaxExperts = 64;
__global__ void __launch_bounds__(1024) moe_route_kernel(const int32_t* __restrict__ sel, int64_t total, int E, int32_t* __restrict__ counts,
                                                         int32_t* __restrict__ posi) {
  __shared__ int cnt[kMaxExperts], offs[kMaxExperts], running[kMaxExperts];
  __shared__ int warp_cnt[32][kMaxExperts];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  if (tid < kMaxExperts) { cnt[tid] = 0; running[tid] = 0; }
  __syncthreads();
  for (int64_t i = tid; i < total; i += blockDim.x) atomicAdd(&cnt[sel[i]], 1);
  __syncthreads();
  if (tid == 0) { int cur = 0; for (int e = 0; e < E; ++e) { offs[e] = cur; cur += cnt[e]; } }
  if (tid < E) counts[tid] = cnt[tid];
  for (int64_t base = 0; base < total; base += blockDim.x) {
    for (int k = tid; k < 32 * kMaxExperts; k += blockDim.x) (&warp_cnt[0][0])[k] = 0;
    __syncthreads();
    const int64_t i = base + tid;
    const bool live = i < total;
    const int e = live ? sel[i] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (live && rank == 0) warp_cnt[warp][e] = __popc(peers);
    __syncthreads();
    if (live) {
      int before = running[e];
      for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
      posi[i] = offs[e] + before + rank;
    }
    __syncthreads();
    if (tid < E) { int add = 0; for (int w = 0; w < nw; ++w) add += warp_cnt[w][tid]; running[tid] += add; }
    __syncthreads();
  }
}

// gathered[posi[i]] = x[i / k]   (one warp per entry); hi/lo (nullable) receive the tf32 split of the row
__global__ void __launch_bounds__(WPB * 32) moe_gather_kernel(float* gathered, float* hi, float* lo, const float* x, const int32_t* posi, int64_t total,
                                                              int k, int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t i = (int64_t)blockIdx.x * WPB + warp;
  if (i >= total) return;
  const float* src = x + (i / k) * d; const int64_t o = (int64_t)posi[i] * d;
  for (int c = lane; c < d; c += 32) {
    const float v = src[c];
    gathered[o + c] = v;
    if (hi) { float h, l; split_tf32(v, h, l); hi[o + c] = h; lo[o + c] = l; }
  }
}
// hidden = silu(clamp_above(gate)) * clamp(up) over the experts' rows, in place over gate, with the tf32 split
__global__ void __launch_bounds__(256) swiglu_split_kernel(float* gate, const float* up, float* hi, float* lo, int64_t n, float clampv) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float g = gate[i], u = up[i];
    if (clampv > 0.0f && g >= clampv) g = clampv;
    if (clampv > 0.0f) { if (u > clampv) u = clampv; else if (u < -clampv) u = -clampv; }
    const float sg = (float)(1.0 / (1.0 + exp((double)(-g))));
    const float v = g * sg * u;
    gate[i] = v;
    float h, l; split_tf32(v, h, l); hi[i] = h; lo[i] = l;
  }
}

// XOUT[r] = MID[r] + (shared[r] + routed[r]),  routed[r] = sum over the row's entries in ascending
// position of (weight * scale) * expert_out[position], each product and sum rounded (model/moe.go:160-169,
// model/block.go:41-45).
__global__ void __launch_bounds__(256) moe_combine_kernel(float* xout, const float* mid, const float* shared, const float* expert_out, const int32_t* posi,
                                                          const float* selw, float scale, int64_t rows, int k, int d) {
  const int64_t total = rows * d;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / d; const int c = (int)(i % d);
    int ps[8]; float ws[8];
    for (int s = 0; s < k; ++s) { ps[s] = posi[r * k + s]; ws[s] = __fmul_rn(selw[r * k + s], scale); }
    for (int a = 1; a < k; ++a) {   // insertion sort by position (k <= 8)
      const int pa = ps[a]; const float wa = ws[a]; int j = a - 1;
      while (j >= 0 && ps[j] > pa) { ps[j + 1] = ps[j]; ws[j + 1] = ws[j]; --j; }
      ps[j + 1] = pa; ws[j + 1] = wa;
    }
    float routed = 0.0f;
    for (int s = 0; s < k; ++s) routed = __fadd_rn(routed, __fmul_rn(ws[s], expert_out[(int64_t)ps[s] * d + c]));
    xout[i] = __fadd_rn(mid[i], __fadd_rn(shared[i], routed));
  }
}

int grid_for(int64_t n) { return (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 16)); }

}  // namespace

// Router affinities logits[r, e] = x[r] . W[e] in plain float32 (model/moe.go:123): the same kernel in inference and in
// training, so that both route alike.
int moe_router_logits(gn_model* m, int l, const float* Mn, float* RL, int64_t rows) {
  const int d = m->d, E = m->E;
  const LayerOffsets& o = m->lo[l];
  cudaStream_t s = m->s();
  if (d % 128 == 0 && d <= 4096) {
    router_logits_kernel<<<ceil_div(rows, WPB), WPB * 32, 0, s>>>(RL, Mn, m->p(o.router), rows, d, E); GN_LAUNCH_CHECK();
    return GN_OK;
  }
  GemmArgs g; g.A = Mn; g.lda = d; g.B = m->p(o.router); g.b_static = 1; g.ldb = d; g.b_trans = 1; g.C = RL; g.ldc = E; g.M = (int)rows; g.N = E; g.K = d;
  return gemm_dispatch(g, 0, s);   // E columns: the float32 kernel (routing must not depend on a split's rounding)
}
int moe_route_launch(const int32_t* sel, int64_t total, int E, int32_t* counts, int32_t* posi, cudaStream_t s) {
  moe_route_kernel<<<1, 1024, 0, s>>>(sel, total, E, counts, posi); GN_LAUNCH_CHECK();
  return GN_OK;
}

int latent_attention(gn_model* m, FwdBufs& b, const FwdArgs& a, int l, const float* H, float* O) {
  const int d = m->d, Hq = m->Hq, Hkv = m->Hkv, D = m->D, lat = m->lat, rope = m->rope, content = m->content;
  const int ratio = Hq / Hkv, hd = lat + rope;
  const int64_t rows = (int64_t)a.B * a.T;
  const int n1 = 2 * lat + (Hq + Hkv) * rope;
  const LayerOffsets& o = m->lo[l];
  const bool tc = m->ctx->gemm_kind == 1;
  cudaStream_t s = m->s();
  GN_REQUIRE(a.cache_rows > 0 && a.max_seq > 0 && m->cache_lat.p && m->cache_rope.p, "latent attention needs its cache (model/mla.go:196-198)");
  // [q_latent | kv_latent | q_rope | k_rope] = H [q_down; kv_down; q_rope; k_rope]^T
  { GemmArgs g; g.A = H; g.lda = d; g.B = m->p(o.mla_cat); g.b_static = 1; g.ldb = d; g.b_trans = 1; g.C = b.P1; g.ldc = n1; g.M = (int)rows; g.N = n1; g.K = d;
    if (tc) { g.a_hi = b.S1h; g.a_lo = b.S1l; } GN_TRY(gemm(m, g)); }
  // content queries [rows, Hq*content] = q_latent Wq_up^T
  { GemmArgs g; g.A = b.P1; g.lda = n1; g.B = m->p(o.mla_q_up); g.b_static = 1; g.ldb = lat; g.b_trans = 1; g.C = b.QC; g.ldc = (int64_t)Hq * content;
    g.M = (int)rows; g.N = Hq * content; g.K = lat; GN_TRY(gemm(m, g)); }
  // absorbed queries: QF[:, hq, 0:lat] = QC[:, hq, :] Wk_up[hk]   (Wk_up[hk] is [content, lat]; model/mla.go:232-243)
  for (int hq = 0; hq < Hq; ++hq) {
    const int hk = hq / ratio;
    GemmArgs g; g.A = b.QC + (int64_t)hq * content; g.lda = (int64_t)Hq * content; g.B = m->p(o.mla_k_up) + (int64_t)hk * content * lat; g.b_static = 1; g.ldb = lat;
    g.b_trans = 0; g.C = b.QF + (int64_t)hq * hd; g.ldc = (int64_t)Hq * hd; g.M = (int)rows; g.N = lat; g.K = content; GN_TRY(gemm(m, g));
  }
  const int64_t lat_layer = (int64_t)a.cache_rows * a.max_seq * lat, rope_layer = (int64_t)a.cache_rows * a.max_seq * Hkv * rope;
  float* lcache = m->cache_lat.f() + (int64_t)l * lat_layer; float* rcache = m->cache_rope.f() + (int64_t)l * rope_layer;
  MlaPost pp; pp.P1 = b.P1; pp.n1 = n1; pp.QF = b.QF; pp.lat_cache = lcache; pp.rope_cache = rcache; pp.cosv = m->cosb.f(); pp.sinv = m->sinb.f();
  pp.pos = m->pos.i(); pp.cache_row_mul = a.cache_row_mul; pp.max_seq = a.max_seq; pp.B = a.B; pp.T = a.T; pp.Hq = Hq; pp.Hkv = Hkv; pp.lat = lat; pp.rope = rope;
  { const int64_t n = rows * (Hq + Hkv + 1); mla_post_kernel<<<ceil_div(n, WPB), WPB * 32, 0, s>>>(pp); GN_LAUNCH_CHECK(); }
  MlaAttn pa; pa.QF = b.QF; pa.lat_cache = lcache; pa.rope_cache = rcache; pa.AL = b.AL; pa.pos = m->pos.i(); pa.cache_row_mul = a.cache_row_mul;
  pa.max_seq = a.max_seq; pa.B = a.B; pa.T = a.T; pa.Hq = Hq; pa.Hkv = Hkv; pa.lat = lat; pa.rope = rope; pa.window = m->windows[l];
  const size_t tiled_smem = mla_tiled_smem(Hq, Hkv, lat, rope);
  if (lat % 8 == 0 && rope % 4 == 0 && lat <= 512 && Hq <= kMlaMaxHeads && tiled_smem <= 200 * 1024) {
    static size_t configured = 0;
    if (tiled_smem > configured) { GN_CUDA(cudaFuncSetAttribute(mla_attention_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tiled_smem)); configured = tiled_smem; }
    mla_attention_tiled_kernel<<<(unsigned)rows, 256, tiled_smem, s>>>(pa); GN_LAUNCH_CHECK();
  } else {
    const int64_t n = rows * Hq; mla_attention_kernel<<<ceil_div(n, 4), 128, 0, s>>>(pa); GN_LAUNCH_CHECK();
  }
  // head outputs: O[:, hq, :] = AL[:, hq, :] Wv_up[hk]^T   (Wv_up[hk] is [D, lat]; model/mla.go:264-274)
  for (int hq = 0; hq < Hq; ++hq) {
    const int hk = hq / ratio;
    GemmArgs g; g.A = b.AL + (int64_t)hq * lat; g.lda = (int64_t)Hq * lat; g.B = m->p(o.mla_v_up) + (int64_t)hk * D * lat; g.b_static = 1; g.ldb = lat; g.b_trans = 1;
    g.C = O + (int64_t)hq * D; g.ldc = (int64_t)Hq * D; g.M = (int)rows; g.N = D; g.K = lat; GN_TRY(gemm(m, g));
  }
  return GN_OK;
}

int moe_ffn(gn_model* m, FwdBufs& b, const FwdArgs& a, int l, const float* Mn, const float* MID, float* XOUT) {
  const int d = m->d, E = m->E, K = m->topk, eh = m->eh, sh = m->sh;
  const int64_t rows = (int64_t)a.B * a.T, total = rows * K;
  const LayerOffsets& o = m->lo[l];
  const bool tc = m->ctx->gemm_kind == 1;
  cudaStream_t s = m->s();
  // ---- shared expert (model/mlp.go:62-76 with the SwiGLU activation): [up | gate] in one product
  { GemmArgs g; g.A = Mn; g.lda = d; g.B = m->p(o.fc); g.b_static = 1; g.ldb = d; g.b_trans = 1; g.C = b.UG; g.ldc = 2 * sh; g.M = (int)rows; g.N = 2 * sh; g.K = d;
    if (tc) { g.a_hi = b.S1h; g.a_lo = b.S1l; } GN_TRY(gemm(m, g)); }
  swiglu_rows_kernel<<<grid_for(rows * sh), 256, 0, s>>>(b.SHH, b.UG, rows, sh, m->moe_clamp); GN_LAUNCH_CHECK();
  { GemmArgs g; g.A = b.SHH; g.lda = sh; g.B = m->p(o.mproj); g.b_static = 1; g.ldb = sh; g.b_trans = 1; g.C = b.SHO; g.ldc = d; g.M = (int)rows; g.N = d; g.K = sh;
    GN_TRY(gemm(m, g)); }
  // ---- router (model/moe.go:123-124): selection on logits + bias, weights = softmax(logits) of the selected
  GN_TRY(moe_router_logits(m, l, Mn, b.RL, rows));
  GN_TRY(moe_gate_topk_launch(b.RL, m->p(o.router_bias), b.PR, b.SEL, b.SELW, (int)rows, E, K, s));
  GN_TRY(moe_route_launch(b.SEL, total, E, b.CNT, b.POSI, s));
  moe_gather_kernel<<<ceil_div(total, WPB), WPB * 32, 0, s>>>(b.GATH, tc ? b.GATHh : nullptr, tc ? b.GATHl : nullptr, Mn, b.POSI, total, K, d); GN_LAUNCH_CHECK();
  // ---- experts: grouped products over the expert-major rows (model/moe.go:155-158), on the tensor cores when the
  //      expert shapes allow it (each 128-row tile of an expert is one CTA; rows past an expert's last are masked)
  const int kind = m->ctx->gemm_kind;
  auto grouped = [&](const float* A, const float* Ah, const float* Al, int64_t w_off, float* C, int n, int k) -> int {
    GemmArgs g; g.A = A; g.lda = k; g.B = m->p(w_off); g.b_static = 1; g.ldb = k; g.b_trans = 1; g.C = C; g.ldc = n; g.M = (int)total; g.N = n; g.K = k;
    g.group_counts = b.CNT; g.groups = E; if (tc) { g.a_hi = Ah; g.a_lo = Al; }
    return gemm_grouped_dispatch(g, kind, s);
  };
  GN_TRY(grouped(b.GATH, b.GATHh, b.GATHl, o.exp_gate, b.GG, eh, d));
  GN_TRY(grouped(b.GATH, b.GATHh, b.GATHl, o.exp_up, b.GU, eh, d));
  swiglu_split_kernel<<<grid_for(total * eh), 256, 0, s>>>(b.GG, b.GU, b.GHh, b.GHl, total * eh, m->moe_clamp); GN_LAUNCH_CHECK();
  GN_TRY(grouped(b.GG, b.GHh, b.GHl, o.exp_down, b.GO, d, eh));
  moe_combine_kernel<<<grid_for(rows * d), 256, 0, s>>>(XOUT, MID, b.SHO, b.GO, b.POSI, b.SELW, m->moe_scale, rows, K, d); GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gnm
