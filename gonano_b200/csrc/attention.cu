// Attention kernels (kernels/backend.go:167-283; scalar statement
// kernels/scalar/attention.go:16-245).
//
//   attention_forward   tiled online-softmax attention over token-major,
//                       strided Q/K/V (all (batch, head) pairs in one launch);
//                       used by prefill, by the training forward and by the
//                       single-head conformance entry point.
//   attention_backward  two deterministic kernels: one CTA per key tile for
//                       dK/dV (it also walks the query heads that share the
//                       kv head, so grouped-query gradients need no atomics),
//                       one CTA per query tile for dQ.
//   attention_decode    one query token per row over the KV cache: warp-level
//                       online softmax, float4 coalesced K/V loads, optional
//                       split over the key range with a combine pass.
//   attention_split / attention_combine  the contract's split-K pair.
//
// Scores are raw q.k (the model applies no 1/sqrt(d)); a masked score is the
// finite -1e30 of the reference (kernels/scalar/attention.go:11).
#include <cstdlib>

#include <atomic>

#include "kernels.cuh"

namespace gn {

constexpr float kMaskedScore = -1e30f;
constexpr int AT = 256;  // threads per CTA in the tiled kernels

// head_dim 128 fast path (defined further down)
static bool fast128_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4);
static int attn_fwd128_go(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s);
static int attn_bwd128_go(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                          float* dq, float* dk, float* dv, int accumulate, cudaStream_t s);

__device__ __forceinline__ bool attn_masked(int qpos, int kj, int window, const int32_t* seg, int seg_len, int32_t qseg) {
  bool m = kj > qpos || (window >= 0 && qpos - kj > window);
  if (!m && seg != nullptr && kj < seg_len && seg[kj] != qseg) m = true;
  return m;
}

// acc[TM][TN] += sum_k A[k][m..m+TM) * B[k][n..n+TN), A and B shared-memory
// tiles stored k-major with row pitches lda / ldb (multiples of 4 floats).
template <int TM, int TN>
__device__ __forceinline__ void mm_acc(float (&acc)[TM][TN], const float* A, int lda, const float* B, int ldb, int K, int m, int n) {
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    float a[TM], b[TN];
    if (TM == 8) {
      float4 v = *reinterpret_cast<const float4*>(A + k * lda + m), w = *reinterpret_cast<const float4*>(A + k * lda + m + 4);
      a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; a[4 % TM] = w.x; a[5 % TM] = w.y; a[6 % TM] = w.z; a[7 % TM] = w.w;
    }
    else if (TM == 4) { float4 v = *reinterpret_cast<const float4*>(A + k * lda + m); a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
    else if (TM == 2) { float2 v = *reinterpret_cast<const float2*>(A + k * lda + m); a[0] = v.x; a[1] = v.y; }
    else { for (int i = 0; i < TM; ++i) a[i] = A[k * lda + m + i]; }
    if (TN == 4) { float4 v = *reinterpret_cast<const float4*>(B + k * ldb + n); b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w; }
    else if (TN == 2) { float2 v = *reinterpret_cast<const float2*>(B + k * ldb + n); b[0] = v.x; b[1] = v.y; }
    else { for (int j = 0; j < TN; ++j) b[j] = B[k * ldb + n + j]; }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// Copies `nrows` token rows of D floats (pitch `tstride` in global memory) into
// shared memory, zero-filling rows >= valid and columns >= D up to DP.
//   row-major:  S[r*ld + c]        transposed: S[c*ld + r]
template <int DP, bool TRANSPOSED>
__device__ __forceinline__ void load_tile(float* S, int ld, const float* g, int64_t tstride, int nrows, int valid, int D) {
  for (int idx = threadIdx.x; idx < nrows * DP; idx += AT) {
    int r = idx / DP, c = idx % DP;
    float v = (r < valid && c < D) ? g[(int64_t)r * tstride + c] : 0.0f;
    if (TRANSPOSED) S[c * ld + r] = v; else S[r * ld + c] = v;
  }
}

// ============================================================== forward
// CTA: 64 queries of one (batch, query head); loops over 64-key tiles.
template <int DP>
__global__ void __launch_bounds__(AT) attn_fwd_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                      float* __restrict__ out, float* __restrict__ lse) {
  constexpr int BQ = 64, BKV = 64, LQ = BQ + 4, LV = DP + 4;
  constexpr int NG = (DP == 128) ? 2 : 1;      // column groups of the output tile per thread
  constexpr int TN = (DP == 32) ? 2 : 4;       // output columns per group per thread
  extern __shared__ __align__(16) float smem[];
  float* Qt = smem;                  // [DP][LQ]
  float* Kt = Qt + DP * LQ;          // [DP][LQ]
  float* Vs = Kt + DP * LQ;          // [BKV][LV]
  float* Pt = Vs + BKV * LV;         // [BKV][LQ]   P transposed: Pt[j][i]

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / sh.Hq, hq = bh % sh.Hq, hk = hq / (sh.Hq / sh.Hkv);
  const int q0 = blockIdx.x * BQ;
  const int qvalid = min(BQ, sh.Tq - q0);
  const int offset = sh.offset0;

  const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * sh.D;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  load_tile<DP, true>(Qt, LQ, qg, sh.q_tstride, BQ, qvalid, sh.D);

  float m_run[4], l_run[4], o[NG][4][TN];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -INFINITY; l_run[i] = 0.0f;
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int j = 0; j < TN; ++j) o[g][i][j] = 0.0f;
  }
  int32_t qseg[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int qpos = offset + q0 + ty * 4 + i;
    qseg[i] = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
  }
  // The reference keeps the last seen query segment when the position runs past
  // the segment array; positions here never do for valid rows.

  // Key range that any query of this tile can see.
  const int max_qpos = offset + q0 + qvalid - 1;
  int k_end = min(sh.Tk, max_qpos + 1);
  int k_begin = 0;
  if (sh.window >= 0) k_begin = max(0, offset + q0 - sh.window);
  k_begin = (k_begin / BKV) * BKV;

  for (int kt = k_begin; kt < k_end; kt += BKV) {
    const int kvalid = min(BKV, sh.Tk - kt);
    __syncthreads();
    load_tile<DP, true>(Kt, LQ, kg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid, sh.D);
    load_tile<DP, false>(Vs, LV, vg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid, sh.D);
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
    mm_acc<4, 4>(s, Qt, LQ, Kt, LQ, DP, ty * 4, tx * 4);
    // mask, row max over the 16 threads that share the rows
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int qpos = offset + q0 + ty * 4 + i;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int kj = kt + tx * 4 + j;
        if (kj >= sh.Tk) s[i][j] = -INFINITY;   // beyond the key array: contributes nothing
        else if (attn_masked(qpos, kj, sh.window, sh.segment_ids, sh.seg_len, qseg[i])) s[i][j] = kMaskedScore;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
      float m_new = fmaxf(m_run[i], mx);
      float alpha = (m_run[i] == -INFINITY) ? 0.0f : __expf(m_run[i] - m_new);
      float rs = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float p = (s[i][j] == -INFINITY) ? 0.0f : __expf(s[i][j] - m_new);
        s[i][j] = p; rs += p;
      }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o2);
      l_run[i] = l_run[i] * alpha + rs;
      m_run[i] = m_new;
#pragma unroll
      for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int j = 0; j < TN; ++j) o[g][i][j] *= alpha;
#pragma unroll
      for (int j = 0; j < 4; ++j) Pt[(tx * 4 + j) * LQ + ty * 4 + i] = s[i][j];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < NG; ++g) mm_acc<4, TN>(o[g], Pt, LQ, Vs, LV, BKV, ty * 4, g * 64 + tx * TN);
  }
  // write out
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int qi = q0 + ty * 4 + i;
    if (qi >= sh.Tq) continue;
    float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
    float* og = out + (int64_t)b * sh.o_bstride + (int64_t)qi * sh.o_tstride + (int64_t)hq * sh.D;
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        int c = g * 64 + tx * TN + j;
        if (c < sh.D) og[c] = o[g][i][j] * inv;
      }
    if (lse && tx == 0) lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] = m_run[i] + logf(l_run[i]);
  }
}

template <int DP>
static int attn_fwd_go(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s) {
  constexpr int LQ = 68, LV = DP + 4;
  size_t smem = sizeof(float) * (size_t)(2 * DP * LQ + 64 * LV + 64 * LQ);
  static PerDeviceOnce configured;
  if (configured.first()) {
    GN_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  dim3 grid(ceil_div(sh.Tq, 64), sh.B * sh.Hq);
  attn_fwd_kernel<DP><<<grid, AT, smem, s>>>(sh, q, k, v, out, lse);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int attention_forward_launch(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s) {
  if (sh.Tq <= 0 || sh.B <= 0) return GN_OK;
  GN_REQUIRE(sh.D > 0 && sh.D <= 128, "attention: head_dim %d outside (0,128]", sh.D);
  GN_REQUIRE(sh.Hkv > 0 && sh.Hq % sh.Hkv == 0, "attention: %d query heads not divisible by %d kv heads", sh.Hq, sh.Hkv);
#ifdef GN_HAVE_TCGEN05
  if (sh.tensor && attention_tc_ok(sh, q, k, v, out)) return attention_tc_forward(sh, q, k, v, out, lse, s);
#endif
  if (sh.tensor && attention_mma_ok(sh, q, k, v, out, nullptr)) return attention_mma_forward(sh, q, k, v, out, lse, s);
  if (fast128_ok(sh, q, k, v, out, nullptr)) return attn_fwd128_go(sh, q, k, v, out, lse, s);
  if (sh.D <= 32) return attn_fwd_go<32>(sh, q, k, v, out, lse, s);
  if (sh.D <= 64) return attn_fwd_go<64>(sh, q, k, v, out, lse, s);
  return attn_fwd_go<128>(sh, q, k, v, out, lse, s);
}

// ============================================================== head_dim 128 fast path
// The model's head width.  Same algorithm as the generic kernels above, retiled so that the
// inner products are FMA-bound instead of shared-memory-bound: 8x4 / 4x4 register tiles fed by
// broadcast float4 reads, transposed tiles written with lane = row (conflict-free), and in the
// backward kernels the probability tiles alias the transposed Q / dO (or V) tiles once those
// have been consumed, which is what lets 64x64 tiles fit in shared memory.
constexpr int FD = 128;

// rows of FD floats -> transposed St[c][r]; consecutive lanes take consecutive rows.
__device__ __forceinline__ void load_rows_T(float* St, int ld, const float* g, int64_t tstride, int nrows, int valid) {
  for (int idx = threadIdx.x; idx < nrows * (FD / 4); idx += AT) {
    const int r = idx % nrows, c = (idx / nrows) * 4;
    float4 v = make_float4(0, 0, 0, 0);
    if (r < valid) v = *reinterpret_cast<const float4*>(g + (int64_t)r * tstride + c);
    St[(c + 0) * ld + r] = v.x; St[(c + 1) * ld + r] = v.y; St[(c + 2) * ld + r] = v.z; St[(c + 3) * ld + r] = v.w;
  }
}
// rows of FD floats -> row-major S[r][c], float4 coalesced.
__device__ __forceinline__ void load_rows(float* S, int ld, const float* g, int64_t tstride, int nrows, int valid) {
  for (int idx = threadIdx.x; idx < nrows * (FD / 4); idx += AT) {
    const int r = idx / (FD / 4), c = (idx % (FD / 4)) * 4;
    float4 v = make_float4(0, 0, 0, 0);
    if (r < valid) v = *reinterpret_cast<const float4*>(g + (int64_t)r * tstride + c);
    *reinterpret_cast<float4*>(S + r * ld + c) = v;
  }
}

// Forward: CTA = 128 queries of one (batch, head); 64-key tiles.
__global__ void __launch_bounds__(AT, 1) attn_fwd128_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k,
                                                            const float* __restrict__ v, float* __restrict__ out, float* __restrict__ lse) {
  constexpr int BQ = 128, BKV = 64, LQ = BQ + 4, LK = BKV + 4, LV = FD + 4;
  extern __shared__ __align__(16) float smem[];
  float* Qt = smem;               // [FD][LQ]
  float* Kt = Qt + FD * LQ;       // [FD][LK]
  float* Vs = Kt + FD * LK;       // [BKV][LV]
  float* Pt = Vs + BKV * LV;      // [BKV][LQ]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / sh.Hq, hq = bh % sh.Hq, hk = hq / (sh.Hq / sh.Hkv);
  const int q0 = blockIdx.x * BQ, qvalid = min(BQ, sh.Tq - q0), offset = sh.offset0;
  const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * FD;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  load_rows_T(Qt, LQ, qg, sh.q_tstride, BQ, qvalid);
  float m_run[8], l_run[8], o[2][8][4];
  int32_t qseg[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    m_run[i] = -INFINITY; l_run[i] = 0.0f;
    const int qpos = offset + q0 + ty * 8 + i;
    qseg[i] = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
#pragma unroll
    for (int g = 0; g < 2; ++g)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[g][i][j] = 0.0f;
  }
  const int max_qpos = offset + q0 + qvalid - 1;
  const int k_end = min(sh.Tk, max_qpos + 1);
  int k_begin = 0;
  if (sh.window >= 0) k_begin = max(0, offset + q0 - sh.window);
  k_begin = (k_begin / BKV) * BKV;
  for (int kt = k_begin; kt < k_end; kt += BKV) {
    const int kvalid = min(BKV, sh.Tk - kt);
    __syncthreads();
    load_rows_T(Kt, LK, kg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid);
    load_rows(Vs, LV, vg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid);
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
    mm_acc<8, 4>(s, Qt, LQ, Kt, LK, FD, ty * 8, tx * 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int qpos = offset + q0 + ty * 8 + i;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = kt + tx * 4 + j;
        if (kj >= sh.Tk) s[i][j] = -INFINITY;
        else if (attn_masked(qpos, kj, sh.window, sh.segment_ids, sh.seg_len, qseg[i])) s[i][j] = kMaskedScore;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
      const float m_new = fmaxf(m_run[i], mx);
      const float alpha = (m_run[i] == -INFINITY) ? 0.0f : __expf(m_run[i] - m_new);
      float rs = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float p = (s[i][j] == -INFINITY) ? 0.0f : __expf(s[i][j] - m_new); s[i][j] = p; rs += p; }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o2);
      l_run[i] = l_run[i] * alpha + rs;
      m_run[i] = m_new;
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[g][i][j] *= alpha;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float* dst = Pt + (tx * 4 + j) * LQ + ty * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(s[0][j], s[1][j], s[2][j], s[3][j]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(s[4][j], s[5][j], s[6][j], s[7][j]);
    }
    __syncthreads();
    mm_acc<8, 4>(o[0], Pt, LQ, Vs, LV, BKV, ty * 8, tx * 4);
    mm_acc<8, 4>(o[1], Pt, LQ, Vs, LV, BKV, ty * 8, 64 + tx * 4);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int qi = q0 + ty * 8 + i;
    if (qi >= sh.Tq) continue;
    const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
    float* og = out + (int64_t)b * sh.o_bstride + (int64_t)qi * sh.o_tstride + (int64_t)hq * FD;
#pragma unroll
    for (int g = 0; g < 2; ++g)
      *reinterpret_cast<float4*>(og + g * 64 + tx * 4) = make_float4(o[g][i][0] * inv, o[g][i][1] * inv, o[g][i][2] * inv, o[g][i][3] * inv);
    if (lse && tx == 0) lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] = m_run[i] + logf(l_run[i]);
  }
}

// dK/dV: CTA = 64 keys of one (batch, kv head); walks the group's query heads and 64-query tiles.
__global__ void __launch_bounds__(AT, 1) attn_bwd128_dkv_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k,
                                                                const float* __restrict__ v, const float* __restrict__ dout,
                                                                const float* __restrict__ lse, const float* __restrict__ delta,
                                                                float* __restrict__ dk, float* __restrict__ dv, int accumulate) {
  constexpr int BQ = 64, BKV = 64, LT = 68, LD = FD + 4;
  extern __shared__ __align__(16) float smem[];
  float* Kt = smem;               // [FD][LT]
  float* Vt = Kt + FD * LT;       // [FD][LT]
  float* Qt = Vt + FD * LT;       // [FD][LT]   reused as Ps [BQ][LT] once S is formed
  float* dOt = Qt + FD * LT;      // [FD][LT]   reused as dSs [BQ][LT]
  float* Qs = dOt + FD * LT;      // [BQ][LD]
  float* dOs = Qs + BQ * LD;      // [BQ][LD]
  float* Ps = Qt; float* dSs = dOt;
  __shared__ float lse_s[BQ], delta_s[BQ];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / sh.Hkv, hk = bh % sh.Hkv, ratio = sh.Hq / sh.Hkv;
  const int k0 = blockIdx.x * BKV, kvalid = min(BKV, sh.Tk - k0), offset = sh.offset0;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)k0 * sh.kv_tstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)k0 * sh.kv_tstride;
  load_rows_T(Kt, LT, kg, sh.kv_tstride, BKV, kvalid);
  load_rows_T(Vt, LT, vg, sh.kv_tstride, BKV, kvalid);
  float adk[2][4][4], adv[2][4][4];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { adk[g][i][j] = 0.0f; adv[g][i][j] = 0.0f; }
  int q_begin = max(0, k0 - offset);
  q_begin = (q_begin / BQ) * BQ;
  int q_end = sh.Tq;
  if (sh.window >= 0) q_end = min(sh.Tq, k0 + kvalid - 1 + sh.window - offset + 1);
  for (int h = 0; h < ratio; ++h) {
    const int hq = hk * ratio + h;
    for (int q0 = q_begin; q0 < q_end; q0 += BQ) {
      const int qvalid = min(BQ, sh.Tq - q0);
      const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * FD;
      const float* dog = dout + (int64_t)b * sh.o_bstride + (int64_t)q0 * sh.o_tstride + (int64_t)hq * FD;
      __syncthreads();
      load_rows_T(Qt, LT, qg, sh.q_tstride, BQ, qvalid);
      load_rows_T(dOt, LT, dog, sh.o_tstride, BQ, qvalid);
      load_rows(Qs, LD, qg, sh.q_tstride, BQ, qvalid);
      load_rows(dOs, LD, dog, sh.o_tstride, BQ, qvalid);
      if (tid < BQ) {
        const int qi = q0 + tid;
        lse_s[tid] = qi < sh.Tq ? lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
        delta_s[tid] = qi < sh.Tq ? delta[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
      }
      __syncthreads();
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { s[i][j] = 0.0f; dp[i][j] = 0.0f; }
      mm_acc<4, 4>(s, Qt, LT, Kt, LT, FD, ty * 4, tx * 4);
      mm_acc<4, 4>(dp, dOt, LT, Vt, LT, FD, ty * 4, tx * 4);
      __syncthreads();   // Qt / dOt are consumed: their memory now holds P and dS
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int il = ty * 4 + i, qi = q0 + il, qpos = offset + qi;
        const int32_t qseg = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
        float pv[4], dsv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kj = k0 + tx * 4 + j;
          float p = 0.0f;
          if (qi < sh.Tq && kj < sh.Tk && !attn_masked(qpos, kj, sh.window, sh.segment_ids, sh.seg_len, qseg)) p = __expf(s[i][j] - lse_s[il]);
          pv[j] = p; dsv[j] = p * (dp[i][j] - delta_s[il]);
        }
        *reinterpret_cast<float4*>(Ps + il * LT + tx * 4) = make_float4(pv[0], pv[1], pv[2], pv[3]);
        *reinterpret_cast<float4*>(dSs + il * LT + tx * 4) = make_float4(dsv[0], dsv[1], dsv[2], dsv[3]);
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        mm_acc<4, 4>(adv[g], Ps, LT, dOs, LD, BQ, ty * 4, g * 64 + tx * 4);
        mm_acc<4, 4>(adk[g], dSs, LT, Qs, LD, BQ, ty * 4, g * 64 + tx * 4);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kj = k0 + ty * 4 + i;
    if (kj >= sh.Tk) continue;
    float* dkg = dk + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)kj * sh.kv_tstride;
    float* dvg = dv + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)kj * sh.kv_tstride;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float4 a = make_float4(adk[g][i][0], adk[g][i][1], adk[g][i][2], adk[g][i][3]);
      float4 c = make_float4(adv[g][i][0], adv[g][i][1], adv[g][i][2], adv[g][i][3]);
      float4* pk = reinterpret_cast<float4*>(dkg + g * 64 + tx * 4); float4* pv = reinterpret_cast<float4*>(dvg + g * 64 + tx * 4);
      if (accumulate) { float4 ok = *pk, ov = *pv; a.x += ok.x; a.y += ok.y; a.z += ok.z; a.w += ok.w; c.x += ov.x; c.y += ov.y; c.z += ov.z; c.w += ov.w; }
      *pk = a; *pv = c;
    }
  }
}

// dQ: CTA = 64 queries of one (batch, query head); walks 64-key tiles.
__global__ void __launch_bounds__(AT, 1) attn_bwd128_dq_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k,
                                                               const float* __restrict__ v, const float* __restrict__ dout,
                                                               const float* __restrict__ lse, const float* __restrict__ delta,
                                                               float* __restrict__ dq, int accumulate) {
  constexpr int BQ = 64, BKV = 64, LT = 68, LD = FD + 4;
  extern __shared__ __align__(16) float smem[];
  float* Qt = smem;               // [FD][LT]
  float* dOt = Qt + FD * LT;      // [FD][LT]
  float* Kt = dOt + FD * LT;      // [FD][LT]
  float* Vt = Kt + FD * LT;       // [FD][LT]   reused as dSt [BKV][LT] once dP is formed
  float* Ks = Vt + FD * LT;       // [BKV][LD]
  float* dSt = Vt;
  __shared__ float lse_s[BQ], delta_s[BQ];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / sh.Hq, hq = bh % sh.Hq, hk = hq / (sh.Hq / sh.Hkv);
  const int q0 = blockIdx.x * BQ, qvalid = min(BQ, sh.Tq - q0), offset = sh.offset0;
  const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * FD;
  const float* dog = dout + (int64_t)b * sh.o_bstride + (int64_t)q0 * sh.o_tstride + (int64_t)hq * FD;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  load_rows_T(Qt, LT, qg, sh.q_tstride, BQ, qvalid);
  load_rows_T(dOt, LT, dog, sh.o_tstride, BQ, qvalid);
  if (tid < BQ) {
    const int qi = q0 + tid;
    lse_s[tid] = qi < sh.Tq ? lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
    delta_s[tid] = qi < sh.Tq ? delta[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
  }
  float adq[2][4][4];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) adq[g][i][j] = 0.0f;
  const int max_qpos = offset + q0 + qvalid - 1;
  const int k_end = min(sh.Tk, max_qpos + 1);
  int k_begin = 0;
  if (sh.window >= 0) k_begin = max(0, offset + q0 - sh.window);
  k_begin = (k_begin / BKV) * BKV;
  for (int kt = k_begin; kt < k_end; kt += BKV) {
    const int kvalid = min(BKV, sh.Tk - kt);
    __syncthreads();
    load_rows_T(Kt, LT, kg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid);
    load_rows_T(Vt, LT, vg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid);
    load_rows(Ks, LD, kg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid);
    __syncthreads();
    float s[4][4], dp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { s[i][j] = 0.0f; dp[i][j] = 0.0f; }
    mm_acc<4, 4>(s, Qt, LT, Kt, LT, FD, ty * 4, tx * 4);
    mm_acc<4, 4>(dp, dOt, LT, Vt, LT, FD, ty * 4, tx * 4);
    __syncthreads();   // Vt is consumed: its memory now holds dS transposed
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kj = kt + tx * 4 + j;
      float dsv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int il = ty * 4 + i, qi = q0 + il, qpos = offset + qi;
        const int32_t qseg = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
        float p = 0.0f;
        if (qi < sh.Tq && kj < sh.Tk && !attn_masked(qpos, kj, sh.window, sh.segment_ids, sh.seg_len, qseg)) p = __expf(s[i][j] - lse_s[il]);
        dsv[i] = p * (dp[i][j] - delta_s[il]);
      }
      *reinterpret_cast<float4*>(dSt + (tx * 4 + j) * LT + ty * 4) = make_float4(dsv[0], dsv[1], dsv[2], dsv[3]);
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < 2; ++g) mm_acc<4, 4>(adq[g], dSt, LT, Ks, LD, BKV, ty * 4, g * 64 + tx * 4);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qi = q0 + ty * 4 + i;
    if (qi >= sh.Tq) continue;
    float* dqg = dq + (int64_t)b * sh.q_bstride + (int64_t)qi * sh.q_tstride + (int64_t)hq * FD;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float4 a = make_float4(adq[g][i][0], adq[g][i][1], adq[g][i][2], adq[g][i][3]);
      float4* pq = reinterpret_cast<float4*>(dqg + g * 64 + tx * 4);
      if (accumulate) { float4 o4 = *pq; a.x += o4.x; a.y += o4.y; a.z += o4.z; a.w += o4.w; }
      *pq = a;
    }
  }
}

// float4 row access needs 16-byte aligned rows.
static bool fast128_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return sh.D == FD && al(p0) && al(p1) && al(p2) && al(p3) && al(p4) && sh.q_tstride % 4 == 0 && sh.q_bstride % 4 == 0 && sh.kv_tstride % 4 == 0 &&
         sh.kv_bstride % 4 == 0 && sh.kv_hstride % 4 == 0 && sh.o_tstride % 4 == 0 && sh.o_bstride % 4 == 0;
}

static int attn_fwd128_go(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s) {
  const size_t smem = sizeof(float) * (size_t)(FD * 132 + FD * 68 + 64 * 132 + 64 * 132);
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(attn_fwd128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); }
  dim3 grid(ceil_div(sh.Tq, 128), sh.B * sh.Hq);
  attn_fwd128_kernel<<<grid, AT, smem, s>>>(sh, q, k, v, out, lse);
  GN_LAUNCH_CHECK();
  return GN_OK;
}
static int attn_bwd128_go(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                          float* dq, float* dk, float* dv, int accumulate, cudaStream_t s) {
  const size_t smem_kv = sizeof(float) * (size_t)(4 * FD * 68 + 2 * 64 * 132);
  const size_t smem_q = sizeof(float) * (size_t)(4 * FD * 68 + 64 * 132);
  static PerDeviceOnce configured;
  if (configured.first()) {
    GN_CUDA(cudaFuncSetAttribute(attn_bwd128_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
    GN_CUDA(cudaFuncSetAttribute(attn_bwd128_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
  }
  dim3 gkv(ceil_div(sh.Tk, 64), sh.B * sh.Hkv);
  attn_bwd128_dkv_kernel<<<gkv, AT, smem_kv, s>>>(sh, q, k, v, dout, lse, delta, dk, dv, accumulate);
  GN_LAUNCH_CHECK();
  dim3 gq(ceil_div(sh.Tq, 64), sh.B * sh.Hq);
  attn_bwd128_dq_kernel<<<gq, AT, smem_q, s>>>(sh, q, k, v, dout, lse, delta, dq, accumulate);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ============================================================== backward
// delta[b,hq,i] = sum_c dO[i][c] * O[i][c]  (equals sum_j P_ij dP_ij).
__global__ void __launch_bounds__(256) attn_delta_kernel(AttnShape sh, const float* out, const float* dout, float* delta) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  int64_t total = (int64_t)sh.B * sh.Hq * sh.Tq;
  if (idx >= total) return;
  int i = (int)(idx % sh.Tq); int bh = (int)(idx / sh.Tq); int b = bh / sh.Hq, hq = bh % sh.Hq;
  const float* o = out + (int64_t)b * sh.o_bstride + (int64_t)i * sh.o_tstride + (int64_t)hq * sh.D;
  const float* d = dout + (int64_t)b * sh.o_bstride + (int64_t)i * sh.o_tstride + (int64_t)hq * sh.D;
  float acc = 0;
  for (int c = lane; c < sh.D; c += 32) acc = fmaf(o[c], d[c], acc);
  acc = warp_sum(acc);
  if (lane == 0) delta[idx] = acc;
}

// dK/dV: CTA = 64 keys of one (batch, kv head).  Walks the query heads of the
// group and 32-query tiles.  dOut/out use the o_* strides, dq the q strides.
template <int DP>
__global__ void __launch_bounds__(AT) attn_bwd_dkv_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                          const float* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta,
                                                          float* __restrict__ dk, float* __restrict__ dv, int accumulate) {
  constexpr int BQ = 32, BKV = 64, LK = BKV + 4, LQ = BQ + 4, LD = DP + 4;
  constexpr int NG = (DP == 128) ? 2 : 1;
  constexpr int TN = (DP == 32) ? 2 : 4;
  extern __shared__ __align__(16) float smem[];
  float* Kt = smem;                   // [DP][LK]
  float* Vt = Kt + DP * LK;           // [DP][LK]
  float* Qt = Vt + DP * LK;           // [DP][LQ]
  float* dOt = Qt + DP * LQ;          // [DP][LQ]
  float* Qs = dOt + DP * LQ;          // [BQ][LD]
  float* dOs = Qs + BQ * LD;          // [BQ][LD]
  float* Ps = dOs + BQ * LD;          // [BQ][LK]   P[i][j]
  float* dSs = Ps + BQ * LK;          // [BQ][LK]
  __shared__ float lse_s[BQ], delta_s[BQ];

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / sh.Hkv, hk = bh % sh.Hkv;
  const int ratio = sh.Hq / sh.Hkv;
  const int k0 = blockIdx.x * BKV;
  const int kvalid = min(BKV, sh.Tk - k0);
  const int offset = sh.offset0;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)k0 * sh.kv_tstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)k0 * sh.kv_tstride;
  load_tile<DP, true>(Kt, LK, kg, sh.kv_tstride, BKV, kvalid, sh.D);
  load_tile<DP, true>(Vt, LK, vg, sh.kv_tstride, BKV, kvalid, sh.D);

  // accumulators: keys ty*4..+3, columns g*64 + tx*TN ..
  float adk[NG][4][TN], adv[NG][4][TN];
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) { adk[g][i][j] = 0.0f; adv[g][i][j] = 0.0f; }

  // queries that can see any key of this tile: qpos >= k0  and qpos - (k0+kvalid-1) <= window ... per-element masks decide.
  int q_begin = max(0, k0 - offset);
  q_begin = (q_begin / BQ) * BQ;
  int q_end = sh.Tq;
  if (sh.window >= 0) q_end = min(sh.Tq, k0 + kvalid - 1 + sh.window - offset + 1);

  for (int h = 0; h < ratio; ++h) {
    const int hq = hk * ratio + h;
    for (int q0 = q_begin; q0 < q_end; q0 += BQ) {
      const int qvalid = min(BQ, sh.Tq - q0);
      const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * sh.D;
      const float* dog = dout + (int64_t)b * sh.o_bstride + (int64_t)q0 * sh.o_tstride + (int64_t)hq * sh.D;
      __syncthreads();
      load_tile<DP, true>(Qt, LQ, qg, sh.q_tstride, BQ, qvalid, sh.D);
      load_tile<DP, false>(Qs, LD, qg, sh.q_tstride, BQ, qvalid, sh.D);
      load_tile<DP, true>(dOt, LQ, dog, sh.o_tstride, BQ, qvalid, sh.D);
      load_tile<DP, false>(dOs, LD, dog, sh.o_tstride, BQ, qvalid, sh.D);
      if (tid < BQ) {
        int qi = q0 + tid;
        lse_s[tid] = qi < sh.Tq ? lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
        delta_s[tid] = qi < sh.Tq ? delta[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
      }
      __syncthreads();
      // S and dP tiles: 32 x 64, thread = rows ty*2..+1, cols tx*4..+3
      float s[2][4], dp[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { s[i][j] = 0.0f; dp[i][j] = 0.0f; }
      mm_acc<2, 4>(s, Qt, LQ, Kt, LK, DP, ty * 2, tx * 4);
      mm_acc<2, 4>(dp, dOt, LQ, Vt, LK, DP, ty * 2, tx * 4);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        int il = ty * 2 + i, qi = q0 + il, qpos = offset + qi;
        int32_t qseg = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int kj = k0 + tx * 4 + j;
          float p = 0.0f;
          if (qi < sh.Tq && kj < sh.Tk && !attn_masked(qpos, kj, sh.window, sh.segment_ids, sh.seg_len, qseg)) p = __expf(s[i][j] - lse_s[il]);
          Ps[il * LK + tx * 4 + j] = p;
          dSs[il * LK + tx * 4 + j] = p * (dp[i][j] - delta_s[il]);
        }
      }
      __syncthreads();
      // dV[j][c] += sum_i P[i][j] dO[i][c] ; dK[j][c] += sum_i dS[i][j] Q[i][c]
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        mm_acc<4, TN>(adv[g], Ps, LK, dOs, LD, BQ, ty * 4, g * 64 + tx * TN);
        mm_acc<4, TN>(adk[g], dSs, LK, Qs, LD, BQ, ty * 4, g * 64 + tx * TN);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int kj = k0 + ty * 4 + i;
    if (kj >= sh.Tk) continue;
    float* dkg = dk + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)kj * sh.kv_tstride;
    float* dvg = dv + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)kj * sh.kv_tstride;
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        int c = g * 64 + tx * TN + j;
        if (c < sh.D) {
          if (accumulate) { dkg[c] += adk[g][i][j]; dvg[c] += adv[g][i][j]; }
          else { dkg[c] = adk[g][i][j]; dvg[c] = adv[g][i][j]; }
        }
      }
  }
}

// dQ: CTA = 64 queries of one (batch, query head); walks 32-key tiles.
template <int DP>
__global__ void __launch_bounds__(AT) attn_bwd_dq_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                         const float* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta,
                                                         float* __restrict__ dq, int accumulate) {
  constexpr int BQ = 64, BKV = 32, LQ = BQ + 4, LK = BKV + 4, LD = DP + 4;
  constexpr int NG = (DP == 128) ? 2 : 1;
  constexpr int TN = (DP == 32) ? 2 : 4;
  extern __shared__ __align__(16) float smem[];
  float* Qt = smem;                   // [DP][LQ]
  float* dOt = Qt + DP * LQ;          // [DP][LQ]
  float* Kt = dOt + DP * LQ;          // [DP][LK]
  float* Vt = Kt + DP * LK;           // [DP][LK]
  float* Ks = Vt + DP * LK;           // [BKV][LD]
  float* dSt = Ks + BKV * LD;         // [BKV][LQ]  dS transposed: dSt[j][i]
  __shared__ float lse_s[BQ], delta_s[BQ];

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int bh = blockIdx.y, b = bh / sh.Hq, hq = bh % sh.Hq, hk = hq / (sh.Hq / sh.Hkv);
  const int q0 = blockIdx.x * BQ;
  const int qvalid = min(BQ, sh.Tq - q0);
  const int offset = sh.offset0;
  const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * sh.D;
  const float* dog = dout + (int64_t)b * sh.o_bstride + (int64_t)q0 * sh.o_tstride + (int64_t)hq * sh.D;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  load_tile<DP, true>(Qt, LQ, qg, sh.q_tstride, BQ, qvalid, sh.D);
  load_tile<DP, true>(dOt, LQ, dog, sh.o_tstride, BQ, qvalid, sh.D);
  if (tid < BQ) {
    int qi = q0 + tid;
    lse_s[tid] = qi < sh.Tq ? lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
    delta_s[tid] = qi < sh.Tq ? delta[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
  }
  float adq[NG][4][TN];
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) adq[g][i][j] = 0.0f;

  const int max_qpos = offset + q0 + qvalid - 1;
  int k_end = min(sh.Tk, max_qpos + 1);
  int k_begin = 0;
  if (sh.window >= 0) k_begin = max(0, offset + q0 - sh.window);
  k_begin = (k_begin / BKV) * BKV;
  // S tile 64 x 32: thread = rows (tid>>3)*2..+1, cols (tid&7)*4..+3
  const int sy = tid >> 3, sx = tid & 7;
  for (int kt = k_begin; kt < k_end; kt += BKV) {
    const int kvalid = min(BKV, sh.Tk - kt);
    __syncthreads();
    load_tile<DP, true>(Kt, LK, kg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid, sh.D);
    load_tile<DP, true>(Vt, LK, vg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid, sh.D);
    load_tile<DP, false>(Ks, LD, kg + (int64_t)kt * sh.kv_tstride, sh.kv_tstride, BKV, kvalid, sh.D);
    __syncthreads();
    float s[2][4], dp[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { s[i][j] = 0.0f; dp[i][j] = 0.0f; }
    mm_acc<2, 4>(s, Qt, LQ, Kt, LK, DP, sy * 2, sx * 4);
    mm_acc<2, 4>(dp, dOt, LQ, Vt, LK, DP, sy * 2, sx * 4);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int il = sy * 2 + i, qi = q0 + il, qpos = offset + qi;
      int32_t qseg = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int kj = kt + sx * 4 + j;
        float p = 0.0f;
        if (qi < sh.Tq && kj < sh.Tk && !attn_masked(qpos, kj, sh.window, sh.segment_ids, sh.seg_len, qseg)) p = __expf(s[i][j] - lse_s[il]);
        dSt[(sx * 4 + j) * LQ + il] = p * (dp[i][j] - delta_s[il]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < NG; ++g) mm_acc<4, TN>(adq[g], dSt, LQ, Ks, LD, BKV, ty * 4, g * 64 + tx * TN);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int qi = q0 + ty * 4 + i;
    if (qi >= sh.Tq) continue;
    float* dqg = dq + (int64_t)b * sh.q_bstride + (int64_t)qi * sh.q_tstride + (int64_t)hq * sh.D;
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        int c = g * 64 + tx * TN + j;
        if (c < sh.D) { if (accumulate) dqg[c] += adq[g][i][j]; else dqg[c] = adq[g][i][j]; }
      }
  }
}

template <int DP>
static int attn_bwd_go(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                       float* dq, float* dk, float* dv, int accumulate, cudaStream_t s) {
  constexpr int LD = DP + 4;
  size_t smem_kv = sizeof(float) * (size_t)(2 * DP * 68 + 2 * DP * 36 + 2 * 32 * LD + 2 * 32 * 68);
  size_t smem_q = sizeof(float) * (size_t)(2 * DP * 68 + 2 * DP * 36 + 32 * LD + 32 * 68);
  static PerDeviceOnce configured;
  if (configured.first()) {
    GN_CUDA(cudaFuncSetAttribute(attn_bwd_dkv_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
    GN_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
  }
  dim3 gkv(ceil_div(sh.Tk, 64), sh.B * sh.Hkv);
  attn_bwd_dkv_kernel<DP><<<gkv, AT, smem_kv, s>>>(sh, q, k, v, dout, lse, delta, dk, dv, accumulate);
  GN_LAUNCH_CHECK();
  dim3 gq(ceil_div(sh.Tq, 64), sh.B * sh.Hq);
  attn_bwd_dq_kernel<DP><<<gq, AT, smem_q, s>>>(sh, q, k, v, dout, lse, delta, dq, accumulate);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int attention_backward_launch(const AttnShape& sh, const float* q, const float* k, const float* v, const float* out, const float* dout,
                              const float* lse, const float* row_correction, float* dq, float* dk, float* dv, int accumulate,
                              float* delta_scratch, cudaStream_t s) {
  if (sh.Tq <= 0 || sh.B <= 0) return GN_OK;
  GN_REQUIRE(sh.D > 0 && sh.D <= 128, "attention: head_dim %d outside (0,128]", sh.D);
  const float* delta = row_correction;
  if (!delta) {
    int64_t total = (int64_t)sh.B * sh.Hq * sh.Tq;
    attn_delta_kernel<<<ceil_div(total, 8), 256, 0, s>>>(sh, out, dout, delta_scratch);
    GN_LAUNCH_CHECK();
    delta = delta_scratch;
  }
#ifdef GN_HAVE_TCGEN05
  if (sh.tensor && attention_tc_backward_ok(sh, q, k, v, dout, dq) && attention_mma_ok(sh, dk, dv, nullptr, nullptr, nullptr))
    return attention_tc_backward(sh, q, k, v, dout, lse, delta, dq, dk, dv, accumulate, s);
#endif
  if (sh.tensor && attention_mma_ok(sh, q, k, v, dout, dq) && attention_mma_ok(sh, dk, dv, nullptr, nullptr, nullptr))
    return attention_mma_backward(sh, q, k, v, dout, lse, delta, dq, dk, dv, accumulate, s);
  if (fast128_ok(sh, q, k, v, dout, dq) && fast128_ok(sh, dk, dv, nullptr, nullptr, nullptr))
    return attn_bwd128_go(sh, q, k, v, dout, lse, delta, dq, dk, dv, accumulate, s);
  if (sh.D <= 32) return attn_bwd_go<32>(sh, q, k, v, dout, lse, delta, dq, dk, dv, accumulate, s);
  if (sh.D <= 64) return attn_bwd_go<64>(sh, q, k, v, dout, lse, delta, dq, dk, dv, accumulate, s);
  return attn_bwd_go<128>(sh, q, k, v, dout, lse, delta, dq, dk, dv, accumulate, s);
}

// ============================================================== split / combine (contract)
// One warp per query row; the shard's keys are walked sequentially.
__global__ void __launch_bounds__(128) attn_split_kernel(AttnShape sh, const float* q, const float* k, const float* v, int kstart, int kend,
                                                         float* acc, float* mx, float* sm) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int i = blockIdx.x * 4 + warp;
  if (i >= sh.Tq) return;
  const int D = sh.D;
  const float* qr = q + (int64_t)i * sh.q_tstride;
  int qpos = sh.offset0 + i;
  int32_t qseg = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
  float qv[4], o[4] = {0, 0, 0, 0};
#pragma unroll
  for (int e = 0; e < 4; ++e) { int c = lane + 32 * e; qv[e] = c < D ? qr[c] : 0.0f; }
  float m = -INFINITY, l = 0.0f;
  for (int kj = kstart; kj < kend; ++kj) {
    const float* kr = k + (int64_t)kj * sh.kv_tstride;
    float d = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) { int c = lane + 32 * e; if (c < D) d = fmaf(qv[e], kr[c], d); }
    d = warp_sum(d);
    bool msk = kj > qpos || (sh.window >= 0 && qpos - kj > sh.window);
    if (!msk && sh.segment_ids && kj < sh.seg_len && qpos < sh.seg_len && sh.segment_ids[kj] != qseg) msk = true;
    if (msk) d = kMaskedScore;
    float mn = fmaxf(m, d);
    float alpha = (m == -INFINITY) ? 0.0f : expf(m - mn);
    float p = expf(d - mn);
    l = l * alpha + p;
    const float* vr = v + (int64_t)kj * sh.kv_tstride;
#pragma unroll
    for (int e = 0; e < 4; ++e) { int c = lane + 32 * e; if (c < D) o[e] = o[e] * alpha + p * vr[c]; }
    m = mn;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) { int c = lane + 32 * e; if (c < D) acc[(int64_t)i * D + c] = o[e]; }
  if (lane == 0) { mx[i] = m; sm[i] = l; }
}
int attention_split_launch(const AttnShape& sh, const float* q, const float* k, const float* v, int kstart, int kend, float* acc, float* mx,
                           float* sm, cudaStream_t s) {
  if (sh.Tq <= 0) return GN_OK;
  GN_REQUIRE(sh.D > 0 && sh.D <= 128, "attention: head_dim %d outside (0,128]", sh.D);
  if (kend > sh.Tk) kend = sh.Tk;
  if (kstart < 0) kstart = 0;
  attn_split_kernel<<<ceil_div(sh.Tq, 4), 128, 0, s>>>(sh, q, k, v, kstart, kend, acc, mx, sm);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// kernels/scalar/attention.go:104-141
__global__ void __launch_bounds__(128) attn_combine_kernel(const float* acc, const float* mx, const float* sm, int parts, int ql, int hd, float* out, float* lse) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int i = blockIdx.x * 4 + warp;
  if (i >= ql) return;
  float gm = -INFINITY;
  for (int p = 0; p < parts; ++p) gm = fmaxf(gm, mx[(int64_t)p * ql + i]);
  float total = 0;
  for (int p = 0; p < parts; ++p) {
    float m = mx[(int64_t)p * ql + i];
    float sc = (m > -INFINITY) ? expf(m - gm) : 0.0f;
    total += sm[(int64_t)p * ql + i] * sc;
  }
  float inv = total > 0 ? 1.0f / total : 1.0f;
  for (int c = lane; c < hd; c += 32) {
    float o = 0;
    for (int p = 0; p < parts; ++p) {
      float m = mx[(int64_t)p * ql + i];
      float sc = (m > -INFINITY) ? expf(m - gm) : 0.0f;
      o += acc[((int64_t)p * ql + i) * hd + c] * sc;
    }
    out[(int64_t)i * hd + c] = o * inv;
  }
  if (lse && lane == 0) lse[i] = gm + logf(total);
}
int attention_combine_launch(const float* acc, const float* mx, const float* sm, int parts, int ql, int hd, float* out, float* lse, cudaStream_t s) {
  if (ql <= 0) return GN_OK;
  attn_combine_kernel<<<ceil_div(ql, 4), 128, 0, s>>>(acc, mx, sm, parts, ql, hd, out, lse);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// ============================================================== decode
// CTA = one (row, kv head, key split); NW warps (4, 8 or 16) stride over the keys of the
// split; each lane owns D/32 consecutive channels (float4 for D = 128), so a
// warp reads one K row and one V row as a single coalesced 512-byte request.
// All query heads of the group are served from the same K/V registers.
// Warp partials are merged through shared memory, splits through a second pass.
template <int DP, int RATIO, int U, int NW>
__global__ void __launch_bounds__(32 * NW) attn_decode_kernel(const float* __restrict__ q, int64_t q_rstride, const float* __restrict__ kcache,
                                                          const float* __restrict__ vcache, int64_t row_stride, int64_t head_stride,
                                                          const int32_t* __restrict__ ctx_len, int Hq, int Hkv, int D, int window, float* __restrict__ out,
                                                          int64_t o_rstride, float* __restrict__ part_acc, float* __restrict__ part_ms, int splits,
                                                          float* __restrict__ out_hi, float* __restrict__ out_lo, int kmin, int slot0, int nslots) {
  pdl_trigger();
  pdl_wait();
  // DP = head_dim rounded up to a multiple of 32; channels >= D are zero padding.
  // Keys below kmin belong to the shared-prefix kernel; this kernel's partial results then go to
  // slots slot0 .. slot0 + splits - 1 of nslots (nslots == splits and slot0 == 0 without a prefix pass).
  constexpr int E = DP / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x / Hkv, hk = blockIdx.x % Hkv, split = blockIdx.y;
  const int ctx = ctx_len[row];
  const int qpos = ctx - 1;
  int kbeg = kmin;
  if (window >= 0) kbeg = max(kmin, qpos - window);
  const int span = ctx - kbeg;
  const int per = (span + splits - 1) / splits;
  const int k0 = kbeg + split * per, k1 = min(ctx, k0 + per);

  float qv[RATIO][E];
#pragma unroll
  for (int h = 0; h < RATIO; ++h)
#pragma unroll
    for (int e = 0; e < E; ++e) qv[h][e] = (lane * E + e < D) ? q[(int64_t)row * q_rstride + (int64_t)(hk * RATIO + h) * D + lane * E + e] : 0.0f;
  float m[RATIO], l[RATIO], o[RATIO][E];
#pragma unroll
  for (int h = 0; h < RATIO; ++h) {
    m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
    for (int e = 0; e < E; ++e) o[h][e] = 0.0f;
  }
  const float* kb = kcache + (int64_t)row * row_stride + (int64_t)hk * head_stride;
  const float* vb = vcache + (int64_t)row * row_stride + (int64_t)hk * head_stride;
  // One key per warp per iteration; the next key's K and V rows are requested before the current one is used, so
  // that two rows per warp are in flight (with a single row the loop runs at the memory latency, not the bandwidth).
  auto load_row = [&](int kj, float (&kr)[E], float (&vr)[E]) {
    if (E == 4 && DP == 128) {
      const float4 a = *reinterpret_cast<const float4*>(kb + (int64_t)kj * D + lane * 4);
      const float4 c = *reinterpret_cast<const float4*>(vb + (int64_t)kj * D + lane * 4);
      kr[0] = a.x; kr[1] = a.y; kr[2] = a.z; kr[3] = a.w; vr[0] = c.x; vr[1] = c.y; vr[2] = c.z; vr[3] = c.w;
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const bool ok = lane * E + e < D;
        kr[e] = ok ? kb[(int64_t)kj * D + lane * E + e] : 0.0f; vr[e] = ok ? vb[(int64_t)kj * D + lane * E + e] : 0.0f;
      }
    }
  };
  // NW warps share the keys of the CTA round-robin (small grids use more warps per CTA instead of more splits, which
  // would need a combine pass).  U keys per warp per iteration (kj, kj + NW, ...), and the next U are requested before these are used: 2U rows per
  // warp in flight, one running-maximum update per U keys.  U = 1 keeps more warps resident (large batches); U = 2
  // shortens the dependent chain when there are few warps per SM.
  float nk[U][E], nv[U][E];
#pragma unroll
  for (int u = 0; u < U; ++u) {
#pragma unroll
    for (int e = 0; e < E; ++e) { nk[u][e] = 0.0f; nv[u][e] = 0.0f; }
    if (k0 + warp + NW * u < k1) load_row(k0 + warp + NW * u, nk[u], nv[u]);
  }
  for (int kj = k0 + warp; kj < k1; kj += NW * U) {
    float kv[U][E], vv[U][E];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int e = 0; e < E; ++e) { kv[u][e] = nk[u][e]; vv[u][e] = nv[u][e]; }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (kj + NW * (U + u) < k1) load_row(kj + NW * (U + u), nk[u], nv[u]);
#pragma unroll
    for (int h = 0; h < RATIO; ++h) {
      float d[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        d[u] = 0;
#pragma unroll
        for (int e = 0; e < E; ++e) d[u] = fmaf(qv[h][e], kv[u][e], d[u]);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int u = 0; u < U; ++u) d[u] += __shfl_xor_sync(0xffffffffu, d[u], off);
      float mn = m[h];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (u > 0 && kj + NW * u >= k1) d[u] = -INFINITY;
        mn = fmaxf(mn, d[u]);
      }
      const float alpha = (m[h] == -INFINITY) ? 0.0f : __expf(m[h] - mn);
      float p[U];
#pragma unroll
      for (int u = 0; u < U; ++u) p[u] = (u > 0 && kj + NW * u >= k1) ? 0.0f : __expf(d[u] - mn);
      float ls = l[h] * alpha;
#pragma unroll
      for (int u = 0; u < U; ++u) ls += p[u];
      l[h] = ls;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        float acc = o[h][e] * alpha;
#pragma unroll
        for (int u = 0; u < U; ++u) acc = fmaf(p[u], vv[u][e], acc);
        o[h][e] = acc;
      }
      m[h] = mn;
    }
  }
  // merge the warps
  __shared__ float sm_o[NW][RATIO][DP];
  __shared__ float sm_m[NW][RATIO], sm_l[NW][RATIO];
#pragma unroll
  for (int h = 0; h < RATIO; ++h) {
#pragma unroll
    for (int e = 0; e < E; ++e) sm_o[warp][h][lane * E + e] = o[h][e];
    if (lane == 0) { sm_m[warp][h] = m[h]; sm_l[warp][h] = l[h]; }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < RATIO * DP; idx += 32 * NW) {
    int h = idx / DP, c = idx % DP;
    if (c >= D) continue;
    float gm = sm_m[0][h];
#pragma unroll
    for (int w = 1; w < NW; ++w) gm = fmaxf(gm, sm_m[w][h]);
    float tot = 0, acc = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      float sc = (sm_m[w][h] == -INFINITY) ? 0.0f : __expf(sm_m[w][h] - gm);
      tot += sm_l[w][h] * sc;
      acc += sm_o[w][h][c] * sc;
    }
    int hq = hk * RATIO + h;
    if (splits == 1) {
      // the only CTA of this (row, kv head): finish here, merging the slots an earlier shared-prefix
      // launch left for this head (slot0 of them; stream order makes them visible)
      const int64_t pi0 = ((int64_t)row * Hq + hq) * nslots;
      if (slot0 > 0) {
        // two passes, so that the loads of a pass do not wait on one another: the maximum over the slots first,
        // then the sums against it (a long prompt leaves dozens of slots)
        float gmax = gm;
#pragma unroll 4
        for (int sl = 0; sl < slot0; ++sl) gmax = fmaxf(gmax, part_ms[(pi0 + sl) * 2]);
        const float a0 = (gm == -INFINITY) ? 0.0f : __expf(gm - gmax);
        tot *= a0; acc *= a0;
#pragma unroll 4
        for (int sl = 0; sl < slot0; ++sl) {
          const float pm = part_ms[(pi0 + sl) * 2], pl = part_ms[(pi0 + sl) * 2 + 1];
          const float a1 = (pm == -INFINITY) ? 0.0f : __expf(pm - gmax);
          tot += pl * a1;
          acc += part_acc[(pi0 + sl) * D + c] * a1;
        }
        gm = gmax;
      }
      const float v = tot > 0 ? acc / tot : 0.0f;
      const int64_t oi = (int64_t)row * o_rstride + (int64_t)hq * D + c;
      out[oi] = v;
      if (out_hi) { float h2, l2; split_tf32(v, h2, l2); out_hi[oi] = h2; out_lo[oi] = l2; }
    } else {
      int64_t pi = ((int64_t)row * Hq + hq) * nslots + slot0 + split;
      part_acc[pi * D + c] = acc;
      if (c == 0) { part_ms[pi * 2] = gm; part_ms[pi * 2 + 1] = tot; }
    }
  }
}
__global__ void __launch_bounds__(128) attn_decode_combine_kernel(const float* part_acc, const float* part_ms, int splits, int Hq, int D, float* out, int64_t o_rstride,
                                                                  float* out_hi, float* out_lo, float* lse_out) {
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.x / Hq, hq = blockIdx.x % Hq;
  int64_t base = ((int64_t)row * Hq + hq) * splits;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, part_ms[(base + s) * 2]);
  float tot = 0;
  for (int s = 0; s < splits; ++s) { float m = part_ms[(base + s) * 2]; tot += (m == -INFINITY) ? 0.0f : part_ms[(base + s) * 2 + 1] * __expf(m - gm); }
  if (lse_out && threadIdx.x == 0) lse_out[(int64_t)row * Hq + hq] = tot > 0 ? gm + logf(tot) : -INFINITY;   // [rows, Hq]
  for (int c = threadIdx.x; c < D; c += 128) {
    float acc = 0;
    for (int s = 0; s < splits; ++s) { float m = part_ms[(base + s) * 2]; if (m != -INFINITY) acc += part_acc[(base + s) * D + c] * __expf(m - gm); }
    const float v = tot > 0 ? acc / tot : 0.0f;
    const int64_t oi = (int64_t)row * o_rstride + (int64_t)hq * D + c;
    out[oi] = v;
    if (out_hi) { float h2, l2; split_tf32(v, h2, l2); out_hi[oi] = h2; out_lo[oi] = l2; }
  }
}

constexpr int kPrefixTile = 32, kPrefixMaxHeads = 32;   // the shared-prefix pass (attention_mma.cu): keys per tile, query vectors per group and kv head
// -1: the rule below decides; 0 / 1: the shared-prefix pass is off / on wherever it applies (process-wide policy).
std::atomic<int> g_prefix_sharing{-1};
void attention_decode_prefix_mode(int mode) { g_prefix_sharing.store(mode < 0 ? -1 : (mode ? 1 : 0), std::memory_order_relaxed); }

// Partial-result slots the shared-prefix pass writes: one per tile of 32 prompt positions
// (0 when the pass does not apply: head_dim other than 128, or more than 32 query vectors per group and kv head).
int attention_decode_prefix_splits(int rows, int group, int Hq, int Hkv, int D, int prefix_len) {
  if (group <= 1 || prefix_len <= 0 || D != 128 || group * (Hq / Hkv) > kPrefixMaxHeads || rows % group != 0) return 0;
  const int tiles = (prefix_len + kPrefixTile - 1) / kPrefixTile;
  // Measured on d12 (128-token prompts, groups of 8): with the pass on the tensor pipe (13.6 us for the 512-row batch) the
  // per-row kernel only walks the generated keys: 23 vs 33 us per layer at context 133, 51 vs 58 at 256, 74 vs 81 at 384
  // with 512 rows, 31 vs 39 at 256 rows; at 128 rows and below the extra launch costs more than it saves (25 vs 18 us).
  // The option "decode_prefix_sharing" (1 / 0) overrides the rule; tests exercise the pass with it.
  const int forced = g_prefix_sharing.load(std::memory_order_relaxed);
  if (forced == 0) return 0;
  if (forced < 0 && (prefix_len < 64 || group < 4 || (int64_t)rows * Hkv < 3 * (int64_t)num_sms())) return 0;
  return tiles;
}

// Warps per CTA of the per-row kernel: 4 on grids that fill the machine, 8 or 16 on smaller ones.
int attention_decode_warps(int rows, int Hkv) {
  const int base = rows * Hkv;
  return base >= num_sms() * 4 ? 4 : (base >= num_sms() * 2 ? 8 : 16);
}

int attention_decode_splits(int rows, int Hkv, int max_ctx) {
  // Fill the machine: aim at the equivalent of >= 4 four-warp CTAs per SM, at least 64 keys per four warps.  The
  // warps of a CTA come first (no second pass); only very small batches also split the context over CTAs.
  const int wf = attention_decode_warps(rows, Hkv) / 4;
  int base = rows * Hkv * wf;
  int splits = 1;
  while (base * splits < num_sms() * 4 && max_ctx / (splits * wf * 2) >= 64 && splits < 16) splits *= 2;
  return splits;
}

template <int DP, int RATIO>
static int decode_go(const float* q, int64_t q_rstride, const float* kcache, const float* vcache, int64_t row_stride, int64_t head_stride,
                     const int32_t* ctx_len, int rows, int Hq, int Hkv, int D, int window, float* out, int64_t o_rstride, float* part_acc, float* part_ms,
                     int splits, cudaStream_t s, float* out_hi, float* out_lo, int group, int prefix_len, float* lse_out) {
  GN_REQUIRE(!lse_out || splits > 1, "decode attention: the log-sum-exp comes from the combine pass (splits %d)", splits);
  int psplits = 0;
  psplits = attention_decode_prefix_splits(rows, group, Hq, Hkv, D, prefix_len);
  if (psplits > 0) {
    GN_TRY(attention_mma_decode_prefix(q, q_rstride, kcache, vcache, row_stride, head_stride, ctx_len, rows, Hq, Hkv, window, group, prefix_len, part_acc, part_ms,
                                       psplits + splits, s));
  }
  const int nslots = psplits + splits;
  dim3 grid(rows * Hkv, splits);
  // fewer than the equivalent of ~5 four-warp CTAs per SM: two keys per iteration (shorter chain); otherwise one
  // (more resident warps)
  const int nw = attention_decode_warps(rows, Hkv);
  // Small grids launch as programmatic dependents (their CTAs are resident and waiting when the kernel in front
  // finishes); a grid of several waves gains nothing from that and would only take residency from the tail of its
  // predecessor, so it launches normally (the kernel's wait is then a no-op).
  const bool dependent = (int64_t)rows * Hkv * splits <= 2 * (int64_t)num_sms();
#define GN_DEC_LAUNCH(UU, WW) do { if (dependent) GN_CUDA(launch_pdl(attn_decode_kernel<DP, RATIO, UU, WW>, grid, dim3(32 * WW), 0, s, q, q_rstride, kcache, vcache, row_stride, head_stride, ctx_len, Hq, Hkv, D, window, out, o_rstride, \
                                                                              part_acc, part_ms, splits, out_hi, out_lo, psplits ? prefix_len : 0, psplits, nslots)); \
    else attn_decode_kernel<DP, RATIO, UU, WW><<<grid, 32 * WW, 0, s>>>(q, q_rstride, kcache, vcache, row_stride, head_stride, ctx_len, Hq, Hkv, D, window, out, o_rstride, \
                                                                              part_acc, part_ms, splits, out_hi, out_lo, psplits ? prefix_len : 0, psplits, nslots); } while (0)
  // the warps' partial results meet in static shared memory (NW x RATIO x DP floats): wide groups get fewer warps
  constexpr int kMaxW = RATIO * DP * 16 <= 10240 ? 16 : (RATIO * DP * 8 <= 10240 ? 8 : 4);
  if (nw == 16 && kMaxW >= 16) { if constexpr (kMaxW >= 16) { GN_DEC_LAUNCH(2, 16); } }
  else if (nw >= 8 && kMaxW >= 8) { if constexpr (kMaxW >= 8) { GN_DEC_LAUNCH(2, 8); } }
  else if ((int64_t)rows * Hkv * splits < (int64_t)num_sms() * 5) { GN_DEC_LAUNCH(2, 4); }
  else { GN_DEC_LAUNCH(1, 4); }
#undef GN_DEC_LAUNCH
  GN_LAUNCH_CHECK();
  if (splits > 1) {
    GN_CUDA(launch_pdl(attn_decode_combine_kernel, dim3(rows * Hq), dim3(128), 0, s, part_acc, part_ms, nslots, Hq, D, out, o_rstride, out_hi, out_lo, lse_out));
    GN_LAUNCH_CHECK();
  }
  return GN_OK;
}

int attention_decode_launch(const float* q, int64_t q_rstride, const float* kcache, const float* vcache, int64_t row_stride, int64_t head_stride,
                            const int32_t* ctx_len, int rows, int Hq, int Hkv, int D, int window, float* out, int64_t o_rstride,
                            float* part_acc, float* part_ms, int splits, cudaStream_t s, float* out_hi, float* out_lo, int group, int prefix_len, float* lse_out) {
  if (rows <= 0) return GN_OK;
  int ratio = Hq / Hkv;
  const int dp = (D + 31) / 32 * 32;
#define GN_DEC(DD, RR) if (dp == DD && ratio == RR) return decode_go<DD, RR>(q, q_rstride, kcache, vcache, row_stride, head_stride, ctx_len, rows, Hq, Hkv, D, window, out, o_rstride, part_acc, part_ms, splits, s, out_hi, out_lo, group, prefix_len, lse_out)
  GN_DEC(128, 1); GN_DEC(128, 2); GN_DEC(128, 3); GN_DEC(128, 4); GN_DEC(128, 8);
  GN_DEC(96, 1); GN_DEC(96, 2); GN_DEC(96, 4);
  GN_DEC(64, 1); GN_DEC(64, 2); GN_DEC(64, 3); GN_DEC(64, 4); GN_DEC(64, 8);
  GN_DEC(32, 1); GN_DEC(32, 2); GN_DEC(32, 3); GN_DEC(32, 4); GN_DEC(32, 8);
#undef GN_DEC
  set_error("decode attention: unsupported head_dim %d / group ratio %d", D, ratio);
  return GN_ERR_INVALID;
}

}  // namespace gn
