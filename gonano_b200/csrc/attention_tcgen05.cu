// head_dim 128 attention on the 5th-generation tensor cores (tcgen05), forward pass, for the training pass and
// the prefill (kernels/backend.go:167-283; scalar statement kernels/scalar/attention.go:16-205).  sm_100a only.
//
// Precision: 3xTF32 as in the products (gemm_tcgen05.cu): every float32 operand x is hi = tf32(x), lo = tf32(x - hi)
// and each product is lo*hi + hi*lo + hi*hi accumulated in float32 in tensor memory.  Scores are raw q.k (the model
// applies no 1/sqrt(d)); a masked score counts as the reference's finite -1e30, i.e. probability 0
// (kernels/scalar/attention.go:11).
//
// One CTA per (sequence, query head, 128 queries), 352 threads, keys in steps of 64:
//   warps 0,10 TMA producers: warp 0 Q once, then per step the K tile (K-major, 4 k-blocks of 32 channels); warp 10
//              the V tile (read MN-major in place: channels contiguous, 2 k-blocks of 32 keys); hi and lo copies each;
//   warp 1     allocates the 512 columns of tensor memory and issues the instructions: S = Q K^T with Q as the A
//              operand IN tensor memory (48 instructions M=128 N=64 K=8), O += P V with P from shared memory
//              (24 instructions N=128); score tiles are issued up to two steps ahead of the P V, so the tensor pipe
//              works while the softmax threads are busy;
//   warps 2-9  two threads per query row (32 keys of a step and 64 channels of O each): copy Q into tensor memory,
//              then per step read the row of S, take the running maximum (the accumulator O is rescaled only when the maximum grew by more than 8: the final
//              division by the running sum makes the result independent of which maximum was used), write
//              P = exp(S - max) as hi/lo tiles in the swizzled K-major layout the tensor core reads, and at the end
//              scale O by 1 / sum and store it with the log-sum-exp.
// Tensor memory: Q hi [0,128), Q lo [128,256), O [256,384), two score buffers [384,448), [448,512).
// Shared memory: K hi/lo 64 KB, V hi/lo 64 KB, P hi/lo 64 KB (Q passes through the P and V areas on its way in).
// Every wait on an mbarrier is bounded; when a bound runs out the kernel raises the products' error flag, drains
// and returns.
#include <atomic>

#include "kernels.cuh"
#include "tcgen05.cuh"

namespace gn {

namespace {

constexpr int AQ = 128;    // queries per CTA = UMMA M
constexpr int AKV = 64;    // keys per step = UMMA N of the score product
constexpr int AD = 128;    // head_dim
constexpr uint32_t K_HI = 0, K_LO = 32768, V_HI = 65536, V_LO = 98304, P_HI = 131072, P_LO = 163840, BARS = 196608, XCH = BARS + 256;
constexpr int kSmemFwd = XCH + 3 * 1024 + 1024;   // + barriers + exchange area + slack for the 1024-byte alignment
constexpr uint32_t COL_QH = 0, COL_QL = 128, COL_O = 256, COL_S = 384;
constexpr float kRescaleStep = 8.0f;

std::atomic<int> g_attn_tc{1};

#ifdef GN_TC_TRACE
__device__ long long g_attn_trace[256];
#define AT_TRACE(slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) g_attn_trace[(slot)] = clock64(); } while (0)
#else
#define AT_TRACE(slot) do { } while (0)
#endif

struct AttnTc {
  int B, Hq, Hkv, Tq, Tk, window, offset;
  int ratio, shift;   // the last key a query at position p sees is p / ratio - shift: (1, 0) causal over positions, (r, 1) over blocks of r positions
  float* out; int64_t o_bstride, o_tstride, o_hstride;
  float* lse;
  __device__ __forceinline__ int last_key(int pos) const { return ratio == 1 ? pos : pos / ratio - shift; }
};

// Packed tf32 splits of the operands: Q as [B * Tq, Hq * 128], K and V as [B * Tk, Hkv * 128], hi and lo.
// One warp per (row, head): a float4 per lane.
__global__ void __launch_bounds__(256) attn_tc_split_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                            float* __restrict__ hi, float* __restrict__ lo, int64_t k_off, int64_t v_off) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nq = (int64_t)sh.B * sh.Tq * sh.Hq, nk = (int64_t)sh.B * sh.Tk * sh.Hkv;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= nq + 2 * nk) return;
  const float* src; int64_t dst;
  if (idx < nq) {
    const int h = (int)(idx % sh.Hq); const int64_t r = idx / sh.Hq; const int64_t b = r / sh.Tq, t = r % sh.Tq;
    src = q + b * sh.q_bstride + t * sh.q_tstride + (int64_t)h * (sh.q_hstride ? sh.q_hstride : AD); dst = idx * AD;
  } else {
    const int64_t i = idx - nq; const bool isv = i >= nk; const int64_t e = isv ? i - nk : i;
    const int h = (int)(e % sh.Hkv); const int64_t r = e / sh.Hkv; const int64_t b = r / sh.Tk, t = r % sh.Tk;
    src = (isv ? v : k) + b * sh.kv_bstride + t * sh.kv_tstride + (int64_t)h * sh.kv_hstride; dst = (isv ? v_off : k_off) + e * AD;
  }
  const float4 x = reinterpret_cast<const float4*>(src)[lane];
  float4 h4, l4;
  split_tf32_int(x.x, h4.x, l4.x); split_tf32_int(x.y, h4.y, l4.y); split_tf32_int(x.z, h4.z, l4.z); split_tf32_int(x.w, h4.w, l4.w);
  reinterpret_cast<float4*>(hi + dst)[lane] = h4;
  reinterpret_cast<float4*>(lo + dst)[lane] = l4;
}

__global__ void __launch_bounds__(352, 1) attn_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQh, const __grid_constant__ CUtensorMap tmQl,
                                                             const __grid_constant__ CUtensorMap tmKh, const __grid_constant__ CUtensorMap tmKl,
                                                             const __grid_constant__ CUtensorMap tmVh, const __grid_constant__ CUtensorMap tmVl,
                                                             AttnTc p, int* err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles want 1024-byte alignment
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + BARS;
  const uint32_t q_full = bars, q_done = bars + 8, k_full = bars + 16, k_empty = bars + 24, v_full = bars + 32, pv_done = bars + 40, p_full = bars + 48;
  auto s_full = [&](int b) { return bars + 56u + 8u * b; };
  auto s_empty = [&](int b) { return bars + 72u + 8u * b; };
  const uint32_t tmem_slot = bars + 88;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + BARS + 88);

  if (threadIdx.x == 0) AT_TRACE(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * AQ;   // the long tiles first
  const int hq = blockIdx.y, b = blockIdx.z, hk = hq / (p.Hq / p.Hkv);
  const int qvalid = min(AQ, p.Tq - q0);
  const int k_end = min(p.Tk, p.last_key(p.offset + q0 + qvalid - 1) + 1);
  int k_begin = p.window >= 0 ? max(0, p.offset + q0 - p.window) : 0;
  k_begin = (k_begin / AKV) * AKV;
  const int n = k_end > k_begin ? (k_end - k_begin + AKV - 1) / AKV : 0;   // key steps of this CTA

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_done, 256); mbar_init(k_full, 1); mbar_init(k_empty, 1); mbar_init(v_full, 1); mbar_init(pv_done, 1);
    mbar_init(p_full, 256);
    for (int i = 0; i < 2; ++i) { mbar_init(s_full(i), 1); mbar_init(s_empty(i), 256); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  bool failed = false;
  pdl_wait();
  if (threadIdx.x == 0) AT_TRACE(1);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer of Q and K
    if (lane == 0 && n > 0) {
      mbar_expect_tx(q_full, 2 * AQ * AD * 4);
      tma_load_3d(base + P_HI, &tmQh, q_full, 0, b * p.Tq + q0, hq * (AD / 32));
      tma_load_3d(base + V_HI, &tmQl, q_full, 0, b * p.Tq + q0, hq * (AD / 32));
      for (int j = 0; j < n; ++j) {
        if (j > 0 && !mbar_wait(k_empty, (uint32_t)(j - 1) & 1u)) { failed = true; break; }
        if (j < 8) AT_TRACE(120 + 2 * j);
        mbar_expect_tx(k_full, 2 * AKV * AD * 4);
        tma_load_3d(base + K_HI, &tmKh, k_full, 0, b * p.Tk + k_begin + j * AKV, hk * (AD / 32));
        tma_load_3d(base + K_LO, &tmKl, k_full, 0, b * p.Tk + k_begin + j * AKV, hk * (AD / 32));
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------- TMA producer of V
    if (lane == 0 && n > 0) {
      for (int j = 0; j < n; ++j) {
        const int row = b * p.Tk + k_begin + j * AKV;
        // the V area is free once Q has left it (first step) or the previous P V has read it
        if (!mbar_wait(j == 0 ? q_done : pv_done, j == 0 ? 0u : (uint32_t)(j - 1) & 1u)) { failed = true; break; }
        if (j < 8) AT_TRACE(121 + 2 * j);
        mbar_expect_tx(v_full, 2 * AKV * AD * 4);
        for (int kk = 0; kk < 2; ++kk) {
          tma_load_3d(base + V_HI + kk * 16384, &tmVh, v_full, 0, row + kk * 32, hk * (AD / 32));
          tma_load_3d(base + V_LO + kk * 16384, &tmVl, v_full, 0, row + kk * 32, hk * (AD / 32));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    // Two queues, scores (js) and P V (jp), each in step order; whichever has its operands ready goes next, P V first
    // (the softmax threads of the next step wait for it), the scores at most two steps ahead (two score buffers).
    if (lane == 0 && n > 0) {
      const uint32_t idS = instr_desc_tf32(AQ, AKV), idO = instr_desc_tf32(AQ, AD, 0, 1);
      if (!mbar_wait(q_done, 0u)) failed = true;
      tc_fence_after();
      int js = 0, jp = 0;
      uint32_t idle = 0;
      while (jp < n && !failed) {
        bool did = false;
        if (jp < js && mbar_test(p_full, (uint32_t)jp & 1u) && mbar_test(v_full, (uint32_t)jp & 1u)) {
          tc_fence_after();
          if (jp < 8) AT_TRACE(82 + 4 * jp);
          const uint32_t d = tmem_base + COL_O;
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            const uint64_t ph = smem_desc_sw128(base + P_HI + kk * 16384), pl = smem_desc_sw128(base + P_LO + kk * 16384);
            const uint64_t vh = kMnDesc | (uint64_t)(((base + V_HI + kk * 16384) & 0x3FFFFu) >> 4), vl = kMnDesc | (uint64_t)(((base + V_LO + kk * 16384) & 0x3FFFFu) >> 4);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              umma_tf32(d, pl + 2u * ks, vh + (uint64_t)kMnKStep * ks, idO, (jp > 0 || kk > 0 || ks > 0) ? 1u : 0u);
              umma_tf32(d, ph + 2u * ks, vl + (uint64_t)kMnKStep * ks, idO, 1u);
              umma_tf32(d, ph + 2u * ks, vh + (uint64_t)kMnKStep * ks, idO, 1u);
            }
          }
          umma_commit(pv_done);
          if (jp < 8) AT_TRACE(83 + 4 * jp);
          ++jp; did = true;
        }
        if (js < n && js <= jp + 2 && mbar_test(k_full, (uint32_t)js & 1u) && (js < 2 || mbar_test(s_empty(js & 1), (uint32_t)((js >> 1) - 1) & 1u))) {
          tc_fence_after();
          if (js < 8) AT_TRACE(80 + 4 * js);
          const uint32_t d = tmem_base + COL_S + (uint32_t)(js & 1) * AKV;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint64_t kh = smem_desc_sw128(base + K_HI + kb * 8192), kl = smem_desc_sw128(base + K_LO + kb * 8192);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint32_t ah = tmem_base + COL_QH + kb * 32 + ks * 8, al = tmem_base + COL_QL + kb * 32 + ks * 8;
              umma_tf32_ts(d, al, kh + 2u * ks, idS, (kb > 0 || ks > 0) ? 1u : 0u);
              umma_tf32_ts(d, ah, kl + 2u * ks, idS, 1u);
              umma_tf32_ts(d, ah, kh + 2u * ks, idS, 1u);
            }
          }
          umma_commit(k_empty);
          umma_commit(s_full(js & 1));
          if (js < 8) AT_TRACE(81 + 4 * js);
          ++js; did = true;
        }
        if (did) idle = 0;
        else { if (++idle > kSpinLimit) failed = true; else if (idle > 4096) __nanosleep(64); }
      }
    }
  } else {
    // ------------------------------------------------------------- softmax threads (warps 2..9): two per query row
    // Thread (quarter, lane, half) owns row = 32 * quarter + lane and the keys [32 * half, +32) of every step, the
    // channels [64 * half, +64) of O.  The two threads of a row exchange their maxima and sums through shared memory.
    const int quarter = warp & 3;                 // a warp reaches the tensor-memory lanes [32 * (warp % 4), +32)
    const int half = ((warp - 2) >> 2) & 1;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t sw = (uint32_t)(row & 7);      // 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8)
    const int qpos = p.last_key(p.offset + q0 + row);   // the last key this row sees
    float* xch = reinterpret_cast<float*>(gen + XCH);   // [2 steps][2 halves][128 rows]
    constexpr float kLog2e = 1.4426950408889634f;
    float m_used = -1e30f, l_run = 0.0f;
    if (n > 0) {
      // Q: shared memory (as the TMA wrote it) -> tensor memory, lane = row, column = channel; half 0 moves hi, half 1 lo
      if (!mbar_wait(q_full, 0u)) failed = true;
      if (threadIdx.x == 64) AT_TRACE(2);
      if (!failed) {
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint8_t* src = gen + (half ? V_HI : P_HI) + kb * 16384 + row * 128;
          uint32_t r[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 x = *reinterpret_cast<const uint4*>(src + ((c ^ sw) << 4));
            r[4 * c] = x.x; r[4 * c + 1] = x.y; r[4 * c + 2] = x.z; r[4 * c + 3] = x.w;
          }
          tmem_st32(lane_addr + (half ? COL_QL : COL_QH) + kb * 32, r);
        }
        tmem_st_wait();
      }
      tc_fence_before();
      mbar_arrive(q_done);
      if (threadIdx.x == 64) AT_TRACE(3);
    }
    for (int j = 0; j < n; ++j) {
      const int kv0 = k_begin + j * AKV;
      if (!failed && !mbar_wait(s_full(j & 1), (uint32_t)(j >> 1) & 1u)) failed = true;
      if (failed) { asm volatile("bar.sync 1, 256;" ::: "memory"); continue; }   // a thread that gave up still meets the others at every barrier
      tc_fence_after();
      if (threadIdx.x == 64 && j < 8) AT_TRACE(16 + 8 * j);
      float s[32];
      {
        uint32_t r[32];
        tmem_ld32(lane_addr + COL_S + (uint32_t)(j & 1) * AKV + half * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]);
      }
      tc_fence_before();
      mbar_arrive(s_empty(j & 1));   // the scores are in registers: the buffer may take step j + 2
      if (threadIdx.x == 64 && j < 8) AT_TRACE(17 + 8 * j);
      // mask (only in steps that touch the diagonal, the window's edge or the end of the sequence): key after the
      // query, key further back than the window, key past the sequence
      const int c0k = kv0 + half * 32;   // first key of this thread's columns
      const bool clean = kv0 + AKV - 1 <= p.last_key(p.offset + q0) && kv0 + AKV - 1 < p.Tk && (p.window < 0 || p.offset + q0 + AQ - 1 - kv0 <= p.window);
      float mx = -1e30f;
      if (clean) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, s[i]);
      } else {
        const int hi_k = min(qpos, p.Tk - 1) - c0k;                               // last valid column of this row
        const int lo_k = p.window >= 0 ? qpos - p.window - c0k : -(1 << 30);      // first valid column
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool ok = i <= hi_k && i >= lo_k;
          s[i] = ok ? s[i] : -1e30f;
          mx = fmaxf(mx, s[i]);
        }
      }
      float* xs = xch + (j & 1) * 256;
      xs[half * 128 + row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, xs[(half ^ 1) * 128 + row]);
      const bool need = mx > m_used + kRescaleStep;
      if (j > 0) {
        // the previous P V has finished: P may be overwritten and O is at rest
        if (!mbar_wait(pv_done, (uint32_t)(j - 1) & 1u)) { failed = true; continue; }
        tc_fence_after();
        if (threadIdx.x == 64 && j < 8) AT_TRACE(18 + 8 * j);
        if (__any_sync(0xffffffffu, need)) {
          const float f = need ? exp2f(m_used * kLog2e - mx * kLog2e) : 1.0f;   // the same rounded exponents P uses
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(lane_addr + COL_O + half * 64 + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
            tmem_st32(lane_addr + COL_O + half * 64 + c0, r);
          }
          tmem_st_wait();
          l_run *= f;
        }
      }
      if (need) m_used = mx;
      if (threadIdx.x == 64 && j < 8) AT_TRACE(19 + 8 * j);
      // P = exp(S - max) as hi/lo tiles, K-major with the 128-byte swizzle; this thread's 32 keys are k-block `half`.
      // hi = P cut to tf32, lo = P - hi (exact; the tensor core reads its leading bits).
      {
        const float mneg = -m_used * kLog2e;
        uint8_t* ph = gen + P_HI + half * 16384 + row * 128;
        uint8_t* pl = gen + P_LO + half * 16384 + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float h[4], l[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float sv = s[4 * c + t];
            float e = exp2f(fmaf(sv, kLog2e, mneg));
            if (!clean) e = sv > -1e29f ? e : 0.0f;
            l_run += e;
            h[t] = __uint_as_float(__float_as_uint(e) & 0xFFFFE000u);
            l[t] = e - h[t];
          }
          *reinterpret_cast<float4*>(ph + ((c ^ sw) << 4)) = make_float4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<float4*>(pl + ((c ^ sw) << 4)) = make_float4(l[0], l[1], l[2], l[3]);
        }
      }
      fence_async_smem();   // the tensor core reads P through the async proxy
      tc_fence_before();
      mbar_arrive(p_full);
      if (threadIdx.x == 64 && j < 8) AT_TRACE(20 + 8 * j);
    }
    // ---- O / sum -> out, log-sum-exp
    if (n > 0 && !failed) {
      if (!mbar_wait(pv_done, (uint32_t)(n - 1) & 1u)) failed = true;
      tc_fence_after();
      if (threadIdx.x == 64) AT_TRACE(8);
    }
    {
      float* xs = xch + 512;   // the sums of the two halves
      xs[half * 128 + row] = l_run;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      l_run += xs[(half ^ 1) * 128 + row];
    }
    if (!failed) {
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      // The thread owns a row, a store wants a row segment: 32 x 32 staging tile per warp (the P area is idle now),
      // then eight lanes write the 128 contiguous bytes of a row.
      float* stg = reinterpret_cast<float*>(gen + P_HI) + (warp - 2) * (32 * 36);
      const int rr0 = lane >> 3, cc = (lane & 7) * 4;
      float* dst0 = p.out + (int64_t)b * p.o_bstride + (int64_t)(q0 + quarter * 32) * p.o_tstride + (int64_t)hq * p.o_hstride + half * 64;
      const int rows_valid = qvalid - quarter * 32;   // rows of this warp inside the sequence
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t r[32];
        if (n > 0) { tmem_ld32(lane_addr + COL_O + half * 64 + c0, r); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(stg + lane * 36 + i) = make_float4(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
                                                                        __uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + rr0;
          if (rr < rows_valid) *reinterpret_cast<float4*>(dst0 + (int64_t)rr * p.o_tstride + c0 + cc) = *reinterpret_cast<const float4*>(stg + rr * 36 + cc);
        }
        __syncwarp();
      }
      if (p.lse && half == 0 && row < qvalid) p.lse[((int64_t)b * p.Hq + hq) * p.Tq + q0 + row] = l_run > 0.0f ? m_used + logf(l_run) : (p.shift ? -INFINITY : -1e30f);
      if (threadIdx.x == 64) AT_TRACE(9);
    }
  }
  if (failed) {
    atomicExch(err, 1);
    for (int i = 0; i < 4096; ++i) __nanosleep(256);   // let bulk copies that are still in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0) AT_TRACE(10);
}

// ================================================================================================ backward
// The backward pass materialises the probabilities: with both Q and dO wanted as resident 128-row operands, a
// flash-style kernel in 3xTF32 (every operand as a hi and a lo copy) does not fit tensor plus shared memory.  Per call:
//   pack    Q, dO -> [B, Hq, Tp, 128], K, V -> [B, Hkv, Tp, 128] as hi/lo tf32 copies, Tp = T rounded up to 128, the
//           padding rows zero (so that no tile crosses a sequence and padded rows add nothing to a contraction);
//   scores  (this file, tcgen05) P = exp(Q K^T - lse) under the causal mask, as hi/lo, [B, Hq, Tp, Tp];
//   scores  dS = P o (dO V^T - delta), as hi/lo;
//   dV = P^T dO and dK = dS^T Q summed over the query heads of a kv head (one contraction over (head, query)), and
//   dQ = dS K: batched products on the tensor-core GEMM, their K loops cut to the causal range.
// The score kernel is the forward kernel without its second product: the stationary operand (Q or dO) sits in tensor
// memory as the A operand, K or V streams through a ring of k-block stages (128 keys x 32 channels, hi and lo), the
// score tile is 128 x 128 in one of two tensor-memory buffers, and 256 threads (two per row) turn it into P or dS and
// store it.  Used when the sequence is causal from position 0 without an effective window (the training pass);
// other shapes keep the mma.sync kernels.
constexpr int SC_STAGES = 5;
constexpr uint32_t SC_STAGE_BYTES = 32768, SC_BARS = SC_STAGES * SC_STAGE_BYTES, SC_STG = SC_BARS + 256;
constexpr int kSmemScore = SC_STG + 8 * 32 * 36 * 4 + 1024;   // stages, barriers, one staging tile per warp, alignment slack

struct ScoreArgs {
  int mode;                 // 0: P from (Q, K, lse); 1: dS from (dO, V, P, delta)
  int Hq, Hkv, T, Tp;
  const float* rowv;        // lse (mode 0) or delta (mode 1), [B, Hq, T]
  float* out_hi; float* out_lo;   // P or dS
  const float* p_hi; const float* p_lo;   // mode 1: P
};

__global__ void __launch_bounds__(256) attn_tc_pack_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                           const float* __restrict__ dout, float* __restrict__ hi, float* __restrict__ lo, int Tp,
                                                           int64_t off_do, int64_t off_k, int64_t off_v) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nq = (int64_t)sh.B * sh.Hq * Tp, nk = (int64_t)sh.B * sh.Hkv * Tp;
  const int64_t idx = (int64_t)blockIdx.x * 8 + warp;
  if (idx >= 2 * nq + 2 * nk) return;
  const float* src = nullptr; int64_t dst;
  if (idx < 2 * nq) {
    const bool isdo = idx >= nq; const int64_t e = isdo ? idx - nq : idx;
    const int t = (int)(e % Tp); const int64_t bh = e / Tp; const int h = (int)(bh % sh.Hq); const int64_t b = bh / sh.Hq;
    if (t < sh.Tq) src = isdo ? dout + b * sh.o_bstride + (int64_t)t * sh.o_tstride + (int64_t)h * AD : q + b * sh.q_bstride + (int64_t)t * sh.q_tstride + (int64_t)h * AD;
    dst = (isdo ? off_do : 0) + e * AD;
  } else {
    const int64_t i = idx - 2 * nq; const bool isv = i >= nk; const int64_t e = isv ? i - nk : i;
    const int t = (int)(e % Tp); const int64_t bh = e / Tp; const int h = (int)(bh % sh.Hkv); const int64_t b = bh / sh.Hkv;
    if (t < sh.Tk) src = (isv ? v : k) + b * sh.kv_bstride + (int64_t)t * sh.kv_tstride + (int64_t)h * sh.kv_hstride;
    dst = (isv ? off_v : off_k) + e * AD;
  }
  float4 h4 = make_float4(0, 0, 0, 0), l4 = h4;
  if (src) {
    const float4 x = reinterpret_cast<const float4*>(src)[lane];
    split_tf32_int(x.x, h4.x, l4.x); split_tf32_int(x.y, h4.y, l4.y); split_tf32_int(x.z, h4.z, l4.z); split_tf32_int(x.w, h4.w, l4.w);
  }
  reinterpret_cast<float4*>(hi + dst)[lane] = h4;
  reinterpret_cast<float4*>(lo + dst)[lane] = l4;
}

// Batch tables of the three products: by (sequence, query head) for dQ, by (sequence, kv head) for dK / dV.
__global__ void attn_tc_batches_kernel(TcBatch* by_q, TcBatch* by_kv, int B, int Hq, int Hkv, int Tp, int64_t q_bstride, int64_t kv_bstride, int64_t kv_hstride) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int gq = Hq / Hkv;
  if (i < B * Hq) {
    const int b = i / Hq, h = i % Hq, hk = h / gq;
    TcBatch t; t.a_m = i * Tp; t.a_k = 0; t.b_n = 0; t.b_k = (b * Hkv + hk) * Tp; t.c_off = (long long)b * q_bstride + (long long)h * AD;
    by_q[i] = t;
  }
  if (i < B * Hkv) {
    const int b = i / Hkv, hk = i % Hkv;
    TcBatch t; t.a_m = 0; t.a_k = (b * Hq + hk * gq) * Tp; t.b_n = 0; t.b_k = t.a_k; t.c_off = (long long)b * kv_bstride + (long long)hk * kv_hstride;
    by_kv[i] = t;
  }
}

__global__ void __launch_bounds__(320, 1) attn_tc_score_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                                                               const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                                                               ScoreArgs p, int* err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + SC_BARS;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (SC_STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (2 * SC_STAGES + b); };
  auto s_empty = [&](int b) { return bars + 8u * (2 * SC_STAGES + 2 + b); };
  const uint32_t q_done = bars + 8u * (2 * SC_STAGES + 4);
  const uint32_t tmem_slot = bars + 8u * (2 * SC_STAGES + 5);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + SC_BARS + 8 * (2 * SC_STAGES + 5));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * AQ;   // the long tiles first
  const int h = blockIdx.y, b = blockIdx.z, hk = h / (p.Hq / p.Hkv);
  const int n = q0 / 128 + 1;                                     // key steps of 128: keys [0, q0 + 128)
  const int a_row0 = (b * p.Hq + h) * p.Tp + q0, b_row0 = (b * p.Hkv + hk) * p.Tp;
  const int total = 4 + 4 * n;                                    // ring iterations: 4 k-blocks of A, then 4 per key step

  if (threadIdx.x == 0) {
    for (int s = 0; s < SC_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(s_full(i), 1); mbar_init(s_empty(i), 256); }
    mbar_init(q_done, 256);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  bool failed = false;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer: the ring of k-block stages
    if (lane == 0) {
      for (int it = 0; it < total; ++it) {
        const int s = it % SC_STAGES;
        if (it >= SC_STAGES && !mbar_wait(empty_bar(s), (uint32_t)(it / SC_STAGES - 1) & 1u)) { failed = true; break; }
        const uint32_t st = base + (uint32_t)s * SC_STAGE_BYTES;
        mbar_expect_tx(full_bar(s), SC_STAGE_BYTES);
        if (it < 4) {
          tma_load_2d(st, &tmAh, full_bar(s), it * 32, a_row0);
          tma_load_2d(st + 16384, &tmAl, full_bar(s), it * 32, a_row0);
        } else {
          const int j = (it - 4) >> 2, kb = (it - 4) & 3;
          tma_load_2d(st, &tmBh, full_bar(s), kb * 32, b_row0 + j * 128);
          tma_load_2d(st + 16384, &tmBl, full_bar(s), kb * 32, b_row0 + j * 128);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idS = instr_desc_tf32(AQ, 128);
      if (!mbar_wait(q_done, 0u)) failed = true;
      tc_fence_after();
      for (int j = 0; j < n && !failed; ++j) {
        if (j >= 2 && !mbar_wait(s_empty(j & 1), (uint32_t)((j >> 1) - 1) & 1u)) { failed = true; break; }
        const uint32_t d = tmem_base + 256u + (uint32_t)(j & 1) * 128u;
        for (int kb = 0; kb < 4; ++kb) {
          const int it = 4 + 4 * j + kb, s = it % SC_STAGES;
          if (!mbar_wait(full_bar(s), (uint32_t)(it / SC_STAGES) & 1u)) { failed = true; break; }
          tc_fence_after();
          const uint32_t st = base + (uint32_t)s * SC_STAGE_BYTES;
          const uint64_t bh = smem_desc_sw128(st), bl = smem_desc_sw128(st + 16384);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t ah = tmem_base + kb * 32 + ks * 8, al = tmem_base + 128 + kb * 32 + ks * 8;
            umma_tf32_ts(d, al, bh + 2u * ks, idS, (kb > 0 || ks > 0) ? 1u : 0u);
            umma_tf32_ts(d, ah, bl + 2u * ks, idS, 1u);
            umma_tf32_ts(d, ah, bh + 2u * ks, idS, 1u);
          }
          umma_commit(empty_bar(s));
        }
        if (!failed) umma_commit(s_full(j & 1));
      }
    }
  } else {
    // ------------------------------------------------------------- 256 threads, two per query row
    const int quarter = warp & 3, half = ((warp - 2) >> 2) & 1;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t sw = (uint32_t)(row & 7);
    // the stationary operand: ring stages 0..3 -> tensor memory (half 0 moves hi to columns [0,128), half 1 lo to [128,256))
    for (int kb = 0; kb < 4; ++kb) {
      if (!failed && !mbar_wait(full_bar(kb), 0u)) failed = true;
      if (!failed) {
        const uint8_t* src = gen + kb * SC_STAGE_BYTES + half * 16384 + row * 128;
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 x = *reinterpret_cast<const uint4*>(src + ((c ^ sw) << 4));
          r[4 * c] = x.x; r[4 * c + 1] = x.y; r[4 * c + 2] = x.z; r[4 * c + 3] = x.w;
        }
        tmem_st32(lane_addr + half * 128 + kb * 32, r);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");          // every thread has read the stage (also met by a thread that gave up)
      if (threadIdx.x == 64) mbar_arrive(empty_bar(kb));
    }
    tmem_st_wait();
    tc_fence_before();
    mbar_arrive(q_done);
    const int q = q0 + row;
    const float rv = q < p.T ? p.rowv[((int64_t)b * p.Hq + h) * p.T + q] : 0.0f;
    const int64_t wbase = ((int64_t)(b * p.Hq + h) * p.Tp + q0 + quarter * 32) * p.Tp;   // row 0 of this warp's 32 rows
    float* stg = reinterpret_cast<float*>(gen + SC_STG) + (warp - 2) * (32 * 36);
    const int rr0 = lane >> 3, cc = (lane & 7) * 4;
    constexpr float kLog2e = 1.4426950408889634f;
    for (int j = 0; j < n && !failed; ++j) {
      if (!mbar_wait(s_full(j & 1), (uint32_t)(j >> 1) & 1u)) { failed = true; break; }
      tc_fence_after();
      const int key0 = j * 128 + half * 64;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + 256u + (uint32_t)(j & 1) * 128u + half * 64 + c0, r);
        tmem_ld_wait();
        if (c0 == 32) { tc_fence_before(); mbar_arrive(s_empty(j & 1)); }   // both halves of the row are in registers
        // The thread owns a row, a store wants a row segment: values pass through a 32 x 32 staging tile of the warp
        // (pitch 36 floats: conflict-free float4 rows), eight lanes then write the 128 contiguous bytes of a row.
        const int lim = min(q, p.T - 1) - (key0 + c0);   // columns [0, lim] are valid keys of this row
        const bool live = q < p.T;
        const int64_t gbase = wbase + key0 + c0;
        float e[32];
        if (p.mode == 0) {
          const float mneg = -rv * kLog2e;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = exp2f(fmaf(__uint_as_float(r[i]), kLog2e, mneg));
            e[i] = (live && i <= lim) ? x : 0.0f;
          }
        } else {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + rr0;
            const float4 a = *reinterpret_cast<const float4*>(p.p_hi + gbase + (int64_t)rr * p.Tp + cc);
            const float4 c = *reinterpret_cast<const float4*>(p.p_lo + gbase + (int64_t)rr * p.Tp + cc);
            *reinterpret_cast<float4*>(stg + rr * 36 + cc) = make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 pv = *reinterpret_cast<const float4*>(stg + lane * 36 + i);
            const float pa[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float x = pa[t] * (__uint_as_float(r[i + t]) - rv);
              e[i + t] = (live && i + t <= lim) ? x : 0.0f;
            }
          }
          __syncwarp();
        }
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          // part 0: hi = the value cut to tf32; part 1: lo = value - hi (exact; the tensor core reads its leading bits)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float o[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float hv = __uint_as_float(__float_as_uint(e[i + t]) & 0xFFFFE000u);
              o[t] = part == 0 ? hv : e[i + t] - hv;
            }
            *reinterpret_cast<float4*>(stg + lane * 36 + i) = make_float4(o[0], o[1], o[2], o[3]);
          }
          __syncwarp();
          float* out = part == 0 ? p.out_hi : p.out_lo;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + rr0;
            *reinterpret_cast<float4*>(out + gbase + (int64_t)rr * p.Tp + cc) = *reinterpret_cast<const float4*>(stg + rr * 36 + cc);
          }
          __syncwarp();
        }
      }
    }
  }
  if (failed) {
    atomicExch(err, 1);
    for (int i = 0; i < 4096; ++i) __nanosleep(256);   // let bulk copies that are still in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

#ifdef GN_TC_TRACE
// Development aid: the timeline of CTA (0,0,0) of the last forward launch (256 slots, SM cycles).
extern "C" int gn_debug_attn_trace(long long* host_out) {
  GN_CUDA(cudaDeviceSynchronize());
  GN_CUDA(cudaMemcpyFromSymbol(host_out, g_attn_trace, sizeof(long long) * 256));
  return GN_OK;
}
#endif

void attention_tc_enable(int on) { g_attn_tc.store(on, std::memory_order_relaxed); }

bool attention_tc_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (g_attn_tc.load(std::memory_order_relaxed) == 0) return false;
  if (sh.key_ratio < 1 || (sh.key_ratio > 1 && sh.window >= 0) || sh.q_hstride % 4 != 0 || sh.o_hstride % 4 != 0 || sh.Tk < 1) return false;
  return sh.D == AD && sh.segment_ids == nullptr && sh.Hkv > 0 && sh.Hq % sh.Hkv == 0 && sh.offset0 >= 0 && al(p0) && al(p1) && al(p2) && al(p3) &&
         sh.q_tstride % 4 == 0 && sh.q_bstride % 4 == 0 && sh.kv_tstride % 4 == 0 && sh.kv_bstride % 4 == 0 && sh.kv_hstride % 4 == 0 &&
         sh.o_tstride % 4 == 0 && sh.o_bstride % 4 == 0 && (int64_t)sh.B * std::max(sh.Tq, sh.Tk) < (1ll << 30);
}

int attention_tc_forward(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s) {
  const int64_t nq = (int64_t)sh.B * sh.Tq * sh.Hq * AD, nk = (int64_t)sh.B * sh.Tk * sh.Hkv * AD;
  float *hi = nullptr, *lo = nullptr; int* err = nullptr;
  GN_TRY(tc_attention_scratch(s, (size_t)(nq + 2 * nk), &hi, &lo, &err));
  {
    const int64_t warps = (int64_t)sh.B * sh.Tq * sh.Hq + 2 * (int64_t)sh.B * sh.Tk * sh.Hkv;
    attn_tc_split_kernel<<<(unsigned)ceil_div(warps, 8), 256, 0, s>>>(sh, q, k, v, hi, lo, nq, nq + nk);
    GN_LAUNCH_CHECK();
  }
  CUtensorMap mqh, mql, mkh, mkl, mvh, mvl;
  GN_TRY(tc_make_map3(&mqh, hi, (int64_t)sh.B * sh.Tq, (int64_t)sh.Hq * AD, (int64_t)sh.Hq * AD, AQ, AD / 32));
  GN_TRY(tc_make_map3(&mql, lo, (int64_t)sh.B * sh.Tq, (int64_t)sh.Hq * AD, (int64_t)sh.Hq * AD, AQ, AD / 32));
  GN_TRY(tc_make_map3(&mkh, hi + nq, (int64_t)sh.B * sh.Tk, (int64_t)sh.Hkv * AD, (int64_t)sh.Hkv * AD, AKV, AD / 32));
  GN_TRY(tc_make_map3(&mkl, lo + nq, (int64_t)sh.B * sh.Tk, (int64_t)sh.Hkv * AD, (int64_t)sh.Hkv * AD, AKV, AD / 32));
  GN_TRY(tc_make_map_mn3(&mvh, hi + nq + nk, (int64_t)sh.Hkv * AD, (int64_t)sh.B * sh.Tk, (int64_t)sh.Hkv * AD, AD / 32));
  GN_TRY(tc_make_map_mn3(&mvl, lo + nq + nk, (int64_t)sh.Hkv * AD, (int64_t)sh.B * sh.Tk, (int64_t)sh.Hkv * AD, AD / 32));
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(attn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFwd)); }
  AttnTc p{};
  p.B = sh.B; p.Hq = sh.Hq; p.Hkv = sh.Hkv; p.Tq = sh.Tq; p.Tk = sh.Tk; p.window = sh.window; p.offset = sh.offset0;
  p.ratio = sh.key_ratio; p.shift = sh.key_ratio > 1 ? 1 : 0;
  p.out = out; p.o_bstride = sh.o_bstride; p.o_tstride = sh.o_tstride; p.o_hstride = sh.o_hstride ? sh.o_hstride : AD; p.lse = lse;
  dim3 grid(ceil_div(sh.Tq, AQ), sh.Hq, sh.B);
  GN_REQUIRE(sh.B <= 65535 && sh.Hq <= 65535, "attention: %d sequences x %d heads exceed the grid", sh.B, sh.Hq);
  attn_tc_fwd_kernel<<<grid, 352, kSmemFwd, s>>>(mqh, mql, mkh, mkl, mvh, mvl, p, err);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// Whether the backward pass of this shape runs on the tensor-core path: causal from position 0, no effective
// window, no segment mask; its scratch (P and dS as hi/lo, 16 bytes per score) below 8 GiB.
bool attention_tc_backward_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4) {
  if (!attention_tc_ok(sh, p0, p1, p2, p3) || (reinterpret_cast<uintptr_t>(p4) & 15) != 0) return false;
  if (sh.Tq != sh.Tk || sh.offset0 != 0 || (sh.window >= 0 && sh.window < sh.Tk - 1) || sh.key_ratio != 1 || sh.q_hstride != 0 || sh.o_hstride != 0) return false;
  const int64_t Tp = (int64_t)(sh.Tq + 127) / 128 * 128;
  if ((int64_t)sh.B * sh.Hq * Tp >= (1ll << 31) / 2) return false;
  return (int64_t)sh.B * sh.Hq * Tp * Tp * 16 <= (8ll << 30);
}

int attention_tc_backward(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                          float* dq, float* dk, float* dv, int accumulate, cudaStream_t s) {
  const int Tp = (sh.Tq + 127) / 128 * 128;
  const int64_t nQ = (int64_t)sh.B * sh.Hq * Tp * AD, nK = (int64_t)sh.B * sh.Hkv * Tp * AD, nP = (int64_t)sh.B * sh.Hq * Tp * Tp;
  const int64_t off_do = nQ, off_k = 2 * nQ, off_v = 2 * nQ + nK, off_p = 2 * nQ + 2 * nK, off_ds = off_p + nP;
  const int nbq = sh.B * sh.Hq, nbk = sh.B * sh.Hkv;
  const int64_t tab_floats = ((int64_t)(nbq + nbk) * (int64_t)sizeof(TcBatch) + 3) / 4 + 64;
  float *hi = nullptr, *lo = nullptr; int* err = nullptr;
  GN_TRY(tc_attention_scratch(s, (size_t)(off_ds + nP + tab_floats), &hi, &lo, &err));
  TcBatch* by_q = reinterpret_cast<TcBatch*>(hi + (off_ds + nP + 63) / 64 * 64);
  TcBatch* by_kv = by_q + nbq;
  {
    const int64_t warps = 2 * (int64_t)sh.B * sh.Hq * Tp + 2 * (int64_t)sh.B * sh.Hkv * Tp;
    attn_tc_pack_kernel<<<(unsigned)ceil_div(warps, 8), 256, 0, s>>>(sh, q, k, v, dout, hi, lo, Tp, off_do, off_k, off_v);
    GN_LAUNCH_CHECK();
    attn_tc_batches_kernel<<<ceil_div(nbq, 256), 256, 0, s>>>(by_q, by_kv, sh.B, sh.Hq, sh.Hkv, Tp, sh.q_bstride, sh.kv_bstride, sh.kv_hstride);
    GN_LAUNCH_CHECK();
  }
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(attn_tc_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemScore)); }
  GN_REQUIRE(sh.B <= 65535 && sh.Hq <= 65535, "attention: %d sequences x %d heads exceed the grid", sh.B, sh.Hq);
  const dim3 grid(Tp / AQ, sh.Hq, sh.B);
  for (int mode = 0; mode < 2; ++mode) {
    CUtensorMap mah, mal, mbh, mbl;
    const int64_t ao = mode ? off_do : 0, bo = mode ? off_v : off_k;
    GN_TRY(tc_make_map(&mah, hi + ao, (int64_t)nbq * Tp, AD, AD, AQ));
    GN_TRY(tc_make_map(&mal, lo + ao, (int64_t)nbq * Tp, AD, AD, AQ));
    GN_TRY(tc_make_map(&mbh, hi + bo, (int64_t)nbk * Tp, AD, AD, 128));
    GN_TRY(tc_make_map(&mbl, lo + bo, (int64_t)nbk * Tp, AD, AD, 128));
    ScoreArgs a{};
    a.mode = mode; a.Hq = sh.Hq; a.Hkv = sh.Hkv; a.T = sh.Tq; a.Tp = Tp; a.rowv = mode ? delta : lse;
    a.out_hi = hi + (mode ? off_ds : off_p); a.out_lo = lo + (mode ? off_ds : off_p); a.p_hi = hi + off_p; a.p_lo = lo + off_p;
    attn_tc_score_kernel<<<grid, 320, kSmemScore, s>>>(mah, mal, mbh, mbl, a, err);
    GN_LAUNCH_CHECK();
  }
  const int gq = sh.Hq / sh.Hkv;
  // dV = P^T dO, dK = dS^T Q: rows = keys, contraction over (query head of the group, query >= key tile)
  for (int which = 0; which < 2; ++which) {
    TcBatched g{};
    const int64_t po = which ? off_ds : off_p, xo = which ? 0 : off_do;
    g.a = TcOperand{hi + po, lo + po, (int64_t)nbq * Tp, Tp, Tp, 1};
    g.b = TcOperand{hi + xo, lo + xo, (int64_t)nbq * Tp, AD, AD, 1};
    g.M = sh.Tk; g.N = AD; g.K = gq * Tp;
    g.C = which ? dk : dv; g.ldc = sh.kv_tstride; g.accumulate = accumulate;
    g.batch = by_kv; g.batches = nbk; g.k_segments = gq; g.k_seg_stride = Tp / 32; g.k_causal = 2;
    GN_TRY(gemm_tc_batched(g, s));
  }
  // dQ = dS K: rows = queries, contraction over the keys up to the tile's last query
  {
    TcBatched g{};
    g.a = TcOperand{hi + off_ds, lo + off_ds, (int64_t)nbq * Tp, Tp, Tp, 0};
    g.b = TcOperand{hi + off_k, lo + off_k, (int64_t)nbk * Tp, AD, AD, 1};
    g.M = sh.Tq; g.N = AD; g.K = Tp;
    g.C = dq; g.ldc = sh.q_tstride; g.accumulate = accumulate;
    g.batch = by_q; g.batches = nbq; g.k_segments = 0; g.k_seg_stride = 0; g.k_causal = 1;
    GN_TRY(gemm_tc_batched(g, s));
  }
  return GN_OK;
}

}  // namespace gn
