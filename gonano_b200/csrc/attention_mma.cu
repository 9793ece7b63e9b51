// head_dim 128 attention on the warp-level tensor-core instruction (mma.sync m16n8k8, tf32
// operands, float32 accumulate), forward and backward, for the prefill and the training pass
// (kernels/backend.go:167-283; scalar statement kernels/scalar/attention.go:16-245).
//
// Precision: every float32 operand x is used as hi = tf32(x) and lo = tf32(x - hi) and each
// product is three instructions, a_lo*b_hi + a_hi*b_lo + a_hi*b_hi (the small terms first), which
// keeps the products at float32 accuracy.  The tiles that serve as B operands (K and V in the forward
// and dQ kernels, Q and dO in the dK/dV kernel) are split once, when they are written to shared
// memory, into a hi tile and a lo tile; A operands are split in registers (the forward's Q tile is
// pre-split too: there is room for it).
//
// Tiling: a CTA is 8 warps; a warp owns 16 rows of the output (queries in the forward and dQ kernels,
// keys in the dK/dV kernel) and all 128 channels; the other operand streams through in tiles of 32
// rows.  All tiles sit row-major in shared memory with a pitch of 132 floats, which makes both
// fragment access patterns (row g, channel t — read with ldmatrix, four 8 x 16-byte matrices per
// instruction — and row 2t, channel g for lane = 4g + t) free of bank conflicts.
//
// The second product of each pair (P V, dS K, P^T dO, dS^T Q) contracts over the index that the
// first product's accumulator fragment holds as columns 2t, 2t+1.  Instead of moving data
// between lanes, the contraction index is permuted: slot t of the k-step stands for column 2t
// and slot t+4 for column 2t+1, on both operands, so the accumulator registers are used
// directly as the A fragment and the B fragment is read from rows 2t and 2t+1.
//
// Scores are raw q.k (the model applies no 1/sqrt(d)); a masked score is the finite -1e30 of
// the reference (kernels/scalar/attention.go:11).
#include "kernels.cuh"

namespace gn {

namespace {

constexpr float kMasked = -1e30f;
constexpr int HD = 128;       // head_dim
constexpr int LD = HD + 4;    // shared-memory pitch in floats
constexpr int NTH = 256;      // threads per CTA: 8 warps x 16 rows
constexpr int BM = 128;       // rows owned by a CTA
constexpr int BT = 32;        // rows of a streamed tile

// hi = x rounded to tf32 (nearest, ties away: add half a unit of the kept mantissa to the magnitude
// bits, clear the 13 dropped ones); lo = x - hi, exact in float32.  lo is handed to the tensor core as
// it is: the instruction reads the tf32 part of the register, so lo is cut to its leading 11 bits,
// an error of 2^-21 |x| at most.  Three integer/float instructions; the conversion instruction costs
// several times that here, and these loops are bound by instruction issue.
__device__ __forceinline__ void split(float x, uint32_t& hi, uint32_t& lo) {
  hi = (__float_as_uint(x) + 0x1000u) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// Four 8-row x 16-byte matrices from shared memory; lane L supplies the address of row L%8 of matrix L/8 and
// receives word L%4 of row L/4 of each matrix, which is the (g, t) element of a tf32 fragment.
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// The three instructions of one product form a dependent chain on the accumulator, so they are issued
// for GR independent accumulator tiles at a time, term by term.  (A second accumulator set for the small terms,
// which halves the chains, was measured: no change — the loops are not bound by these chains.)
constexpr int GR = 4;
__device__ __forceinline__ void mma3_group(float (*c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4], const uint32_t (&bh)[GR][2], const uint32_t (&bl)[GR][2]) {
#pragma unroll
  for (int i = 0; i < GR; ++i) mma(c[i], al, bh[i]);
#pragma unroll
  for (int i = 0; i < GR; ++i) mma(c[i], ah, bl[i]);
#pragma unroll
  for (int i = 0; i < GR; ++i) mma(c[i], ah, bh[i]);
}

// acc[nt] (16 x 8 tiles) += A[16 rows][128] . B[8*nt + n][128]^T.  A points at the warp's first row: a raw float32
// tile (Alo == nullptr, split here) or a pre-split pair; Bh / Bl are the pre-split tile.
// BRAW: Bh is a raw float32 tile (Bl unused) and the B fragments are split in registers, two 8-row tiles per load.
template <int NT, bool APRE, bool BRAW = false>
__device__ __forceinline__ void mm_rows(float (&acc)[NT][4], const float* A, const float* Alo, const float* Bh, const float* Bl, int lane) {
  const int mat = lane >> 3, r = lane & 7;
  const int a_off = ((mat & 1) * 8 + r) * LD + (mat >> 1) * 4;
  const uint32_t a_addr = smem_addr(A + a_off);
  const uint32_t al_addr = APRE ? smem_addr(Alo + a_off) : 0u;
  const uint32_t b_addr = BRAW ? smem_addr(Bh + ((mat >> 1) * 8 + r) * LD + (mat & 1) * 4) : smem_addr((mat < 2 ? Bh : Bl) + r * LD + (mat & 1) * 4);
#pragma unroll 2
  for (int ks = 0; ks < HD / 8; ++ks) {
    uint32_t ah[4], al[4];
    if (APRE) {
      ldsm4(ah, a_addr + ks * 32);
      ldsm4(al, al_addr + ks * 32);
    } else {
      uint32_t raw[4];
      ldsm4(raw, a_addr + ks * 32);
#pragma unroll
      for (int e = 0; e < 4; ++e) split(__uint_as_float(raw[e]), ah[e], al[e]);
    }
#pragma unroll
    for (int n0 = 0; n0 < NT; n0 += GR) {
      uint32_t bh[GR][2], bl[GR][2];
      if (BRAW) {
#pragma unroll
        for (int i = 0; i < GR; i += 2) {
          uint32_t f[4];
          ldsm4(f, b_addr + (uint32_t)(((n0 + i) * 8 * LD + ks * 8) * 4));
          split(__uint_as_float(f[0]), bh[i][0], bl[i][0]); split(__uint_as_float(f[1]), bh[i][1], bl[i][1]);
          split(__uint_as_float(f[2]), bh[i + 1][0], bl[i + 1][0]); split(__uint_as_float(f[3]), bh[i + 1][1], bl[i + 1][1]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < GR; ++i) {
          uint32_t f[4];
          ldsm4(f, b_addr + (uint32_t)(((n0 + i) * 8 * LD + ks * 8) * 4));
          bh[i][0] = f[0]; bh[i][1] = f[1]; bl[i][0] = f[2]; bl[i][1] = f[3];
        }
      }
      mma3_group(&acc[n0], ah, al, bh, bl);
    }
  }
}

// acc[nt] (16 x 8 tiles over the 128 channels) += P[16][8*NK] . B[8*NK rows][128], where P is held
// as NK accumulator fragments (columns 2t, 2t+1 of each 8-wide tile) and B (pre-split) is row-major.
template <int NK, bool BRAW = false>
__device__ __forceinline__ void mm_perm(float (&acc)[HD / 8][4], const float (&p)[NK][4], const float* Bh, const float* Bl, int g, int t) {
#pragma unroll
  for (int ks = 0; ks < NK; ++ks) {
    uint32_t ah[4], al[4];
    split(p[ks][0], ah[0], al[0]); split(p[ks][2], ah[1], al[1]); split(p[ks][1], ah[2], al[2]); split(p[ks][3], ah[3], al[3]);
    const int off = (ks * 8 + 2 * t) * LD + g;
    const uint32_t* hrow = reinterpret_cast<const uint32_t*>(Bh) + off;
    const uint32_t* lrow = reinterpret_cast<const uint32_t*>(Bl) + off;
#pragma unroll
    for (int n0 = 0; n0 < HD / 8; n0 += GR) {
      uint32_t bh[GR][2], bl[GR][2];
#pragma unroll
      for (int i = 0; i < GR; ++i) {
        if (BRAW) {
          split(__uint_as_float(hrow[(n0 + i) * 8]), bh[i][0], bl[i][0]); split(__uint_as_float(hrow[LD + (n0 + i) * 8]), bh[i][1], bl[i][1]);
        } else {
          bh[i][0] = hrow[(n0 + i) * 8]; bh[i][1] = hrow[LD + (n0 + i) * 8];
          bl[i][0] = lrow[(n0 + i) * 8]; bl[i][1] = lrow[LD + (n0 + i) * 8];
        }
      }
      mma3_group(&acc[n0], ah, al, bh, bl);
    }
  }
}

// rows of 128 floats -> row-major tile, float4 coalesced; rows >= valid are zero.
__device__ __forceinline__ void load_tile(float* S, const float* gsrc, int64_t tstride, int nrows, int valid) {
  for (int idx = threadIdx.x; idx < nrows * (HD / 4); idx += NTH) {
    const int r = idx / (HD / 4), c = (idx % (HD / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < valid) v = *reinterpret_cast<const float4*>(gsrc + (int64_t)r * tstride + c);
    *reinterpret_cast<float4*>(S + r * LD + c) = v;
  }
}
// A streamed tile (32 rows) is fetched into registers while the previous tile is being used (4 float4 per thread)
// and split into its hi and lo tiles in shared memory between two barriers.
struct TileRegs { float4 v[BT * (HD / 4) / NTH]; };
__device__ __forceinline__ void fetch_tile(TileRegs& r, const float* gsrc, int64_t tstride, int valid) {
#pragma unroll
  for (int i = 0; i < BT * (HD / 4) / NTH; ++i) {
    const int idx = threadIdx.x + i * NTH, row = idx / (HD / 4), c = (idx % (HD / 4)) * 4;
    r.v[i] = row < valid ? *reinterpret_cast<const float4*>(gsrc + (int64_t)row * tstride + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
__device__ __forceinline__ void stash_tile(const TileRegs& r, float* Sh, float* Sl) {
#pragma unroll
  for (int i = 0; i < BT * (HD / 4) / NTH; ++i) {
    const int idx = threadIdx.x + i * NTH, row = idx / (HD / 4), c = (idx % (HD / 4)) * 4;
    uint4 h, l;
    split(r.v[i].x, h.x, l.x); split(r.v[i].y, h.y, l.y); split(r.v[i].z, h.z, l.z); split(r.v[i].w, h.w, l.w);
    *reinterpret_cast<uint4*>(Sh + row * LD + c) = h;
    *reinterpret_cast<uint4*>(Sl + row * LD + c) = l;
  }
}
// the same, written as a hi tile and a lo tile
__device__ __forceinline__ void load_tile_split(float* Sh, float* Sl, const float* gsrc, int64_t tstride, int nrows, int valid) {
  for (int idx = threadIdx.x; idx < nrows * (HD / 4); idx += NTH) {
    const int r = idx / (HD / 4), c = (idx % (HD / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < valid) v = *reinterpret_cast<const float4*>(gsrc + (int64_t)r * tstride + c);
    uint4 h, l;
    split(v.x, h.x, l.x); split(v.y, h.y, l.y); split(v.z, h.z, l.z); split(v.w, h.w, l.w);
    *reinterpret_cast<uint4*>(Sh + r * LD + c) = h;
    *reinterpret_cast<uint4*>(Sl + r * LD + c) = l;
  }
}

__device__ __forceinline__ bool masked(int qpos, int kj, int window, const int32_t* seg, int seg_len, int32_t qseg) {
  bool m = kj > qpos || (window >= 0 && qpos - kj > window);
  if (!m && seg != nullptr && kj < seg_len && seg[kj] != qseg) m = true;
  return m;
}

// ------------------------------------------------------------------ forward
// CTA = 128 queries of one (batch, head); 32-key tiles; later (heavier) query tiles are scheduled first.
// A warp skips the key tiles that lie wholly after its own 16 queries.
__global__ void __launch_bounds__(NTH, 1) attn_mma_fwd_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k,
                                                              const float* __restrict__ v, float* __restrict__ out, float* __restrict__ lse) {
  pdl_trigger();
  extern __shared__ __align__(16) float smem[];
  float* Qh = smem; float* Ql = Qh + BM * LD; float* Kh = Ql + BM * LD; float* Kl = Kh + BT * LD; float* Vh = Kl + BT * LD; float* Vl = Vh + BT * LD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.y, b = bh / sh.Hq, hq = bh % sh.Hq, hk = hq / (sh.Hq / sh.Hkv);
  const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM, qvalid = min(BM, sh.Tq - q0), offset = sh.offset0;
  const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + (int64_t)hq * HD;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  load_tile_split(Qh, Ql, qg, sh.q_tstride, BM, qvalid);
  float o[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  int qpos2[2]; int32_t qseg[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    qpos2[h] = offset + q0 + warp * 16 + g + 8 * h;
    qseg[h] = (sh.segment_ids && qpos2[h] < sh.seg_len) ? sh.segment_ids[qpos2[h]] : 0;
  }
  const int warp_last = offset + q0 + warp * 16 + 15;   // last query position of this warp
  const int max_qpos = offset + q0 + qvalid - 1;
  const int k_end = min(sh.Tk, max_qpos + 1);
  int k_begin = 0;
  if (sh.window >= 0) k_begin = max(0, offset + q0 - sh.window);
  k_begin = (k_begin / BT) * BT;
  TileRegs kr, vr;
  if (k_begin < k_end) {
    fetch_tile(kr, kg + (int64_t)k_begin * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - k_begin));
    fetch_tile(vr, vg + (int64_t)k_begin * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - k_begin));
  }
  for (int kt = k_begin; kt < k_end; kt += BT) {
    __syncthreads();
    stash_tile(kr, Kh, Kl);
    stash_tile(vr, Vh, Vl);
    __syncthreads();
    if (kt + BT < k_end) {   // the next tile travels while this one is used
      fetch_tile(kr, kg + (int64_t)(kt + BT) * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - kt - BT));
      fetch_tile(vr, vg + (int64_t)(kt + BT) * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - kt - BT));
    }
    if (kt > warp_last) continue;   // every key of the tile is in this warp's future
    float s[BT / 8][4];
#pragma unroll
    for (int nt = 0; nt < BT / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
    mm_rows<BT / 8, true>(s, Qh + warp * 16 * LD, Ql + warp * 16 * LD, Kh, Kl, lane);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < BT / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1, kj = kt + nt * 8 + 2 * t + (e & 1);
        if (kj >= sh.Tk) s[nt][e] = -INFINITY;
        else if (masked(qpos2[h], kj, sh.window, sh.segment_ids, sh.seg_len, qseg[h])) s[nt][e] = kMasked;
        mx[h] = fmaxf(mx[h], s[nt][e]);
      }
    float alpha[2], rs[2] = {0.0f, 0.0f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      alpha[h] = (m_run[h] == -INFINITY) ? 0.0f : __expf(m_run[h] - m_new);
      m_run[h] = m_new;
    }
#pragma unroll
    for (int nt = 0; nt < BT / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const float p = (s[nt][e] == -INFINITY) ? 0.0f : __expf(s[nt][e] - m_run[h]);
        s[nt][e] = p; rs[h] += p;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
      l_run[h] = l_run[h] * alpha[h] + rs[h];
    }
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) { o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1]; }
    mm_perm<BT / 8>(o, s, Vh, Vl, g, t);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int qi = q0 + warp * 16 + g + 8 * h;
    if (qi >= sh.Tq) continue;
    const float inv = l_run[h] > 0.0f ? 1.0f / l_run[h] : 0.0f;
    float* og = out + (int64_t)b * sh.o_bstride + (int64_t)qi * sh.o_tstride + (int64_t)hq * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<float2*>(og + nt * 8 + 2 * t) = make_float2(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
    if (lse && t == 0) lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] = m_run[h] + logf(l_run[h]);
  }
}

// ------------------------------------------------------------------ dK / dV
// CTA = 128 keys of one (batch, kv head), 16 per warp; walks the group's query heads and 32-query
// tiles.  The warp computes S^T and dP^T (keys x queries) so that both gradients accumulate in its
// own registers: no atomics, a fixed summation order.  A warp skips the query tiles that lie wholly
// before its own 16 keys.
__global__ void __launch_bounds__(NTH, 1) attn_mma_dkv_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k,
                                                              const float* __restrict__ v, const float* __restrict__ dout,
                                                              const float* __restrict__ lse, const float* __restrict__ delta,
                                                              float* __restrict__ dk, float* __restrict__ dv, int accumulate) {
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem; float* Vs = Ks + BM * LD; float* Qh = Vs + BM * LD; float* Ql = Qh + BT * LD; float* dOh = Ql + BT * LD; float* dOl = dOh + BT * LD;
  __shared__ float lse_s[BT], delta_s[BT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.y, b = bh / sh.Hkv, hk = bh % sh.Hkv, ratio = sh.Hq / sh.Hkv;
  const int k0 = blockIdx.x * BM, kvalid = min(BM, sh.Tk - k0), offset = sh.offset0;
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)k0 * sh.kv_tstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)k0 * sh.kv_tstride;
  load_tile(Ks, kg, sh.kv_tstride, BM, kvalid);
  load_tile(Vs, vg, sh.kv_tstride, BM, kvalid);
  float adk[HD / 8][4], adv[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) { adk[nt][0] = adk[nt][1] = adk[nt][2] = adk[nt][3] = 0.0f; adv[nt][0] = adv[nt][1] = adv[nt][2] = adv[nt][3] = 0.0f; }
  int q_begin = max(0, sh.first_position(k0) - offset);
  q_begin = (q_begin / BT) * BT;
  int q_end = sh.Tq;
  if (sh.window >= 0) q_end = min(sh.Tq, k0 + kvalid - 1 + sh.window - offset + 1);
  const int kj2[2] = {k0 + warp * 16 + g, k0 + warp * 16 + g + 8};
  const int warp_first = k0 + warp * 16;   // first key of this warp
  // one flat sequence of (query head, query tile) steps, so that the next step's tiles can be fetched early
  const int n_qt = q_end > q_begin ? (q_end - q_begin + BT - 1) / BT : 0, n_steps = ratio * n_qt;
  TileRegs qr, dor;
  auto fetch_step = [&](int step) {
    const int hq = hk * ratio + step / n_qt, q0 = q_begin + (step % n_qt) * BT, qvalid = min(BT, sh.Tq - q0);
    fetch_tile(qr, q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + sh.q_head(hq), sh.q_tstride, qvalid);
    fetch_tile(dor, dout + (int64_t)b * sh.o_bstride + (int64_t)q0 * sh.o_tstride + sh.o_head(hq), sh.o_tstride, qvalid);
  };
  if (n_steps > 0) fetch_step(0);
  for (int step = 0; step < n_steps; ++step) {
    {
      const int hq = hk * ratio + step / n_qt, q0 = q_begin + (step % n_qt) * BT;
      __syncthreads();
      stash_tile(qr, Qh, Ql);
      stash_tile(dor, dOh, dOl);
      if (threadIdx.x < BT) {
        const int qi = q0 + threadIdx.x;
        lse_s[threadIdx.x] = qi < sh.Tq ? lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
        delta_s[threadIdx.x] = qi < sh.Tq ? delta[((int64_t)b * sh.Hq + hq) * sh.Tq + qi] : 0.0f;
      }
      __syncthreads();
      if (step + 1 < n_steps) fetch_step(step + 1);
      if (sh.last_key(offset + q0 + BT - 1) < warp_first) continue;   // no query of the tile sees this warp's keys
      float st[BT / 8][4], dpt[BT / 8][4];
#pragma unroll
      for (int nt = 0; nt < BT / 8; ++nt) { st[nt][0] = st[nt][1] = st[nt][2] = st[nt][3] = 0.0f; dpt[nt][0] = dpt[nt][1] = dpt[nt][2] = dpt[nt][3] = 0.0f; }
      mm_rows<BT / 8, false>(st, Ks + warp * 16 * LD, nullptr, Qh, Ql, lane);
      mm_rows<BT / 8, false>(dpt, Vs + warp * 16 * LD, nullptr, dOh, dOl, lane);
#pragma unroll
      for (int nt = 0; nt < BT / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int il = nt * 8 + 2 * t + (e & 1), qi = q0 + il, qpos = offset + qi, kj = kj2[e >> 1];
          const int32_t qseg = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
          float p = 0.0f;
          if (qi < sh.Tq && kj < sh.Tk && !masked(sh.last_key(qpos), kj, sh.window, sh.segment_ids, sh.seg_len, qseg)) p = __expf(st[nt][e] - lse_s[il]);
          st[nt][e] = p;
          dpt[nt][e] = p * (dpt[nt][e] - delta_s[il]);
        }
      mm_perm<BT / 8>(adv, st, dOh, dOl, g, t);
      mm_perm<BT / 8>(adk, dpt, Qh, Ql, g, t);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int kj = kj2[h];
    if (kj >= sh.Tk) continue;
    float* dkg = dk + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)kj * sh.kv_tstride;
    float* dvg = dv + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride + (int64_t)kj * sh.kv_tstride;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      float2 a = make_float2(adk[nt][2 * h], adk[nt][2 * h + 1]);
      float2 c = make_float2(adv[nt][2 * h], adv[nt][2 * h + 1]);
      float2* pk = reinterpret_cast<float2*>(dkg + nt * 8 + 2 * t); float2* pv = reinterpret_cast<float2*>(dvg + nt * 8 + 2 * t);
      if (accumulate) { const float2 ok = *pk, ov = *pv; a.x += ok.x; a.y += ok.y; c.x += ov.x; c.y += ov.y; }
      *pk = a; *pv = c;
    }
  }
}

// ------------------------------------------------------------------ dQ
// CTA = 128 queries of one (batch, query head), 16 per warp; walks 32-key tiles.
__global__ void __launch_bounds__(NTH, 1) attn_mma_dq_kernel(AttnShape sh, const float* __restrict__ q, const float* __restrict__ k,
                                                             const float* __restrict__ v, const float* __restrict__ dout,
                                                             const float* __restrict__ lse, const float* __restrict__ delta,
                                                             float* __restrict__ dq, int accumulate) {
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem; float* dOs = Qs + BM * LD; float* Kh = dOs + BM * LD; float* Kl = Kh + BT * LD; float* Vh = Kl + BT * LD; float* Vl = Vh + BT * LD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.y, b = bh / sh.Hq, hq = bh % sh.Hq, hk = hq / (sh.Hq / sh.Hkv);
  const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM, qvalid = min(BM, sh.Tq - q0), offset = sh.offset0;
  const float* qg = q + (int64_t)b * sh.q_bstride + (int64_t)q0 * sh.q_tstride + sh.q_head(hq);
  const float* dog = dout + (int64_t)b * sh.o_bstride + (int64_t)q0 * sh.o_tstride + sh.o_head(hq);
  const float* kg = k + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  const float* vg = v + (int64_t)b * sh.kv_bstride + (int64_t)hk * sh.kv_hstride;
  load_tile(Qs, qg, sh.q_tstride, BM, qvalid);
  load_tile(dOs, dog, sh.o_tstride, BM, qvalid);
  float lse2[2], delta2[2]; int qi2[2]; int32_t qseg[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    qi2[h] = q0 + warp * 16 + g + 8 * h;
    const bool ok = qi2[h] < sh.Tq;
    lse2[h] = ok ? lse[((int64_t)b * sh.Hq + hq) * sh.Tq + qi2[h]] : 0.0f;
    delta2[h] = ok ? delta[((int64_t)b * sh.Hq + hq) * sh.Tq + qi2[h]] : 0.0f;
    const int qpos = offset + qi2[h];
    qseg[h] = (sh.segment_ids && qpos < sh.seg_len) ? sh.segment_ids[qpos] : 0;
  }
  float adq[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) { adq[nt][0] = adq[nt][1] = adq[nt][2] = adq[nt][3] = 0.0f; }
  const int warp_last = sh.last_key(offset + q0 + warp * 16 + 15);   // the last key any query of this warp sees
  const int max_qpos = offset + q0 + qvalid - 1;
  const int k_end = min(sh.Tk, sh.last_key(max_qpos) + 1);
  int k_begin = 0;
  if (sh.window >= 0) k_begin = max(0, offset + q0 - sh.window);
  k_begin = (k_begin / BT) * BT;
  TileRegs kr, vr;
  if (k_begin < k_end) {
    fetch_tile(kr, kg + (int64_t)k_begin * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - k_begin));
    fetch_tile(vr, vg + (int64_t)k_begin * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - k_begin));
  }
  for (int kt = k_begin; kt < k_end; kt += BT) {
    __syncthreads();
    stash_tile(kr, Kh, Kl);
    stash_tile(vr, Vh, Vl);
    __syncthreads();
    if (kt + BT < k_end) {   // the next tile travels while this one is used
      fetch_tile(kr, kg + (int64_t)(kt + BT) * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - kt - BT));
      fetch_tile(vr, vg + (int64_t)(kt + BT) * sh.kv_tstride, sh.kv_tstride, min(BT, sh.Tk - kt - BT));
    }
    if (kt > warp_last) continue;   // every key of the tile is in this warp's future: p = 0
    float s[BT / 8][4], dp[BT / 8][4];
#pragma unroll
    for (int nt = 0; nt < BT / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; dp[nt][0] = dp[nt][1] = dp[nt][2] = dp[nt][3] = 0.0f; }
    mm_rows<BT / 8, false>(s, Qs + warp * 16 * LD, nullptr, Kh, Kl, lane);
    mm_rows<BT / 8, false>(dp, dOs + warp * 16 * LD, nullptr, Vh, Vl, lane);
#pragma unroll
    for (int nt = 0; nt < BT / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1, kj = kt + nt * 8 + 2 * t + (e & 1);
        float p = 0.0f;
        if (qi2[h] < sh.Tq && kj < sh.Tk && !masked(sh.last_key(offset + qi2[h]), kj, sh.window, sh.segment_ids, sh.seg_len, qseg[h])) p = __expf(s[nt][e] - lse2[h]);
        dp[nt][e] = p * (dp[nt][e] - delta2[h]);
      }
    mm_perm<BT / 8>(adq, dp, Kh, Kl, g, t);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (qi2[h] >= sh.Tq) continue;
    float* dqg = dq + (int64_t)b * sh.q_bstride + (int64_t)qi2[h] * sh.q_tstride + sh.q_head(hq);
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      float2 a = make_float2(adq[nt][2 * h], adq[nt][2 * h + 1]);
      float2* pq = reinterpret_cast<float2*>(dqg + nt * 8 + 2 * t);
      if (accumulate) { const float2 o2 = *pq; a.x += o2.x; a.y += o2.y; }
      *pq = a;
    }
  }
}

constexpr size_t kSmemAll = sizeof(float) * (size_t)((2 * BM + 4 * BT) * LD);   // the three kernels use the same amount
constexpr size_t kSmemFwd = kSmemAll, kSmemDkv = kSmemAll, kSmemDq = kSmemAll;

// ------------------------------------------------------------------ decode: the prompt shared by a group
// The G rows of a group hold identical K/V for the prompt positions (the prefill was replicated,
// model/kvcache.go:383-448), so their G x RATIO query vectors of one kv head are treated as the rows of one small
// attention problem against the first row's copy: CTA = (prompt, kv head, tile of 32 keys), two warps of 16 query rows
// each (rows >= G x RATIO are zero padding).  The tile yields one partial-result slot per (row, head): (max, sum,
// unnormalised output), merged with the per-row kernel's slots by its combine step.  The same arithmetic as the forward
// kernel above (3xTF32 products on mma.sync, softmax on the accumulator fragments); Q, K and V reach shared memory as
// raw float32 through cp.async (no registers in between, every request of the CTA in flight at once) and are split
// into their tf32 parts as fragments are formed.
constexpr int PFX_THREADS = 64;
constexpr size_t kSmemPrefix = sizeof(float) * (size_t)(32 * LD + 2 * BT * LD);
__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool valid) {
  const uint32_t d = smem_addr(dst);
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__global__ void __launch_bounds__(PFX_THREADS, 4) attn_decode_prefix_mma_kernel(const float* __restrict__ q, int64_t q_rstride, const float* __restrict__ kcache,
                                                                              const float* __restrict__ vcache, int64_t row_stride, int64_t head_stride,
                                                                              const int32_t* __restrict__ ctx_len, int Hq, int Hkv, int ratio, int window,
                                                                              int group, int prefix_len, float* __restrict__ part_acc,
                                                                              float* __restrict__ part_ms, int nslots) {
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem; float* Ks = Qs + 32 * LD; float* Vs = Ks + BT * LD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int p = blockIdx.x / Hkv, hk = blockIdx.x % Hkv, tile = blockIdx.y;
  const int NH = group * ratio;
  const int k0 = tile * BT, kvalid = min(BT, prefix_len - k0);
  const float* kb = kcache + (int64_t)p * group * row_stride + (int64_t)hk * head_stride + (int64_t)k0 * HD;
  const float* vb = vcache + (int64_t)p * group * row_stride + (int64_t)hk * head_stride + (int64_t)k0 * HD;
  // the group's query vectors: row hh = (row of the group hh / ratio, head hh % ratio of this kv head)
  for (int idx = threadIdx.x; idx < 32 * (HD / 4); idx += PFX_THREADS) {
    const int hh = idx / (HD / 4), c = (idx % (HD / 4)) * 4;
    const bool ok = hh < NH;
    cp_async16(Qs + hh * LD + c, ok ? q + (int64_t)(p * group + hh / ratio) * q_rstride + (int64_t)(hk * ratio + hh % ratio) * HD + c : q, ok);
  }
  for (int idx = threadIdx.x; idx < BT * (HD / 4); idx += PFX_THREADS) {
    const int r = idx / (HD / 4), c = (idx % (HD / 4)) * 4;
    const bool ok = r < kvalid;
    cp_async16(Ks + r * LD + c, ok ? kb + (int64_t)r * HD + c : kb, ok);
    cp_async16(Vs + r * LD + c, ok ? vb + (int64_t)r * HD + c : vb, ok);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  int qpos2[2]; bool live[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int hh = warp * 16 + g + 8 * h;
    live[h] = hh < NH;
    qpos2[h] = live[h] ? ctx_len[p * group + hh / ratio] - 1 : 0;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  float s[BT / 8][4];
#pragma unroll
  for (int nt = 0; nt < BT / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
  mm_rows<BT / 8, false, true>(s, Qs + warp * 16 * LD, nullptr, Ks, Ks, lane);
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < BT / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int h = e >> 1, kj = k0 + nt * 8 + 2 * t + (e & 1);
      if (kj >= prefix_len || (window >= 0 && qpos2[h] - kj > window)) s[nt][e] = -INFINITY;
      mx[h] = fmaxf(mx[h], s[nt][e]);
    }
  float rs[2] = {0.0f, 0.0f};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
  }
#pragma unroll
  for (int nt = 0; nt < BT / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int h = e >> 1;
      const float pj = (s[nt][e] == -INFINITY) ? 0.0f : __expf(s[nt][e] - mx[h]);
      s[nt][e] = pj; rs[h] += pj;
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
    rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
  }
  float o[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f; }
  mm_perm<BT / 8, true>(o, s, Vs, Vs, g, t);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!live[h]) continue;
    const int hh = warp * 16 + g + 8 * h;
    const int row = p * group + hh / ratio, hq = hk * ratio + hh % ratio;
    const int64_t pi = ((int64_t)row * Hq + hq) * nslots + tile;
    float* og = part_acc + pi * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) *reinterpret_cast<float2*>(og + nt * 8 + 2 * t) = make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
    if (t == 0) { part_ms[pi * 2] = mx[h]; part_ms[pi * 2 + 1] = rs[h]; }
  }
}

}  // namespace

// Row access is by float4 / float2: 16-byte aligned rows, head_dim 128.
bool attention_mma_ok(const AttnShape& sh, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return sh.D == HD && al(p0) && al(p1) && al(p2) && al(p3) && al(p4) && sh.q_tstride % 4 == 0 && sh.q_bstride % 4 == 0 && sh.kv_tstride % 4 == 0 &&
         sh.kv_bstride % 4 == 0 && sh.kv_hstride % 4 == 0 && sh.o_tstride % 4 == 0 && sh.o_bstride % 4 == 0;
}

int attention_mma_forward(const AttnShape& sh, const float* q, const float* k, const float* v, float* out, float* lse, cudaStream_t s) {
  GN_REQUIRE(sh.key_ratio == 1 && sh.q_hstride == 0 && sh.o_hstride == 0, "attention (mma.sync forward): keys counted in blocks and head-major queries are not served here");
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(attn_mma_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFwd)); }
  dim3 grid(ceil_div(sh.Tq, BM), sh.B * sh.Hq);
  attn_mma_fwd_kernel<<<grid, NTH, kSmemFwd, s>>>(sh, q, k, v, out, lse);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int attention_mma_decode_prefix(const float* q, int64_t q_rstride, const float* kcache, const float* vcache, int64_t row_stride, int64_t head_stride,
                                const int32_t* ctx_len, int rows, int Hq, int Hkv, int window, int group, int prefix_len, float* part_acc, float* part_ms,
                                int nslots, cudaStream_t s) {
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(attn_decode_prefix_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPrefix)); }
  const int tiles = (prefix_len + BT - 1) / BT;
  dim3 grid((rows / group) * Hkv, tiles);
  attn_decode_prefix_mma_kernel<<<grid, PFX_THREADS, kSmemPrefix, s>>>(q, q_rstride, kcache, vcache, row_stride, head_stride, ctx_len, Hq, Hkv, Hq / Hkv, window,
                                                                       group, prefix_len, part_acc, part_ms, nslots);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int attention_mma_backward(const AttnShape& sh, const float* q, const float* k, const float* v, const float* dout, const float* lse, const float* delta,
                           float* dq, float* dk, float* dv, int accumulate, cudaStream_t s) {
  GN_REQUIRE(sh.key_ratio == 1 || sh.window < 0, "attention (mma.sync backward): keys counted in blocks take no window");
  static PerDeviceOnce configured;
  if (configured.first()) {
    GN_CUDA(cudaFuncSetAttribute(attn_mma_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemDkv));
    GN_CUDA(cudaFuncSetAttribute(attn_mma_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemDq));
  }
  dim3 gkv(ceil_div(sh.Tk, BM), sh.B * sh.Hkv);
  attn_mma_dkv_kernel<<<gkv, NTH, kSmemDkv, s>>>(sh, q, k, v, dout, lse, delta, dk, dv, accumulate);
  GN_LAUNCH_CHECK();
  dim3 gq(ceil_div(sh.Tq, BM), sh.B * sh.Hq);
  attn_mma_dq_kernel<<<gq, NTH, kSmemDq, s>>>(sh, q, k, v, dout, lse, delta, dq, accumulate);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

}  // namespace gn
