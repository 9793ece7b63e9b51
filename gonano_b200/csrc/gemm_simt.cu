// Float32 SIMT GEMM with fused epilogues.  It serves every layout the backend
// contract needs (MatMul / MatMulTransposed, kernels/backend.go:82-93, and the
// weight-gradient form dY^T X that the reference computes through an explicit
// transpose, model/layers/linear.go:45-53) and every shape, including the
// unaligned ones of the conformance tests.  The tensor-core path
// (gemm_tcgen05.cu) takes over the large aligned products.
//
// Tiling: 128x128x16 per CTA, 256 threads, 8x8 register tile per thread split
// 4+4 in both directions so that shared-memory reads are conflict-free float4
// and global stores are 256-byte row segments.  Global loads are register
// staged one k-block ahead of the math.
#include "kernels.cuh"

namespace gn {

constexpr int BM = 128, BN = 128, BK = 16, GT = 256;

template <int EPI>
__device__ __forceinline__ void epilogue_store(const GemmArgs& g, int m, int n, float acc) {
  float* c = g.C + (int64_t)m * g.ldc + n;
  if (EPI == EPI_STORE) *c = acc;
  else if (EPI == EPI_ACCUM) *c += acc;
  else if (EPI == EPI_RESIDUAL) *c = g.aux[(int64_t)m * g.ldaux + n] + acc;
  else if (EPI == EPI_RELU2) { if (g.aux) g.aux[(int64_t)m * g.ldaux + n] = acc; float r = acc < 0.0f ? 0.0f : acc; *c = r * r; }
  else if (EPI == EPI_SOFTCAP) { *c = g.scalar * tanhf(acc * (1.0f / g.scalar)); }
  else if (EPI == EPI_RELU2_BWD) { float u = g.aux[(int64_t)m * g.ldaux + n]; *c = u > 0.0f ? acc * 2.0f * u : 0.0f; }
}

// Loads a (ROWS x BK) slab whose "row" index is the M (or N) coordinate and
// whose k index runs along K, into registers: 4 consecutive elements along
// the contiguous direction per load.
//   trans == false ("k contiguous"): element(r,k) = P[r*ld + k]
//   trans == true  ("r contiguous"): element(r,k) = P[k*ld + r]
template <bool ALIGNED>
__device__ __forceinline__ void load_slab(float (&reg)[2][4], const float* P, int64_t ld, bool r_contig, int r0, int k0, int R, int K, int tid) {
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    int idx = tid + it * GT;  // 512 float4 slots cover 128 x 16
    int r, k;
    if (!r_contig) { r = idx >> 2; k = (idx & 3) << 2; }       // 4 float4 along k per row
    else { k = idx >> 5; r = (idx & 31) << 2; }                // 32 float4 along r per k
    int gr = r0 + r, gk = k0 + k;
    if (!r_contig) {
      const float* p = P + (int64_t)gr * ld + gk;
      if (ALIGNED) {
        if (gr < R && gk < K) { float4 v = *reinterpret_cast<const float4*>(p); reg[it][0] = v.x; reg[it][1] = v.y; reg[it][2] = v.z; reg[it][3] = v.w; }
        else { reg[it][0] = reg[it][1] = reg[it][2] = reg[it][3] = 0.0f; }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) reg[it][e] = (gr < R && gk + e < K) ? p[e] : 0.0f;
      }
    } else {
      const float* p = P + (int64_t)gk * ld + gr;
      if (ALIGNED) {
        if (gr < R && gk < K) { float4 v = *reinterpret_cast<const float4*>(p); reg[it][0] = v.x; reg[it][1] = v.y; reg[it][2] = v.z; reg[it][3] = v.w; }
        else { reg[it][0] = reg[it][1] = reg[it][2] = reg[it][3] = 0.0f; }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) reg[it][e] = (gk < K && gr + e < R) ? p[e] : 0.0f;
      }
    }
  }
}
__device__ __forceinline__ void store_slab(float (*S)[BM + 4], const float (&reg)[2][4], bool r_contig, int tid) {
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    int idx = tid + it * GT;
    if (!r_contig) {
      int r = idx >> 2, k = (idx & 3) << 2;
#pragma unroll
      for (int e = 0; e < 4; ++e) S[k + e][r] = reg[it][e];
    } else {
      int k = idx >> 5, r = (idx & 31) << 2;
      *reinterpret_cast<float4*>(&S[k][r]) = make_float4(reg[it][0], reg[it][1], reg[it][2], reg[it][3]);
    }
  }
}

template <int EPI, bool ALIGNED>
__global__ void __launch_bounds__(GT, 2) gemm_simt_kernel(GemmArgs g) {
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // A slab rows are M; A is "r contiguous" when a_trans.  B slab rows are N; B is
  // "r contiguous" when !b_trans (B stored [K,N]).
  const bool a_rc = g.a_trans != 0, b_rc = g.b_trans == 0;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  float ra[2][4], rb[2][4];
  load_slab<ALIGNED>(ra, g.A, g.lda, a_rc, m0, 0, g.M, g.K, tid);
  load_slab<ALIGNED>(rb, g.B, g.ldb, b_rc, n0, 0, g.N, g.K, tid);
  store_slab(As[0], ra, a_rc, tid);
  store_slab(Bs[0], rb, b_rc, tid);
  __syncthreads();

  const int nk = (g.K + BK - 1) / BK;
  for (int kb = 0; kb < nk; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < nk) {
      load_slab<ALIGNED>(ra, g.A, g.lda, a_rc, m0, (kb + 1) * BK, g.M, g.K, tid);
      load_slab<ALIGNED>(rb, g.B, g.ldb, b_rc, n0, (kb + 1) * BK, g.N, g.K, tid);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * 4]);
      float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + ty * 4]);
      float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * 4]);
      float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + tx * 4]);
      float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kb + 1 < nk) {
      store_slab(As[cur ^ 1], ra, a_rc, tid);
      store_slab(Bs[cur ^ 1], rb, b_rc, tid);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (n < g.N) epilogue_store<EPI>(g, m, n, acc[i][j]);
    }
  }
}

template <int EPI>
static int launch_epi(const GemmArgs& g, bool aligned, cudaStream_t s) {
  dim3 grid(ceil_div(g.N, BN), ceil_div(g.M, BM));
  if (aligned) gemm_simt_kernel<EPI, true><<<grid, GT, 0, s>>>(g);
  else gemm_simt_kernel<EPI, false><<<grid, GT, 0, s>>>(g);
  GN_LAUNCH_CHECK();
  return GN_OK;
}

int gemm_simt(const GemmArgs& g, cudaStream_t s) {
  if (g.M <= 0 || g.N <= 0) return GN_OK;
  GN_REQUIRE(g.K >= 0, "gemm: negative K");
  // float4 global loads need 16-byte aligned rows in the contiguous direction.
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  bool a_ok = al(g.A) && (g.lda % 4 == 0) && ((g.a_trans ? g.M : g.K) % 4 == 0);
  bool b_ok = al(g.B) && (g.ldb % 4 == 0) && ((g.b_trans ? g.K : g.N) % 4 == 0);
  bool aligned = a_ok && b_ok;
  switch (g.epilogue) {
    case EPI_STORE: return launch_epi<EPI_STORE>(g, aligned, s);
    case EPI_ACCUM: return launch_epi<EPI_ACCUM>(g, aligned, s);
    case EPI_RESIDUAL: return launch_epi<EPI_RESIDUAL>(g, aligned, s);
    case EPI_RELU2: return launch_epi<EPI_RELU2>(g, aligned, s);
    case EPI_SOFTCAP: return launch_epi<EPI_SOFTCAP>(g, aligned, s);
    case EPI_RELU2_BWD: return launch_epi<EPI_RELU2_BWD>(g, aligned, s);
  }
  set_error("gemm: unknown epilogue %d", g.epilogue);
  return GN_ERR_INVALID;
}

}  // namespace gn
