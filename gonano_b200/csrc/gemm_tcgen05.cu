// 3xTF32 GEMM on the 5th-generation tensor cores (tcgen05), sm_100a only.
//
//   C[M,N] (epilogue)= A[M,K] * B[N,K]^T      float32 in, float32 out
//
// Every float32 operand x is split once into hi = tf32(x) and lo = tf32(x - hi);
// the product is accumulated as  lo_a*hi_b + hi_a*lo_b + hi_a*hi_b  in float32
// inside tensor memory (the lo*lo term, ~2^-22 relative, is dropped).  This keeps
// the results float32-faithful against the reference, which is float32
// throughout (guides/06-numeric-precision.md), while the multiplies run on the
// TF32 tensor pipe.
//
// Kernel structure (one 128 x BN output tile per CTA, 192 threads):
//   warp 0     TMA producer: four tiled bulk-tensor loads per k-block (A hi/lo,
//              B hi/lo; 32 floats = one 128-byte swizzle row each) into a ring of
//              shared-memory stages, completion on the stage's "full" mbarrier.
//   warp 1     allocates tensor memory; one elected lane issues the
//              tcgen05.mma.kind::tf32 instructions (M=128, N=BN, K=8; twelve per
//              k-block) and commits each stage back to its "empty" mbarrier and the
//              finished tile to the "accumulator full" mbarrier.
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp its own 32-lane
//              quarter), apply the fused epilogue, store to global memory.
// Every wait on an mbarrier is bounded; when a bound runs out the kernel raises a
// flag in global memory, drains and returns, and the host reports GN_ERR_TIMEOUT.
//
// Operands are read K-major (x W^T: both as stored) or MN-major (an operand stored [K, M] or
// [K, N], as in the weight gradient dY^T X and the data gradient dY W: read in place through the
// 128-byte swizzle with 32-byte atoms, no transposed copy).  Split copies of parameter tensors
// are cached per stream until the parameters change.
#include <cuda.h>

#include <atomic>
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

#include "kernels.cuh"
#include <unordered_map>
#include "tcgen05.cuh"

namespace gn {

namespace {


struct TcEpilogue {
  float* C; int64_t ldc;
  float* aux; int64_t ldaux;
  int epi; float scalar;
  int64_t split_stride;   // split-K: floats between the partial tiles of consecutive splits
  float* c_hi; float* c_lo; // optional: the output split for the next product (pitch ldc)
  long long* trace;   // timeline of CTA (0,0) in SM cycles when the library is built with GN_TC_TRACE, else unused
  // Grouped product (expert-major rows): group g owns group_counts[g] consecutive rows of A and C and the
  // weight rows [g * N, (g + 1) * N) of B; blockIdx.y enumerates (group, 128-row tile) pairs in group order.
  const int32_t* group_counts; int groups;
  int a_mn, b_mn;   // operand arrives MN-major (tensor map over a row-major [K, MN] source) instead of K-major
  // persistent form: the grid is one CTA per SM and CTA b works on output tiles b, b + gridDim.x, ... of tiles_total
  // (tile t = column tile t % tiles_n of row tile t / tiles_n); 0 = one tile per CTA, taken from blockIdx
  // The tiles are walked in bands of tiles_gn column tiles: inside a band the column tile runs fastest, so the CTAs
  // that are in flight together cover tiles_gn column tiles x a few row tiles and both operands are re-read from L2,
  // not from HBM (with plain row-major order a 49 k x 32768 product re-reads its 201 MB of weights for every row tile).
  int tiles_total, tiles_n, tiles_gn;
  // Batched product (one-tile form only): blockIdx.z selects an entry of `batch`.  The K loop of a tile walks
  // k_segments segments of the contraction index, k_seg_stride k-blocks apart (0 segments = the plain loop); k_causal
  // cuts each segment to the k-blocks in which a causal operand is non-zero: 1 = k < m0 + 128 (the contraction runs over
  // keys, the rows are queries), 2 = k >= m0 (the contraction runs over queries, the rows are keys).
  const TcBatch* batch; int k_segments, k_seg_stride, k_causal;
  int tma_store;   // 1: a one-tile CTA writes its tile with bulk-tensor stores through the map of C (plain stores only)
};

#ifdef GN_TC_TRACE
#define TC_TRACE(slot) do { if (ep.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ep.trace[(slot)] = clock64(); } while (0)
#else
#define TC_TRACE(slot) do { } while (0)
#endif
// trace slots: [0,256) producer issue per k-block, [256,512) MMA saw the stage full, [512,768) MMA issued,
// [768,832) epilogue saw chunk full, [832,896) epilogue drained chunk, 896 start, 897 end,
// 898 / 899 / 900 one-tile store: before staging, staged, stored (first epilogue warp)

// aux_in: the value of the aux operand at this element (residual / saved pre-activation).
__device__ __forceinline__ float epi_value(const TcEpilogue& e, float acc, float aux_in, float cold, bool& write_aux, float& auxv) {
  write_aux = false;
  switch (e.epi) {
    case EPI_STORE: return acc;
    case EPI_ACCUM: return cold + acc;
    case EPI_RESIDUAL: return aux_in + acc;
    case EPI_RELU2: { write_aux = e.aux != nullptr; auxv = acc; float r = acc < 0.0f ? 0.0f : acc; return r * r; }
    case EPI_SOFTCAP: return e.scalar * tanhf(acc * (1.0f / e.scalar));
    case EPI_RELU2_BWD: return aux_in > 0.0f ? acc * 2.0f * aux_in : 0.0f;
  }
  return acc;
}

// Two-level accumulation.  The tensor core adds into its float32 accumulator with
// truncation, so the error of one long K loop grows linearly with K (measured: 2e-5 of
// the largest output at K = 3072).  The K loop is therefore cut into chunks of
// kChunkBlocks k-blocks (384 elements: 2.5e-6 by that measurement; two chunks in flight also let the MMA warp run a
// whole K = 768 tile ahead of the epilogue warps in the persistent form); each chunk accumulates from zero in one of two tensor-memory
// buffers and the epilogue warps add the finished chunk into float32 registers with
// round-to-nearest while the next chunk is being multiplied.
constexpr int kChunkBlocks = 4;          // one-tile CTAs: 4 x 32 = 128 elements of K per chunk
constexpr int kChunkBlocksPersistent = 12;   // persistent form: 384

template <int BN, int STAGES>
struct TcSmem {
  static constexpr int A_BYTES = TBM * TBK * 4;   // 16 KB
  static constexpr int B_BYTES = BN * TBK * 4;
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // output staging of the persistent form: 32 rows x 32 columns (pitch 33) per epilogue warp, outside the pipeline
  // stages because the next tile's loads are already landing there while a tile is being stored
  static constexpr int STG_OFFSET = BAR_OFFSET + 256;
  static constexpr int STG_WARP_FLOATS = 32 * 33;
  static constexpr int STG_BYTES = (BN > 128 ? 8 : 4) * STG_WARP_FLOATS * 4;
  static constexpr int TOTAL = STG_OFFSET + STG_BYTES + 1024;  // + slack for the 1024-byte alignment
};

template <int BN, int STAGES, bool PERSIST>
__global__ void __launch_bounds__(64 + 32 * (BN > 128 ? 8 : 4), 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                                                         const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                                                         const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmCh, const __grid_constant__ CUtensorMap tmCl,
                                                         TcEpilogue ep, int M, int N, int K, int* err) {
  using S = TcSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // swizzled tiles want 1024-byte alignment
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + S::BAR_OFFSET;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + S::BAR_OFFSET + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int m0 = blockIdx.y * TBM, b_row0 = blockIdx.x * BN;
  const int n0 = blockIdx.x * BN;
  if (ep.groups > 0) {
    // find this CTA's (group, tile); surplus CTAs of the host's upper-bound grid leave before any barrier exists
    int t = blockIdx.y, g = 0, off = 0;
    for (; g < ep.groups; ++g) {
      const int c = ep.group_counts[g], tiles = (c + TBM - 1) / TBM;
      if (t < tiles) { M = off + c; break; }     // rows past the group's last one are computed but never stored
      t -= tiles; off += c;
    }
    if (g == ep.groups) return;
    m0 = off + t * TBM; b_row0 = g * N + n0;
  }
  // persistent form: this CTA's tiles are tile0, tile0 + tile_step, ...; otherwise the single tile found above
  constexpr bool persistent = PERSIST;   // a compile-time form: the one-tile kernel carries none of the tile loop
  const int tile0 = persistent ? (int)blockIdx.x : 0, tile_step = persistent ? (int)gridDim.x : 1, tile_end = persistent ? ep.tiles_total : 1;
  auto tile_origin = [&](int t, int& tm0, int& tn0, int& tb0) {
    if (persistent) {
      const int tiles_m = ep.tiles_total / ep.tiles_n, band_tiles = ep.tiles_gn * tiles_m;
      const int band = t / band_tiles, within = t - band * band_tiles;
      const int width = min(ep.tiles_gn, ep.tiles_n - band * ep.tiles_gn);   // the last band may be narrower
      tm0 = (within / width) * TBM; tn0 = (band * ep.tiles_gn + within % width) * BN; tb0 = tn0;
    }
    else { tm0 = m0; tn0 = n0; tb0 = b_row0; }
  };
  // split-K: CTA z works on k-blocks [kb0, kb0 + nk) and writes a partial tile
  const bool batched = !PERSIST && ep.batch != nullptr;
  const int zsplits = batched ? 1 : (int)gridDim.z, zi = batched ? 0 : (int)blockIdx.z;
  const int nk_total = (K + TBK - 1) / TBK;
  const int per_split = (nk_total + zsplits - 1) / zsplits;
  const int kb0 = zi * per_split;
  int nk = max(0, min(per_split, nk_total - kb0));
  int a_m_off = 0, a_k_off = 0, b_n_off = 0, b_k_off = 0, seg_nk = 1, seg_kb0 = 0, seg_stride = 0;
  if (batched) {
    const TcBatch bt = ep.batch[blockIdx.z];
    a_m_off = bt.a_m; a_k_off = bt.a_k; b_n_off = bt.b_n; b_k_off = bt.b_k;
    ep.C += bt.c_off;
    const int segs = max(1, ep.k_segments);
    seg_stride = ep.k_segments > 0 ? ep.k_seg_stride : 0;
    const int seg_total = ep.k_segments > 0 ? ep.k_seg_stride : nk_total;
    seg_kb0 = ep.k_causal == 2 ? min(seg_total, m0 / TBK) : 0;
    seg_nk = ep.k_causal == 1 ? min(seg_total, (m0 + TBM) / TBK) : seg_total - seg_kb0;
    nk = segs * seg_nk;
    if (seg_nk <= 0) { seg_nk = 1; nk = 0; }
  }
  // first element of the contraction index of this CTA's k-block number kb
  auto kcoord = [&](int kb) { return batched ? ((kb / seg_nk) * seg_stride + seg_kb0 + kb % seg_nk) * TBK : (kb0 + kb) * TBK; };
  constexpr int chunk_blocks = PERSIST ? kChunkBlocksPersistent : kChunkBlocks;
  const int nchunks = (nk + chunk_blocks - 1) / chunk_blocks;
  if (zsplits > 1) ep.C += (int64_t)blockIdx.z * ep.split_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), BN > 128 ? 8 : 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);   // two accumulator buffers of BN float32 columns (a power of two >= 32)
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  bool failed = false;
  pdl_wait();   // everything above ran in the shadow of the kernel that produces this product's operands
  if (threadIdx.x == 0) TC_TRACE(896);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int it = 0;   // k-blocks issued so far, over all of this CTA's tiles
      for (int t = tile0; t < tile_end && !failed; t += tile_step) {
        int tm0, tn0, tb0;
        tile_origin(t, tm0, tn0, tb0);
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = (uint32_t)(it / STAGES);
          if (it >= STAGES && !mbar_wait(empty_bar(s), (round - 1) & 1u)) { failed = true; break; }
          const uint32_t st = base + (uint32_t)s * S::STAGE_BYTES;
          if (it < 256) TC_TRACE(it);
          mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
          const int kc = kcoord(kb);
          if (ep.a_mn == 2) {   // the whole MN-major tile as one 3-D box (MN a multiple of 32)
            tma_load_3d(st, &tmAh, full_bar(s), 0, kc + a_k_off, (tm0 + a_m_off) / 32);
            tma_load_3d(st + S::A_BYTES, &tmAl, full_bar(s), 0, kc + a_k_off, (tm0 + a_m_off) / 32);
          } else if (ep.a_mn) {
#pragma unroll
            for (int j = 0; j < TBM / 32; ++j) {
              tma_load_2d(st + j * 4096, &tmAh, full_bar(s), tm0 + 32 * j + a_m_off, kc + a_k_off);
              tma_load_2d(st + S::A_BYTES + j * 4096, &tmAl, full_bar(s), tm0 + 32 * j + a_m_off, kc + a_k_off);
            }
          } else {
            tma_load_2d(st, &tmAh, full_bar(s), kc + a_k_off, tm0 + a_m_off);
            tma_load_2d(st + S::A_BYTES, &tmAl, full_bar(s), kc + a_k_off, tm0 + a_m_off);
          }
          if (ep.b_mn == 2) {
            tma_load_3d(st + 2 * S::A_BYTES, &tmBh, full_bar(s), 0, kc + b_k_off, (tb0 + b_n_off) / 32);
            tma_load_3d(st + 2 * S::A_BYTES + S::B_BYTES, &tmBl, full_bar(s), 0, kc + b_k_off, (tb0 + b_n_off) / 32);
          } else if (ep.b_mn) {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) {
              tma_load_2d(st + 2 * S::A_BYTES + j * 4096, &tmBh, full_bar(s), tb0 + 32 * j + b_n_off, kc + b_k_off);
              tma_load_2d(st + 2 * S::A_BYTES + S::B_BYTES + j * 4096, &tmBl, full_bar(s), tb0 + 32 * j + b_n_off, kc + b_k_off);
            }
          } else {
            tma_load_2d(st + 2 * S::A_BYTES, &tmBh, full_bar(s), kc + b_k_off, tb0 + b_n_off);
            tma_load_2d(st + 2 * S::A_BYTES + S::B_BYTES, &tmBl, full_bar(s), kc + b_k_off, tb0 + b_n_off);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_tf32(TBM, BN, ep.a_mn != 0, ep.b_mn != 0);
      int it = 0, gc = 0;   // k-blocks and chunks consumed so far, over all of this CTA's tiles
      for (int t = tile0; t < tile_end && !failed; t += tile_step) {
        for (int c = 0; c < nchunks && !failed; ++c, ++gc) {
          const int buf = gc & 1;
          // the epilogue must have drained this buffer's previous chunk
          if (gc >= 2 && !mbar_wait(acc_empty(buf), (uint32_t)(gc / 2 - 1) & 1u)) { failed = true; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
          const int kb_end = min(nk, (c + 1) * chunk_blocks);
          for (int kb = c * chunk_blocks; kb < kb_end; ++kb, ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(full_bar(s), (uint32_t)(it / STAGES) & 1u)) { failed = true; break; }
            tc_fence_after();
            if (it < 256) TC_TRACE(256 + it);
            const uint32_t st = base + (uint32_t)s * S::STAGE_BYTES;
            auto mn_desc = [&](uint32_t addr) { return kMnDesc | (uint64_t)((addr & 0x3FFFFu) >> 4); };
            const uint64_t ah = ep.a_mn ? mn_desc(st) : smem_desc_sw128(st);
            const uint64_t al = ep.a_mn ? mn_desc(st + S::A_BYTES) : smem_desc_sw128(st + S::A_BYTES);
            const uint64_t bh = ep.b_mn ? mn_desc(st + 2 * S::A_BYTES) : smem_desc_sw128(st + 2 * S::A_BYTES);
            const uint64_t bl = ep.b_mn ? mn_desc(st + 2 * S::A_BYTES + S::B_BYTES) : smem_desc_sw128(st + 2 * S::A_BYTES + S::B_BYTES);
            // advancing by one instruction's K = 8: K-major +32 bytes inside the 128-byte swizzle row (+2 in the address
            // field); MN-major the next k-group of 8, 1024 bytes on (+64)
            const uint64_t a_step = ep.a_mn ? kMnKStep : (uint64_t)((UMMA_K * 4) >> 4), b_step = ep.b_mn ? kMnKStep : (uint64_t)((UMMA_K * 4) >> 4);
#pragma unroll
            for (int k = 0; k < TBK / UMMA_K; ++k) {
              const uint64_t aa = a_step * (uint64_t)k, ba = b_step * (uint64_t)k;
              umma_tf32(d_tmem, al + aa, bh + ba, idesc, (kb > c * chunk_blocks || k > 0) ? 1u : 0u);
              umma_tf32(d_tmem, ah + aa, bl + ba, idesc, 1u);
              umma_tf32(d_tmem, ah + aa, bh + ba, idesc, 1u);
            }
            umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
            if (it < 256) TC_TRACE(512 + it);
          }
          if (!failed) umma_commit(acc_full(buf));   // this chunk's partial sums are complete
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (warps 2..5)
    // Each epilogue thread owns one accumulator row and ACC of its columns: 4 warps cover a tile
    // up to 128 columns wide, 8 warps (two column halves) a 256-column tile.
    constexpr int ACC = BN > 128 ? 128 : BN;
    const int quarter = warp & 3;    // tcgen05.ld: a warp reads lanes [32*(warp%4), +32)
    const int chalf = ((warp - 2) >> 2) * ACC;   // first column of this warp's share
    float acc[ACC];
    int gc = 0;   // chunks drained so far, over all of this CTA's tiles
    for (int t = tile0; t < tile_end && !failed; t += tile_step) {
    int tm0, tn0, tb0;
    tile_origin(t, tm0, tn0, tb0);
#pragma unroll
    for (int j = 0; j < ACC; ++j) acc[j] = 0.0f;
    for (int c = 0; c < nchunks; ++c, ++gc) {
      const int buf = gc & 1;
      if (!mbar_wait(acc_full(buf), (uint32_t)(gc / 2) & 1u)) { failed = true; break; }
      tc_fence_after();
      if (warp == 2 && lane == 0 && gc < 64) TC_TRACE(768 + gc);
#pragma unroll
      for (int c0 = 0; c0 < ACC; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + chalf + c0), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(r[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
      if (warp == 2 && lane == 0 && gc < 64) TC_TRACE(832 + gc);
    }
    if (!failed && persistent) {
      // The next tile's loads and MMAs are already running, so the tile leaves through a small staging area of its
      // own, 32 columns at a time: a thread owns a row of the accumulator, a warp store wants a row segment.
      float* stg = reinterpret_cast<float*>(gen_base + S::STG_OFFSET) + (size_t)(warp - 2) * S::STG_WARP_FLOATS;
#pragma unroll
      for (int c0 = 0; c0 < ACC; c0 += 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = acc[c0 + j];
        __syncwarp();
        const int n = tn0 + chalf + c0 + lane;
        const int64_t row0 = (int64_t)tm0 + quarter * 32;
        const int rows_valid = (int)min((int64_t)32, (int64_t)M - row0);
        if (n < N) {
          float* cp = ep.C + row0 * ep.ldc + n;
          float* ap = ep.aux ? ep.aux + row0 * ep.ldaux + n : nullptr;
          float* hp = ep.c_hi ? ep.c_hi + row0 * ep.ldc + n : nullptr;
          float* lp = ep.c_lo ? ep.c_lo + row0 * ep.ldc + n : nullptr;
          const bool reads_aux = ep.epi == EPI_RESIDUAL || ep.epi == EPI_RELU2_BWD;
          if (ep.epi == EPI_ACCUM || reads_aux) {
            // four rows at a time: first the reads of the block (the output for accumulate, the aux operand), then the
            // arithmetic and the stores, so that four loads per warp are in flight instead of one
            for (int r0 = 0; r0 < rows_valid; r0 += 4) {
              float cold[4], ax[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const bool ok = r0 + i < rows_valid;
                cold[i] = (ep.epi == EPI_ACCUM && ok) ? cp[(int64_t)(r0 + i) * ep.ldc] : 0.0f;
                ax[i] = (reads_aux && ok) ? ap[(int64_t)(r0 + i) * ep.ldaux] : 0.0f;
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int r = r0 + i;
                if (r < rows_valid) {
                  bool wa = false; float av = 0.0f;
                  const float out = epi_value(ep, stg[r * 33 + lane], ax[i], cold[i], wa, av);
                  cp[(int64_t)r * ep.ldc] = out;
                  if (hp) { float h, l; split_tf32(out, h, l); hp[(int64_t)r * ep.ldc] = h; lp[(int64_t)r * ep.ldc] = l; }
                }
              }
            }
          } else {
#pragma unroll 4
            for (int r = 0; r < rows_valid; ++r) {
              bool wa = false; float av = 0.0f;
              const float out = epi_value(ep, stg[r * 33 + lane], 0.0f, 0.0f, wa, av);
              if (wa) ap[(int64_t)r * ep.ldaux] = av;
              cp[(int64_t)r * ep.ldc] = out;
              if (hp) { float h, l; split_tf32(out, h, l); hp[(int64_t)r * ep.ldc] = h; lp[(int64_t)r * ep.ldc] = l; }
            }
          }
        }
        __syncwarp();
      }
    }
    if (!failed && !persistent && ep.tma_store) {
      // Results without a read-modify-write (plain, relu^2, softcap; K-split partial planes) leave through the
      // bulk-tensor path: each warp stages its 32 rows as 32-column blocks in the 128-byte-swizzled layout (lane = row,
      // chunk c at c ^ (row % 8): conflict-free) and one lane issues a store per block; rows and columns outside the
      // matrix are clipped by the map.  The tf32 split of the result, when asked for, follows through maps of its own.
      const uint32_t sb = base + (uint32_t)(warp - 2) * (uint32_t)(ACC * 128);
      uint8_t* sg = gen_base + (size_t)(warp - 2) * (ACC * 128);
      if (warp == 2 && lane == 0) TC_TRACE(898);
      if (ep.epi == EPI_RELU2) {
#pragma unroll
        for (int j = 0; j < ACC; ++j) { const float t = acc[j] < 0.0f ? 0.0f : acc[j]; acc[j] = t * t; }
      } else if (ep.epi == EPI_SOFTCAP) {
        const float invs = 1.0f / ep.scalar;
#pragma unroll
        for (int j = 0; j < ACC; ++j) acc[j] = ep.scalar * tanhf(acc[j] * invs);
      }
      // part 0: the value; parts 1 and 2: its tf32 hi and lo (compile-time, so that the accumulator stays in registers)
      auto store_part = [&](auto part_c, const CUtensorMap* mp) {
        constexpr int part = decltype(part_c)::value;
#pragma unroll
        for (int cb = 0; cb < ACC / 32; ++cb)
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float o[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float v = acc[cb * 32 + 4 * c + t];
              if (part == 0) o[t] = v;
              else { float h, l; split_tf32(v, h, l); o[t] = part == 1 ? h : l; }
            }
            *reinterpret_cast<float4*>(sg + cb * 4096 + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_float4(o[0], o[1], o[2], o[3]);
          }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int cb = 0; cb < ACC / 32; ++cb) tma_store_3d(mp, sb + cb * 4096, n0 + chalf + cb * 32, m0 + quarter * 32, zsplits > 1 ? (int)blockIdx.z : 0);
          tma_store_commit_wait();
        }
        __syncwarp();
      };
      store_part(std::integral_constant<int, 0>{}, &tmC);
      if (warp == 2 && lane == 0) TC_TRACE(899);
      if (ep.c_hi) {
        store_part(std::integral_constant<int, 1>{}, &tmCh);
        store_part(std::integral_constant<int, 2>{}, &tmCl);
      }
    } else if (!failed && !persistent) {
      // The accumulator row of a thread is scattered (thread = row), so it goes through shared
      // memory first: the pipeline stages are idle once the last chunk has been drained, and
      // each warp then writes whole 512-byte row segments (a thread-per-row store pattern was
      // measured at 3.5x the cost of the entire K loop).
      constexpr int PITCH = ACC + 4;           // floats per staged row: conflict-free float4 rows
      constexpr int LPR = ACC / 4;             // lanes that cover one row with float4
      constexpr int RPI = 32 / LPR;            // rows a warp writes per iteration
      float* stg = reinterpret_cast<float*>(gen_base) + (size_t)(warp - 2) * 32 * PITCH;
      if (warp == 2 && lane == 0) TC_TRACE(898);
#pragma unroll
      for (int j = 0; j < ACC; j += 4) *reinterpret_cast<float4*>(&stg[lane * PITCH + j]) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
      __syncwarp();
      if (warp == 2 && lane == 0) TC_TRACE(899);
      const bool vec_ok = (ep.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(ep.C) & 15) == 0) &&
                          (ep.aux == nullptr || ((ep.ldaux % 4 == 0) && ((reinterpret_cast<uintptr_t>(ep.aux) & 15) == 0)));
      const int col = (lane % LPR) * 4;
      const int n = n0 + chalf + col;
#pragma unroll 4
      for (int r0 = 0; r0 < 32; r0 += RPI) {
        const int r = r0 + lane / LPR;
        const int64_t m = (int64_t)m0 + quarter * 32 + r;
        if (m >= M) continue;
        const float4 v4 = *reinterpret_cast<const float4*>(&stg[r * PITCH + col]);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
        float* crow = ep.C + m * ep.ldc;
        if (vec_ok && n + 4 <= N) {
          float4 cold = make_float4(0, 0, 0, 0);
          if (ep.epi == EPI_ACCUM) cold = *reinterpret_cast<const float4*>(crow + n);
          float4 a4 = make_float4(0, 0, 0, 0);
          if (ep.epi == EPI_RESIDUAL || ep.epi == EPI_RELU2_BWD) a4 = *reinterpret_cast<const float4*>(ep.aux + m * ep.ldaux + n);
          const float co[4] = {cold.x, cold.y, cold.z, cold.w}, ax[4] = {a4.x, a4.y, a4.z, a4.w};
          float out[4], av[4];
          bool wa = false;
#pragma unroll
          for (int e = 0; e < 4; ++e) out[e] = epi_value(ep, v[e], ax[e], co[e], wa, av[e]);
          if (wa) *reinterpret_cast<float4*>(ep.aux + m * ep.ldaux + n) = make_float4(av[0], av[1], av[2], av[3]);
          *reinterpret_cast<float4*>(crow + n) = make_float4(out[0], out[1], out[2], out[3]);
          if (ep.c_hi) {
            float h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32(out[e], h[e], l[e]);
            *reinterpret_cast<float4*>(ep.c_hi + m * ep.ldc + n) = make_float4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<float4*>(ep.c_lo + m * ep.ldc + n) = make_float4(l[0], l[1], l[2], l[3]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (n + e < N) {
              bool wa = false; float av = 0.0f;
              const float cold = (ep.epi == EPI_ACCUM) ? crow[n + e] : 0.0f;
              const float ax = (ep.epi == EPI_RESIDUAL || ep.epi == EPI_RELU2_BWD) ? ep.aux[m * ep.ldaux + n + e] : 0.0f;
              const float out = epi_value(ep, v[e], ax, cold, wa, av);
              if (wa) ep.aux[m * ep.ldaux + n + e] = av;
              crow[n + e] = out;
              if (ep.c_hi) { float h, l; split_tf32(out, h, l); ep.c_hi[m * ep.ldc + n + e] = h; ep.c_lo[m * ep.ldc + n + e] = l; }
            }
          }
        }
      }
    }
    if (warp == 2 && lane == 0) TC_TRACE(900);
    }   // tiles
  }
  if (failed) {
    atomicExch(err, 1);
    // give bulk copies that are still in flight time to land before the CTA goes away
    for (int i = 0; i < 4096; ++i) __nanosleep(256);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TC_TRACE(897);
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------ few-row products (the rollout's decode step)
//
//   C[rows, N] = X[rows, K] * W[N, K]^T   rows in blocks of at most 256 per CTA
//
// With a few hundred rows or fewer a product of the decode step is bound by streaming its weights, not by the
// multiplies.  This form therefore swaps the operands of the tensor-core instruction: a slab of 128 WEIGHT rows is the
// 128-row A operand and the activation rows are the (narrow) B operand, so that every CTA streams a different 16 KB of
// weights per k-block and the whole grid pulls on HBM at once, the K dimension being split over CTAs as well.  The
// weights are read as raw float32, once: the producer warp fetches each 128 x 32 tile with one bulk-tensor copy, four
// converter warps rewrite it in place as hi = tf32(w) and write lo = tf32(w - hi) beside it (the same split the
// cached-copy path stores in HBM, so 4 bytes per weight cross HBM instead of 8 and no split copy is kept), and the
// issuing thread multiplies lo*hi + hi*lo + hi*hi into tensor memory.  The activations arrive already split.
// The accumulator holds C^T: lane = weight row n, column = activation row m; each thread of the four epilogue warps
// (the converter warps, once the K loop is done) owns one n and stores along m, 32 consecutive n per warp store.
//
// With programmatic dependent launch the weight tiles of the first stages are requested BEFORE the wait on the
// preceding kernel (weights do not depend on it), so they stream in while the small kernel in front of the product
// still runs; the activation tiles follow after the wait.
//
// grid = (row blocks, weight slabs, K splits): the row blocks of one weight tile are neighbours in launch order, so
// the tile is fetched from HBM once and found in L2 by the others.  splits > 1 leaves partial planes [split][rows][N] that the
// consumer (or splitk_reduce_kernel) sums in a fixed order.
constexpr int SK_W_BYTES = TBM * TBK * 4;        // 16 KB: one raw weight tile, and as much again for its lo part
constexpr int SK_MAX_STAGES = 6;
struct SkinnyArgs {
  TcEpilogue ep;
  int M, N, K;          // activation rows, weight rows, inner dimension
  int block_rows;       // activation rows per CTA (a multiple of 16, at most 256)
  int rowsN;            // UMMA N of a full row block: min(M, block_rows) rounded up to 16
  int nk_per_split;     // k-blocks per K split
  int stages;
  int tmem_cols;        // power of two >= max(32, rowsN)
  int prefetch;         // 1: the weights may be requested before the wait on the preceding kernel
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Epilogue of the few-row form for one thread (= one weight row n): 16 accumulator columns (= activation rows) at a
// time out of tensor memory, the fused epilogue, one 4-byte store per row; the 32 lanes of a warp write 32
// consecutive n of the same row.  SPLIT also writes the tf32 split of the result (c_hi / c_lo may still be null).
template <int EPI, bool SPLIT>
__device__ __forceinline__ void skinny_store(const TcEpilogue& e, float* Cb, uint32_t tmem_base, int quarter, int n, int m0, int un, int M, int N, bool have) {
  for (int c0 = 0; c0 < un; c0 += 16) {
    uint32_t r[16];
    if (have) { tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r); tmem_ld_wait(); }
    else {
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = 0u;
    }
    if (n >= N) continue;
    const int64_t mfirst = (int64_t)m0 + c0;
    const int valid = (int)min((int64_t)16, (int64_t)M - mfirst);
    float* cp = Cb + mfirst * e.ldc + n;
    const float* ap = (EPI == EPI_RESIDUAL || EPI == EPI_RELU2_BWD) ? e.aux + mfirst * e.ldaux + n : nullptr;
    float cold[16];
    if (EPI == EPI_ACCUM || EPI == EPI_RESIDUAL || EPI == EPI_RELU2_BWD) {   // the reads of the block first, so that they are in flight together
#pragma unroll
      for (int j = 0; j < 16; ++j) cold[j] = (j < valid) ? (EPI == EPI_ACCUM ? cp[(int64_t)j * e.ldc] : ap[(int64_t)j * e.ldaux]) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < valid) {
        const float acc = __uint_as_float(r[j]);
        float out;
        if (EPI == EPI_STORE) out = acc;
        else if (EPI == EPI_ACCUM || EPI == EPI_RESIDUAL) out = cold[j] + acc;
        else if (EPI == EPI_RELU2) { if (e.aux) e.aux[(mfirst + j) * e.ldaux + n] = acc; const float t = acc < 0.0f ? 0.0f : acc; out = t * t; }
        else if (EPI == EPI_SOFTCAP) out = e.scalar * tanhf(acc * (1.0f / e.scalar));
        else out = cold[j] > 0.0f ? acc * 2.0f * cold[j] : 0.0f;
        cp[(int64_t)j * e.ldc] = out;
        if (SPLIT && e.c_hi) { float h, l; split_tf32(out, h, l); e.c_hi[(mfirst + j) * e.ldc + n] = h; e.c_lo[(mfirst + j) * e.ldc + n] = l; }
      }
    }
  }
}

__global__ void __launch_bounds__(192, 2) gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmXh,
                                                             const __grid_constant__ CUtensorMap tmXl, SkinnyArgs p, int* err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const int XB = p.rowsN * TBK * 4;                       // bytes of one activation tile (hi or lo)
  const int stage_bytes = 2 * SK_W_BYTES + 2 * XB;
  const uint32_t bars = base + (uint32_t)p.stages * stage_bytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto conv_bar = [&](int s) { return bars + 8u * (SK_MAX_STAGES + s); };
  auto empty_bar = [&](int s) { return bars + 8u * (2 * SK_MAX_STAGES + s); };
  const uint32_t acc_bar = bars + 8u * (3 * SK_MAX_STAGES);
  const uint32_t tmem_slot = bars + 8u * (3 * SK_MAX_STAGES + 1);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (size_t)p.stages * stage_bytes + 8 * (3 * SK_MAX_STAGES + 1));

  const TcEpilogue& ep = p.ep;
  if (threadIdx.x == 0) TC_TRACE(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * TBM;
  const int nk_total = (p.K + TBK - 1) / TBK;
  const int kb0 = (int)blockIdx.z * p.nk_per_split;
  const int nk = max(0, min(p.nk_per_split, nk_total - kb0));
  const int m0 = (int)blockIdx.x * p.block_rows;
  const int rows_here = min(p.block_rows, p.M - m0);
  const int un = (rows_here + 15) & ~15;                  // UMMA N of this row block

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(conv_bar(s), 4); mbar_init(empty_bar(s), 1); }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) { tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  bool failed = false;
  if (threadIdx.x == 0) TC_TRACE(1);
  pdl_trigger();   // the next kernel may set up (and request its own weights) while this one runs

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint32_t tx = (uint32_t)(SK_W_BYTES + 2 * XB);
      const int pre = p.prefetch ? min(nk, p.stages) : 0;
      for (int kb = 0; kb < pre; ++kb) {          // weights of the first stages: independent of the preceding kernel
        const uint32_t st = base + (uint32_t)kb * stage_bytes;
        mbar_expect_tx(full_bar(kb), tx);
        tma_load_2d(st, &tmW, full_bar(kb), (kb0 + kb) * TBK, n0);
      }
      TC_TRACE(2);
      pdl_wait();
      TC_TRACE(3);
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % p.stages;
        const uint32_t st = base + (uint32_t)s * stage_bytes;
        if (kb >= pre) {
          if (kb >= p.stages && !mbar_wait(empty_bar(s), (uint32_t)(kb / p.stages - 1) & 1u)) { failed = true; break; }
          mbar_expect_tx(full_bar(s), tx);
          tma_load_2d(st, &tmW, full_bar(s), (kb0 + kb) * TBK, n0);
        }
        tma_load_2d(st + 2 * SK_W_BYTES, &tmXh, full_bar(s), (kb0 + kb) * TBK, m0);
        tma_load_2d(st + 2 * SK_W_BYTES + XB, &tmXl, full_bar(s), (kb0 + kb) * TBK, m0);
        if (kb < 32) TC_TRACE(16 + kb);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_tf32(TBM, un);
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % p.stages;
        if (!mbar_wait(conv_bar(s), (uint32_t)(kb / p.stages) & 1u)) { failed = true; break; }
        tc_fence_after();
        if (kb < 32) TC_TRACE(48 + kb);
        const uint32_t st = base + (uint32_t)s * stage_bytes;
        const uint64_t wh = smem_desc_sw128(st), wl = smem_desc_sw128(st + SK_W_BYTES);
        const uint64_t xh = smem_desc_sw128(st + 2 * SK_W_BYTES), xl = smem_desc_sw128(st + 2 * SK_W_BYTES + XB);
#pragma unroll
        for (int k = 0; k < TBK / UMMA_K; ++k) {
          const uint64_t adv = (uint64_t)((UMMA_K * 4) >> 4) * (uint64_t)k;
          umma_tf32(tmem_base, wl + adv, xh + adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_tf32(tmem_base, wh + adv, xl + adv, idesc, 1u);
          umma_tf32(tmem_base, wh + adv, xh + adv, idesc, 1u);
        }
        umma_commit(empty_bar(s));
        if (kb < 32) TC_TRACE(80 + kb);
      }
      if (!failed) umma_commit(acc_bar);
    }
  } else {
    // ------------------------------------------------------------- converters, then epilogue (warps 2..5)
    const int ct = threadIdx.x - 64;   // 0..127
    for (int kb = 0; kb < nk && !failed; ++kb) {
      const int s = kb % p.stages;
      if (!mbar_wait(full_bar(s), (uint32_t)(kb / p.stages) & 1u)) { failed = true; break; }
      if (ct == 0 && kb < 32) TC_TRACE(112 + kb);
      float4* wt = reinterpret_cast<float4*>(gen_base + (size_t)s * stage_bytes);
      float4* wlo = reinterpret_cast<float4*>(gen_base + (size_t)s * stage_bytes + SK_W_BYTES);
#pragma unroll
      for (int i = 0; i < SK_W_BYTES / 16 / 128; ++i) {
        const int c = i * 128 + ct;
        const float4 v = wt[c];
        float4 h, l;
        split_tf32_int(v.x, h.x, l.x); split_tf32_int(v.y, h.y, l.y); split_tf32_int(v.z, h.z, l.z); split_tf32_int(v.w, h.w, l.w);
        wt[c] = h; wlo[c] = l;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads these tiles through the async proxy
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(conv_bar(s)) : "memory");
      if (ct == 0 && kb < 32) TC_TRACE(144 + kb);
    }
    if (!failed && nk > 0 && !mbar_wait(acc_bar, 0u)) failed = true;
    if (ct == 0) TC_TRACE(4);
    if (!failed) {
      tc_fence_after();
      const int quarter = warp & 3;
      const int n = n0 + quarter * 32 + lane;
      const TcEpilogue& e = ep;
      float* Cb = e.C + (gridDim.z > 1 ? (int64_t)blockIdx.z * e.split_stride : 0);
      // One specialised store loop per epilogue kind, selected once per CTA: the loop bodies stay small and straight.
      switch (e.epi) {
        case EPI_STORE: if (e.c_hi) skinny_store<EPI_STORE, true>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0);
                        else skinny_store<EPI_STORE, false>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0);
                        break;
        case EPI_ACCUM: skinny_store<EPI_ACCUM, false>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0); break;
        case EPI_RESIDUAL: if (e.c_hi) skinny_store<EPI_RESIDUAL, true>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0);
                           else skinny_store<EPI_RESIDUAL, false>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0);
                           break;
        case EPI_RELU2: skinny_store<EPI_RELU2, true>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0); break;
        case EPI_SOFTCAP: skinny_store<EPI_SOFTCAP, false>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0); break;
        default: skinny_store<EPI_RELU2_BWD, false>(e, Cb, tmem_base, quarter, n, m0, un, p.M, p.N, nk > 0); break;
      }
    }
  }
  if (threadIdx.x == 64) TC_TRACE(5);
  if (failed) {
    atomicExch(err, 1);
    for (int i = 0; i < 4096; ++i) __nanosleep(256);   // let bulk copies that are still in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TC_TRACE(6);
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

// ------------------------------------------------------------------ operand split
// src [rows, cols] (pitch ld) -> hi, lo [rows, cols] (pitch ldd)
__global__ void __launch_bounds__(256) split_kernel(const float* __restrict__ src, int64_t ld, float* __restrict__ hi, float* __restrict__ lo, int64_t ldd,
                                                    int64_t rows, int cols) {
  const int cv = cols >> 2;  // cols is a multiple of 4
  int64_t total = rows * cv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / cv; int c = (int)(i % cv) * 4;
    float4 v = *reinterpret_cast<const float4*>(src + r * ld + c);
    float4 h, l;
    split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
    *reinterpret_cast<float4*>(hi + r * ldd + c) = h;
    *reinterpret_cast<float4*>(lo + r * ldd + c) = l;
  }
}
// src [rows, cols] (pitch ld) -> hi, lo [cols, rows_padded] (pitch ldd), zero-filled padding
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ src, int64_t ld, float* __restrict__ hi, float* __restrict__ lo,
                                                              int64_t ldd, int64_t rows, int cols) {
  __shared__ float th[32][33], tl[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t r0 = (int64_t)blockIdx.y * 32; const int c0 = blockIdx.x * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t r = r0 + ty + 8 * i; int c = c0 + tx;
    float h = 0.0f, l = 0.0f;
    if (r < rows && c < cols) split_tf32(src[r * ld + c], h, l);
    th[ty + 8 * i][tx] = h; tl[ty + 8 * i][tx] = l;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int c = c0 + ty + 8 * i; int64_t r = r0 + tx;
    if (c < cols && r < ldd) { hi[(int64_t)c * ldd + r] = th[tx][ty + 8 * i]; lo[(int64_t)c * ldd + r] = tl[tx][ty + 8 * i]; }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
long long* g_trace = nullptr;   // device buffer of 1024 slots (GN_TC_TRACE builds)
std::mutex g_mu;

struct SplitBuf { float* hi = nullptr; float* lo = nullptr; size_t floats = 0; int64_t ld = 0; bool fresh = true; bool mn = false; };

// Everything a product needs beyond its operands lives here, one instance per (device, stream): products issued on
// different streams or devices never share scratch, and the bounded-wait flag is read on the stream that raised it.
struct GemmState {
  int device = 0;
  cudaStream_t stream = nullptr;
  int* err_flag = nullptr;
  // Cached splits of parameter tensors: key = (pointer, rows, cols, transposed).
  std::map<std::tuple<const void*, int64_t, int64_t, int>, SplitBuf> statics;
  SplitBuf dyn[2];  // scratch for the activation operands (A and B of the current product)
  struct { const void* src = nullptr; int64_t ld = 0, rows = 0, cols = 0; bool valid = false; } last_a;   // what dyn[0] holds
  float* splitk_ws = nullptr;
  size_t splitk_floats = 0;
  SplitBuf attn;    // tf32 splits of Q, K, V (and dO) for the attention kernels
  // options (gn_ctx_set_option)
  int persistent_ctas = -1;   // CTAs of the persistent form: -1 = one per SM, 0 = form off, n = run it on n CTAs
  bool pdl = true;            // programmatic dependent launch of the products
  bool mn = true;             // read [K, M] / [K, N] operands MN-major instead of transposing them while splitting
  bool mn3d = true;           // one 3-D TMA box per MN-major tile instead of one 2-D box per 32 columns
  bool tma_store = true;      // one-tile CTAs store plain results through a tensor map of C
  bool wide_split = true;     // 128 x 256 tiles with a K split for outputs of half a wave to a wave of 128-wide tiles
};
std::map<std::pair<int, cudaStream_t>, GemmState*> g_states;

// g_mu held by the caller.
int state_for(cudaStream_t s, GemmState** out) {
  int device = 0;
  GN_CUDA(cudaGetDevice(&device));
  auto key = std::make_pair(device, s);
  auto it = g_states.find(key);
  if (it == g_states.end()) {
    GemmState* st = new GemmState();
    st->device = device; st->stream = s;
    GN_CUDA(cudaMalloc((void**)&st->err_flag, sizeof(int)));
    GN_CUDA(cudaMemsetAsync(st->err_flag, 0, sizeof(int), s));
    it = g_states.emplace(key, st).first;
  }
  *out = it->second;
  return GN_OK;
}
int persistent_ctas(const GemmState& st) { return st.persistent_ctas < 0 ? num_sms() : st.persistent_ctas; }

int ensure_init() {
  if (g_encode) return GN_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  GN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  GN_REQUIRE(fn != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available from this driver");
  g_encode = (EncodeTiledFn)fn;
  return GN_OK;
}

// A tensor map depends on the address, the extents, the pitch and the box alone, never on the data, and the same few thousand
// (array, shape) pairs come back every step: encoded maps are kept per host thread and copied out (128 bytes) instead of being
// encoded again (several per product, which shows where launches are the bound: the optimizer step, the eager decode loop).
struct MapKey {
  const void* base; int64_t a, b, c; int d, e, kind;
  bool operator==(const MapKey& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d && e == o.e && kind == o.kind; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    auto mix = [&](uint64_t v) { h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2); };
    mix((uint64_t)k.a); mix((uint64_t)k.b); mix((uint64_t)k.c); mix(((uint64_t)(uint32_t)k.d << 32) | (uint32_t)k.e); mix((uint64_t)k.kind);
    return (size_t)h;
  }
};
template <typename F>
int cached_map(CUtensorMap* map, const MapKey& key, F&& encode) {
  thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  auto it = maps.find(key);
  if (it != maps.end()) { *map = it->second; return GN_OK; }
  GN_TRY(encode());
  if (maps.size() >= (1u << 16)) maps.clear();
  maps.emplace(key, *map);
  return GN_OK;
}

int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  return cached_map(map, MapKey{base, rows, k, ld, box_rows, 0, 0}, [&]() -> int {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)TBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with %d (rows %lld, k %lld, ld %lld)", (int)r, (long long)rows, (long long)k, (long long)ld); return GN_ERR_CUDA; }
  return GN_OK;
  });
}

// 3-D map over the same array, for mn a multiple of 32: dimensions {32 consecutive mn, k, mn / 32}; a box
// {32, 32, groups} is a whole MN-major tile (its MN groups land 4096 bytes apart, as the four or eight 2-D boxes do),
// so a k-block costs one copy per operand half instead of up to twelve.
int make_map_mn3(CUtensorMap* map, const float* base, int64_t mn, int64_t k, int64_t ld, int groups) {
  return cached_map(map, MapKey{base, mn, k, ld, groups, 0, 1}, [&]() -> int {
  cuuint64_t dims[3] = {32, (cuuint64_t)k, (cuuint64_t)(mn / 32)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(float), 32 * sizeof(float)};
  cuuint32_t box[3] = {32, (cuuint32_t)TBK, (cuuint32_t)groups};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (MN-major, 3-D) failed with %d (mn %lld, k %lld, ld %lld)", (int)r, (long long)mn, (long long)k, (long long)ld); return GN_ERR_CUDA; }
  return GN_OK;
  });
}

// 2-D map over a row-major [k, mn] array (pitch ld floats): a box [32 mn x 32 k] is one MN group of the MN-major tile above.
int make_map_mn(CUtensorMap* map, const float* base, int64_t mn, int64_t k, int64_t ld) {
  return cached_map(map, MapKey{base, mn, k, ld, 0, 0, 2}, [&]() -> int {
  cuuint64_t dims[2] = {(cuuint64_t)mn, (cuuint64_t)k};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {32, (cuuint32_t)TBK};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (MN-major) failed with %d (mn %lld, k %lld, ld %lld)", (int)r, (long long)mn, (long long)k, (long long)ld); return GN_ERR_CUDA; }
  return GN_OK;
  });
}

int ensure_buf(SplitBuf& b, size_t floats) {
  if (floats <= b.floats) return GN_OK;
  if (b.hi) { cudaFree(b.hi); cudaFree(b.lo); b.hi = b.lo = nullptr; b.floats = 0; }
  cudaError_t e1 = cudaMalloc((void**)&b.hi, floats * sizeof(float));
  cudaError_t e2 = e1 == cudaSuccess ? cudaMalloc((void**)&b.lo, floats * sizeof(float)) : e1;
  if (e1 != cudaSuccess || e2 != cudaSuccess) { set_error("tcgen05 gemm: cannot allocate %zu-byte operand split buffers", 2 * floats * sizeof(float)); return GN_ERR_NOMEM; }
  b.floats = floats;
  return GN_OK;
}

// Produces K-major hi/lo copies of an operand.  `rows` x `k` is the logical operand
// (rows = M or N).  stored_transposed: the source is stored [k, rows] (pitch ld).
int split_operand(GemmState& gs, const float* src, int64_t ld, int64_t rows, int64_t k, bool stored_transposed, bool is_static, int which, SplitBuf& out,
                  cudaStream_t s, bool allow_mn = false) {
  if (stored_transposed && allow_mn && !is_static && rows % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    // The source is row-major [k, rows]: keep it that way (a plain split, no transpose) and let the tensor core read it MN-major.
    SplitBuf* target = &gs.dyn[which];
    GN_TRY(ensure_buf(*target, (size_t)k * rows));
    target->ld = rows; target->mn = true;
    const int64_t total = k * (rows / 4);
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)num_sms() * 16);
    split_kernel<<<std::max(blocks, 1), 256, 0, s>>>(src, ld, target->hi, target->lo, rows, k, (int)rows);
    GN_LAUNCH_CHECK();
    out = *target;
    return GN_OK;
  }
  const int64_t kp = (k + 3) / 4 * 4;
  auto key = std::make_tuple((const void*)src, rows, k, stored_transposed ? 1 : 0);
  SplitBuf buf;
  if (is_static) {
    auto it = gs.statics.find(key);
    if (it != gs.statics.end()) {
      if (it->second.fresh) { out = it->second; return GN_OK; }
      buf = it->second;          // the parameters changed: split again into the buffers this entry already owns
    }
  }
  SplitBuf* target = is_static ? &buf : &gs.dyn[which];
  GN_TRY(ensure_buf(*target, (size_t)rows * kp));
  target->ld = kp; target->mn = false;
  if (!stored_transposed) {
    int64_t total = rows * (k / 4);
    int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)num_sms() * 16);
    split_kernel<<<std::max(blocks, 1), 256, 0, s>>>(src, ld, target->hi, target->lo, kp, rows, (int)k);
  } else {
    dim3 grid(ceil_div(rows, 32), ceil_div(kp, 32));   // source is [k, rows]: x over its columns (= rows), y over its rows (= k)
    split_transpose_kernel<<<grid, 256, 0, s>>>(src, ld, target->hi, target->lo, kp, k, (int)rows);
  }
  GN_LAUNCH_CHECK();
  target->fresh = true;
  if (is_static) gs.statics[key] = *target;
  out = *target;
  return GN_OK;
}

// Split-K second pass: C = epilogue(sum over splits of the partial tiles), in a fixed order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int splits, int64_t split_stride, TcEpilogue ep, int M, int N) {
  pdl_trigger();
  pdl_wait();
  const int nv = N >> 2;   // N is a multiple of 4 on this path
  const int64_t total = (int64_t)M * nv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / nv; const int n = (int)(i % nv) * 4;
    float4 acc = *reinterpret_cast<const float4*>(part + m * N + n);
    for (int z = 1; z < splits; ++z) {
      const float4 p = *reinterpret_cast<const float4*>(part + (int64_t)z * split_stride + m * N + n);
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    float* crow = ep.C + m * ep.ldc + n;
    const float v[4] = {acc.x, acc.y, acc.z, acc.w};
    float out[4], av[4]; bool wa = false;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float cold = (ep.epi == EPI_ACCUM) ? crow[e] : 0.0f;
      const float ax = (ep.epi == EPI_RESIDUAL || ep.epi == EPI_RELU2_BWD) ? ep.aux[m * ep.ldaux + n + e] : 0.0f;
      out[e] = epi_value(ep, v[e], ax, cold, wa, av[e]);
    }
    if (wa) { for (int e = 0; e < 4; ++e) ep.aux[m * ep.ldaux + n + e] = av[e]; }
    for (int e = 0; e < 4; ++e) crow[e] = out[e];
    if (ep.c_hi) {
      for (int e = 0; e < 4; ++e) { float h, l; split_tf32(out[e], h, l); ep.c_hi[m * ep.ldc + n + e] = h; ep.c_lo[m * ep.ldc + n + e] = l; }
    }
  }
}


template <int BN, int STAGES>
int launch_tc(GemmState& gs, const SplitBuf& a, const SplitBuf& b, const TcEpilogue& ep_in, int M, int N, int K, int splits, cudaStream_t s, Partials* leave = nullptr) {
  using S = TcSmem<BN, STAGES>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    GN_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL - S::STG_BYTES));
    GN_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
  }
  CUtensorMap mah, mal, mbh, mbl;
  const bool a3 = a.mn && gs.mn3d && M % 32 == 0;
  if (a3) { GN_TRY(make_map_mn3(&mah, a.hi, M, K, a.ld, TBM / 32)); GN_TRY(make_map_mn3(&mal, a.lo, M, K, a.ld, TBM / 32)); }
  else if (a.mn) { GN_TRY(make_map_mn(&mah, a.hi, M, K, a.ld)); GN_TRY(make_map_mn(&mal, a.lo, M, K, a.ld)); }
  else { GN_TRY(make_map(&mah, a.hi, M, K, a.ld, TBM)); GN_TRY(make_map(&mal, a.lo, M, K, a.ld, TBM)); }
  const int brows = ep_in.groups > 0 ? ep_in.groups * N : N;
  const bool b3 = b.mn && gs.mn3d && brows % 32 == 0;
  if (b3) { GN_TRY(make_map_mn3(&mbh, b.hi, brows, K, b.ld, BN / 32)); GN_TRY(make_map_mn3(&mbl, b.lo, brows, K, b.ld, BN / 32)); }
  else if (b.mn) { GN_TRY(make_map_mn(&mbh, b.hi, brows, K, b.ld)); GN_TRY(make_map_mn(&mbl, b.lo, brows, K, b.ld)); }
  else { GN_TRY(make_map(&mbh, b.hi, brows, K, b.ld, BN)); GN_TRY(make_map(&mbl, b.lo, brows, K, b.ld, BN)); }
  TcEpilogue ep = ep_in;
  ep.a_mn = a3 ? 2 : (a.mn ? 1 : 0); ep.b_mn = b3 ? 2 : (b.mn ? 1 : 0);
  if (splits > 1) {
    size_t need = (size_t)splits * M * N;
    if (need > gs.splitk_floats) {
      if (gs.splitk_ws) cudaFree(gs.splitk_ws);
      gs.splitk_ws = nullptr; gs.splitk_floats = 0;
      if (cudaMalloc((void**)&gs.splitk_ws, need * sizeof(float)) != cudaSuccess) { set_error("tcgen05 gemm: cannot allocate the split-K workspace"); return GN_ERR_NOMEM; }
      gs.splitk_floats = need;
    }
    ep.C = gs.splitk_ws; ep.ldc = N; ep.aux = nullptr; ep.epi = EPI_STORE; ep.split_stride = (int64_t)M * N; ep.c_hi = ep.c_lo = nullptr;
  }
  dim3 grid(ceil_div(N, BN), ceil_div(M, TBM) + ep_in.groups, splits);   // grouped: an upper bound on the sum of per-group tiles
  // More tiles than SMs and a short K loop: one CTA per SM walks the tiles, so that a tile's store (a fifth of a
  // one-tile CTA's life at K = 768: an SM stores about 16 bytes per clock, 128 KB take 8-11 thousand cycles)
  // overlaps the next tile's K loop.  With long K loops the store is negligible and one-tile CTAs, which the hardware
  // hands out as SMs free up, balance better than a fixed round-robin (measured on the 16384-deep weight gradient).
  // Epilogues that read (accumulate, residual, relu^2 backward) gain nothing from the form but lose nothing either
  // once their reads are issued four rows at a time.
  const int64_t tiles_total = (int64_t)ceil_div(N, BN) * ceil_div(M, TBM);
  const int pctas = persistent_ctas(gs);
  if (pctas > 0 && splits == 1 && ep_in.groups == 0 && tiles_total > pctas && tiles_total < (int64_t)1 << 30 &&
      K <= 4096) {
    ep.tiles_total = (int)tiles_total; ep.tiles_n = ceil_div(N, BN);
    const int tiles_m = ceil_div(M, TBM);
    // few row tiles (the rollout's lm_head): all of them next to each other; otherwise bands of 16 column tiles
    ep.tiles_gn = tiles_m < 10 ? std::max(1, pctas / tiles_m) : 16;   // measured: lm_head at 512 rows 0.217 -> 0.193 ms, 16384 x 32768 x 768 4.10 -> 3.42 ms
    if (ep.tiles_gn > ep.tiles_n) ep.tiles_gn = ep.tiles_n;
    grid = dim3(pctas, 1, 1);
  }
  // One-tile CTAs whose epilogue reads nothing (plain, relu^2 without the saved pre-activation, softcap; K-split partial
  // planes) write through tensor maps of C and of the result's tf32 split.
  CUtensorMap mc = mah, mch = mah, mcl = mah;
  const bool tma_epi = ep.epi == EPI_STORE || (ep.epi == EPI_RELU2 && ep.aux == nullptr) || ep.epi == EPI_SOFTCAP;
  if (gs.tma_store && ep.tiles_total == 0 && ep.groups == 0 && tma_epi && ep.aux == nullptr && ep.ldc % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(ep.C) & 15) == 0 && (splits == 1 || ((int64_t)M * N) % 4 == 0) &&
      (ep.c_hi == nullptr || (((reinterpret_cast<uintptr_t>(ep.c_hi) | reinterpret_cast<uintptr_t>(ep.c_lo)) & 15) == 0))) {
    cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)splits};
    cuuint64_t strides[2] = {(cuuint64_t)ep.ldc * sizeof(float), (cuuint64_t)(splits > 1 ? ep.split_stride : (int64_t)M * ep.ldc) * sizeof(float)};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    auto enc = [&](CUtensorMap* mp, float* ptr) {
      const MapKey key{ptr, ((int64_t)M << 32) | (int64_t)(uint32_t)N, (int64_t)strides[0], (int64_t)strides[1], splits, 0, 4};
      return cached_map(mp, key, [&]() -> int {
        return g_encode(mp, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? GN_OK : GN_ERR_CUDA;
      }) == GN_OK;
    };
    bool ok = enc(&mc, ep.C);
    if (ok && ep.c_hi) ok = enc(&mch, ep.c_hi) && enc(&mcl, ep.c_lo);
    if (ok) ep.tma_store = 1;
  }
  {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(64 + 32 * (BN > 128 ? 8 : 4)); cfg.dynamicSmemBytes = ep.tiles_total > 0 ? S::TOTAL : S::TOTAL - S::STG_BYTES; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = gs.pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (ep.tiles_total > 0) GN_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES, true>, mah, mal, mbh, mbl, mc, mch, mcl, ep, M, N, K, gs.err_flag));
    else GN_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES, false>, mah, mal, mbh, mbl, mc, mch, mcl, ep, M, N, K, gs.err_flag));
  }
  GN_LAUNCH_CHECK();
  if (leave) {
    if (splits > 1) *leave = Partials{gs.splitk_ws, splits, (int64_t)M * N, (int64_t)N};
    else *leave = Partials{ep_in.C, 1, 0, ep_in.ldc};
  } else if (splits > 1) {
    int blocks = (int)std::min<int64_t>(((int64_t)M * (N / 4) + 255) / 256, (int64_t)num_sms() * 8);
    GN_CUDA(launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, (const float*)gs.splitk_ws, splits, (int64_t)M * N, ep_in, M, N));
    GN_LAUNCH_CHECK();
  }
  return GN_OK;
}


// Rows up to which x W^T products take the few-row form (0 = never).  Process-wide policy, like the tile shapes.
std::atomic<int> g_skinny_max_rows{256};
// Smallest number of k-blocks a K split of the few-row form may get.
std::atomic<int> g_skinny_min_kblocks{2};
// Activation rows one CTA of the few-row form takes (more rows: row blocks side by side on the same weight tile).
std::atomic<int> g_skinny_block_rows{128};

bool skinny_applies(const GemmArgs& g) {
  const int max_rows = g_skinny_max_rows.load(std::memory_order_relaxed);
  if (max_rows <= 0 || g.M < 1 || g.M > max_rows || g.groups > 0 || g.a_trans || !g.b_trans) return false;
  if (g.N < 64 || g.K < 32 || g.K % 4 != 0 || g.ldb % 4 != 0 || g.lda % 4 != 0) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return al(g.A) && al(g.B);
}

int launch_skinny(GemmState& gs, const SplitBuf& a, const GemmArgs& g, const TcEpilogue& ep_in, cudaStream_t s) {
  const int M = g.M, N = g.N, K = g.K;
  SkinnyArgs p{};
  p.M = M; p.N = N; p.K = K;
  p.block_rows = std::max(16, std::min(256, g_skinny_block_rows.load(std::memory_order_relaxed) / 16 * 16));
  p.rowsN = (std::min(M, p.block_rows) + 15) / 16 * 16;
  p.tmem_cols = 32; while (p.tmem_cols < p.rowsN) p.tmem_cols *= 2;
  p.prefetch = g.b_prefetch ? 1 : 0;
  const int stage_bytes = 2 * SK_W_BYTES + 2 * p.rowsN * TBK * 4;
  const int slabs = ceil_div(N, TBM), rblocks = ceil_div(M, p.block_rows), nk_total = ceil_div(K, TBK);
  // K splits: about one CTA per SM, every split at least min_kblocks k-blocks and at most 24 (768 elements of K are
  // accumulated in tensor memory in one go; longer sums are cut so that the accumulator's truncating adds stay
  // below 5e-6 of the result, as measured for the one-level K loop)
  const bool can_split = g.leave != nullptr || (N % 4 == 0 && g.ldc % 4 == 0);
  const int min_kb = std::max(1, g_skinny_min_kblocks.load(std::memory_order_relaxed));
  int splits = 1;
  if (can_split) splits = std::max(1, std::min(num_sms() / std::max(1, slabs * rblocks), nk_total / min_kb));
  int nkps = ceil_div(nk_total, splits);
  if (nkps > 24 && can_split) nkps = 24;
  splits = ceil_div(nk_total, nkps);
  p.nk_per_split = nkps;
  const int64_t ctas = (int64_t)slabs * rblocks * splits;
  // stages: as many as fit (more weight bytes in flight per SM); when there are more CTAs than SMs, two CTAs per SM
  const int bar_bytes = (3 * SK_MAX_STAGES + 2) * 8 + 1024;
  const int smem_one = 227 * 1024 - bar_bytes, smem_two = (227 * 1024) / 2 - 1024 - bar_bytes;
  int stages = std::min(SK_MAX_STAGES, smem_one / stage_bytes);
  if (ctas > num_sms() && smem_two / stage_bytes >= 2) stages = std::min(SK_MAX_STAGES, smem_two / stage_bytes);
  stages = std::max(1, std::min(stages, std::max(nkps, 1)));
  GN_REQUIRE(stages >= 1 && stage_bytes * stages + bar_bytes <= 227 * 1024, "few-row product: a stage of %d bytes does not fit shared memory", stage_bytes);
  p.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + bar_bytes;
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); }
  CUtensorMap mw, mxh, mxl;
  GN_TRY(make_map(&mw, g.B, N, K, g.ldb, TBM));
  GN_TRY(make_map(&mxh, a.hi, M, K, a.ld, p.rowsN));
  GN_TRY(make_map(&mxl, a.lo, M, K, a.ld, p.rowsN));
  p.ep = ep_in;
  if (splits > 1) {
    const size_t need = (size_t)splits * M * N;
    if (need > gs.splitk_floats) {
      if (gs.splitk_ws) cudaFree(gs.splitk_ws);
      gs.splitk_ws = nullptr; gs.splitk_floats = 0;
      if (cudaMalloc((void**)&gs.splitk_ws, need * sizeof(float)) != cudaSuccess) { set_error("tcgen05 gemm: cannot allocate the split-K workspace"); return GN_ERR_NOMEM; }
      gs.splitk_floats = need;
    }
    p.ep.C = gs.splitk_ws; p.ep.ldc = N; p.ep.aux = nullptr; p.ep.epi = EPI_STORE; p.ep.split_stride = (int64_t)M * N; p.ep.c_hi = p.ep.c_lo = nullptr;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(rblocks, slabs, splits); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = gs.pdl ? 1 : 0;
  cfg.attrs = attr; cfg.numAttrs = 1;
  GN_CUDA(cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, mw, mxh, mxl, p, gs.err_flag));
  GN_LAUNCH_CHECK();
  if (g.leave) {
    if (splits > 1) *g.leave = Partials{gs.splitk_ws, splits, (int64_t)M * N, (int64_t)N};
    else *g.leave = Partials{ep_in.C, 1, 0, ep_in.ldc};
  } else if (splits > 1) {
    int blocks = (int)std::min<int64_t>(((int64_t)M * (N / 4) + 255) / 256, (int64_t)num_sms() * 8);
    GN_CUDA(launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, (const float*)gs.splitk_ws, splits, (int64_t)M * N, ep_in, M, N));
    GN_LAUNCH_CHECK();
  }
  return GN_OK;
}

}  // namespace

int gemm_tcgen05_supported(const GemmArgs& g) {
  if (skinny_applies(g)) return 1;                      // x W^T with few rows: the weight-streaming form
  if (g.M < 64 || g.N < 64 || g.K < 32) return 0;      // tiny products stay on the SIMT kernel
  if (g.groups > 0 && (!g.b_trans || g.a_trans || g.epilogue != EPI_STORE || g.N % 4 != 0)) return 0;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(g.A) || !al(g.B)) return 0;
  // Sources read with float4 need a contiguous extent that is a multiple of 4; the
  // transposing split reads scalars and pads.
  if (!g.a_trans && (g.K % 4 != 0 || g.lda % 4 != 0)) return 0;
  if (g.b_trans && (g.K % 4 != 0 || g.ldb % 4 != 0)) return 0;
  return 1;
}

int gemm_tcgen05(const GemmArgs& g, cudaStream_t s) {
  std::lock_guard<std::mutex> lock(g_mu);
  GN_TRY(ensure_init());
  GemmState* gsp = nullptr;
  GN_TRY(state_for(s, &gsp));
  GemmState& gs = *gsp;
  SplitBuf a, b;
  // A is logically [M, K]; stored transposed ([K, M]) when a_trans.
  // the source of A as stored: [src_rows, src_cols]
  const int64_t src_rows = g.a_trans ? g.K : g.M, src_cols = g.a_trans ? g.M : g.K;
  if (g.a_hi && g.a_lo && !g.a_trans) { a.hi = const_cast<float*>(g.a_hi); a.lo = const_cast<float*>(g.a_lo); a.ld = g.lda; }   // split by the producer
  else if (g.a_reuse && gs.last_a.valid && gs.last_a.src == g.A && gs.last_a.ld == g.lda && gs.last_a.rows == src_rows && gs.last_a.cols == src_cols &&
           (!g.a_trans || gs.mn)) {
    a = gs.dyn[0]; a.ld = src_cols; a.mn = g.a_trans != 0;   // the plain split of the previous product, read K-major or MN-major
  } else {
    GN_TRY(split_operand(gs, g.A, g.lda, g.M, g.K, g.a_trans != 0, g.a_static != 0, 0, a, s, gs.mn));
    // a plain (untransposed) split with an unpadded pitch can serve the next product too
    const bool plain = !g.a_static && src_cols % 4 == 0 && (g.a_trans ? a.mn : true);
    gs.last_a.valid = plain; gs.last_a.src = g.A; gs.last_a.ld = g.lda; gs.last_a.rows = src_rows; gs.last_a.cols = src_cols;
  }
  if (skinny_applies(g)) {
    // few rows against a weight matrix: the weights are streamed raw and split on chip
    TcEpilogue ep{g.C, g.ldc, g.aux, g.ldaux, g.epilogue, g.scalar, 0, g.c_hi, g.c_lo, g_trace, nullptr, 0, 0, 0, 0, 0, 1};
    return launch_skinny(gs, a, g, ep, s);
  }
  // B is logically [N, K]; stored that way when b_trans (weights [out, in]), else stored [K, N].
  if (g.b_hi && g.b_lo && !g.b_trans && gs.mn && g.groups == 0 && g.ldb % 4 == 0) {
    b.hi = const_cast<float*>(g.b_hi); b.lo = const_cast<float*>(g.b_lo); b.ld = g.ldb; b.mn = true;   // split by the producer
  } else {
    GN_TRY(split_operand(gs, g.B, g.ldb, g.groups > 0 ? (int64_t)g.groups * g.N : g.N, g.K, g.b_trans == 0, g.b_static != 0, 1, b, s, gs.mn));
  }
  TcEpilogue ep{g.C, g.ldc, g.aux, g.ldaux, g.epilogue, g.scalar, 0, g.c_hi, g.c_lo, g_trace, g.group_counts, g.groups, 0, 0, 0, 0, 1};
  if (g.groups > 0) return launch_tc<128, 3>(gs, a, b, ep, g.M, g.N, g.K, 1, s, nullptr);
  // Filling the machine when the output has few tiles (the rollout's products have 512 rows):
  // the K loop is split over gridDim.z so that about one CTA per SM runs, each writing a partial
  // tile that a second pass sums in a fixed order (deterministic, unlike atomics).  Narrow tiles
  // would also add CTAs but re-read the activation operand once per column tile, and the kernel
  // is bound by the 64 B/clk/SM path from L2.
  const int64_t tiles = (int64_t)ceil_div(g.M, TBM) * ceil_div(g.N, 128);
  const int nk = ceil_div(g.K, TBK);
  const int sms = num_sms();
  // Wide 128 x 256 tiles when the output is large: the K loop is bound by the 64 B/clk/SM path from
  // L2, and a 256-column tile reads the A operand once for twice the work (96 KB per k-block for
  // two 128 x 128 units instead of 128 KB).
  if (g.N >= 512 && (int64_t)ceil_div(g.M, TBM) * ceil_div(g.N, 256) >= sms * 3 / 2)
    return launch_tc<256, 2>(gs, a, b, ep, g.M, g.N, g.K, 1, s, g.leave);
  // Up to about a wave of tiles: the tile width and the K split with the smallest estimated time.  A k-block costs a
  // CTA ~1080 cycles with 128-wide tiles and ~1600 with 256-wide ones (both bound by the L2 -> SM path: 64 and 96 KB),
  // a CTA ~12 000 cycles of set-up and store, a K split a reduction pass over its planes.
  const bool can_split = g.N % 4 == 0 && g.ldc % 4 == 0;
  auto estimate = [&](int bn, int sp) {
    const int64_t t = (int64_t)ceil_div(g.M, TBM) * ceil_div(g.N, bn);
    const double waves = (double)ceil_div(t * sp, sms);
    double c = waves * (ceil_div(nk, sp) * (bn == 256 ? 1600.0 : 1080.0) + 12000.0);
    if (sp > 1) c += 6000.0 + (double)g.M * g.N * 4.0 * (sp + 1) / 1600.0;
    return c;
  };
  // 128-wide tiles: the K loop split over gridDim.z until about one CTA per SM runs (at least 4 k-blocks per split)
  int best_bn = 128, best_sp = 1;
  if (tiles < sms / 2 && can_split) best_sp = (int)std::max<int64_t>(1, std::min<int64_t>(sms / tiles, nk / 4));
  double best = estimate(128, best_sp);
  auto consider = [&](int bn, int sp) {
    if (sp < 1 || (sp > 1 && !can_split)) return;
    const double c = estimate(bn, sp);
    if (c < best) { best = c; best_bn = bn; best_sp = sp; }
  };
  if (gs.wide_split && g.N % 256 == 0 && nk >= 8) {
    const int64_t wide = (int64_t)ceil_div(g.M, TBM) * (g.N / 256);
    consider(256, 1);
    if (wide < sms) consider(256, (int)std::min<int64_t>(sms / wide, nk / 4));
  }
  if (best_bn == 256) return launch_tc<256, 2>(gs, a, b, ep, g.M, g.N, g.K, best_sp, s, g.leave);
  const int splits = best_sp;
  return launch_tc<128, 3>(gs, a, b, ep, g.M, g.N, g.K, splits, s, g.leave);
}

// The parameters changed in place (an optimizer step, an upload): cached splits on this device keep their buffers and
// are redone on next use.
void gemm_tcgen05_mark_stale() {
  std::lock_guard<std::mutex> lock(g_mu);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return;
  for (auto& st : g_states)
    if (st.first.first == device)
      for (auto& kv : st.second->statics) kv.second.fresh = false;
}
// Parameter storage on this device is going away: free the cached splits that are keyed by its addresses.
void gemm_tcgen05_invalidate() {
  std::lock_guard<std::mutex> lock(g_mu);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return;
  cudaDeviceSynchronize();
  for (auto& st : g_states) {
    if (st.first.first != device) continue;
    for (auto& kv : st.second->statics) { cudaFree(kv.second.hi); cudaFree(kv.second.lo); }
    st.second->statics.clear();
  }
}
// The stream is going away (its context is destroyed): free everything held for it.
void gemm_tcgen05_release(cudaStream_t s) {
  std::lock_guard<std::mutex> lock(g_mu);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return;
  auto it = g_states.find(std::make_pair(device, s));
  if (it == g_states.end()) return;
  cudaStreamSynchronize(s);
  GemmState* st = it->second;
  for (auto& kv : st->statics) { cudaFree(kv.second.hi); cudaFree(kv.second.lo); }
  for (SplitBuf& b : st->dyn) { if (b.hi) { cudaFree(b.hi); cudaFree(b.lo); } }
  if (st->attn.hi) { cudaFree(st->attn.hi); cudaFree(st->attn.lo); }
  if (st->splitk_ws) cudaFree(st->splitk_ws);
  if (st->err_flag) cudaFree(st->err_flag);
  delete st;
  g_states.erase(it);
}
// Options of the products issued on stream s.  Unknown names return GN_ERR_INVALID.
int gemm_tcgen05_option(cudaStream_t s, const char* name, int value) {
  std::lock_guard<std::mutex> lock(g_mu);
  GemmState* st = nullptr;
  GN_TRY(state_for(s, &st));
  const std::string n = name;
  if (n == "gemm_persistent_ctas") st->persistent_ctas = value;
  else if (n == "gemm_pdl") st->pdl = value != 0;
  else if (n == "gemm_mn_major") st->mn = value != 0;
  else if (n == "gemm_mn_3d") st->mn3d = value != 0;
  else if (n == "gemm_tma_store") st->tma_store = value != 0;
  else if (n == "gemm_wide_split") st->wide_split = value != 0;
  else if (n == "gemm_few_rows_max") g_skinny_max_rows.store(value, std::memory_order_relaxed);
  else if (n == "gemm_few_rows_min_kblocks") g_skinny_min_kblocks.store(value, std::memory_order_relaxed);
  else if (n == "gemm_few_rows_block") g_skinny_block_rows.store(value, std::memory_order_relaxed);
  else { set_error("unknown option '%s'", name); return GN_ERR_INVALID; }
  return GN_OK;
}

#ifdef GN_TC_TRACE
// Development aid: the next products record CTA (0,0)'s timeline; returns it (1024 slots).
extern "C" int gn_debug_gemm_trace(long long* host_out, int arm) {
  if (arm) {
    if (!g_trace) GN_CUDA(cudaMalloc((void**)&g_trace, 1024 * sizeof(long long)));
    GN_CUDA(cudaMemset(g_trace, 0, 1024 * sizeof(long long)));
    return GN_OK;
  }
  GN_CUDA(cudaDeviceSynchronize());
  if (g_trace && host_out) GN_CUDA(cudaMemcpy(host_out, g_trace, 1024 * sizeof(long long), cudaMemcpyDeviceToHost));
  return GN_OK;
}
#endif

int tc_make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int box_rows) {
  GN_TRY(ensure_init());
  return make_map(map, base, rows, k, ld, box_rows);
}
int tc_make_map_mn(CUtensorMap* map, const float* base, int64_t mn, int64_t k, int64_t ld) {
  GN_TRY(ensure_init());
  return make_map_mn(map, base, mn, k, ld);
}
int tc_make_map_mn3(CUtensorMap* map, const float* base, int64_t mn, int64_t k, int64_t ld, int groups) {
  GN_TRY(ensure_init());
  return make_map_mn3(map, base, mn, k, ld, groups);
}
int tc_make_map3(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int box_rows, int kblocks) {
  GN_TRY(ensure_init());
  return cached_map(map, MapKey{base, rows, k, ld, box_rows, kblocks, 3}, [&]() -> int {
  cuuint64_t dims[3] = {32, (cuuint64_t)rows, (cuuint64_t)(k / 32)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * sizeof(float), 32 * sizeof(float)};
  cuuint32_t box[3] = {32, (cuuint32_t)box_rows, (cuuint32_t)kblocks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (K-major, 3-D) failed with %d (rows %lld, k %lld, ld %lld)", (int)r, (long long)rows, (long long)k, (long long)ld); return GN_ERR_CUDA; }
  return GN_OK;
  });
}
int tc_attention_scratch(cudaStream_t s, size_t floats, float** hi, float** lo, int** err_flag) {
  std::lock_guard<std::mutex> lock(g_mu);
  GemmState* st = nullptr;
  GN_TRY(state_for(s, &st));
  GN_TRY(ensure_buf(st->attn, floats));
  *hi = st->attn.hi; *lo = st->attn.lo; *err_flag = st->err_flag;
  return GN_OK;
}

int gemm_tc_batched(const TcBatched& g, cudaStream_t s) {
  std::lock_guard<std::mutex> lock(g_mu);
  GemmState* st = nullptr;
  GN_TRY(state_for(s, &st));
  GN_TRY(ensure_init());
  using S = TcSmem<128, 3>;
  static PerDeviceOnce configured;
  if (configured.first()) { GN_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<128, 3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL - S::STG_BYTES)); }
  GN_REQUIRE(g.batches >= 1 && g.batches <= 65535 && g.batch != nullptr, "batched product: %d batches", g.batches);
  CUtensorMap mah, mal, mbh, mbl;
  // MN-major operands whose MN extent is a multiple of 32 come as one 3-D box per tile (the batch offsets in MN must then be multiples of 32)
  const bool a3 = g.a.mn && g.a.cols % 32 == 0, b3 = g.b.mn && g.b.cols % 32 == 0;
  if (a3) { GN_TRY(make_map_mn3(&mah, g.a.hi, g.a.cols, g.a.rows, g.a.ld, TBM / 32)); GN_TRY(make_map_mn3(&mal, g.a.lo, g.a.cols, g.a.rows, g.a.ld, TBM / 32)); }
  else if (g.a.mn) { GN_TRY(make_map_mn(&mah, g.a.hi, g.a.cols, g.a.rows, g.a.ld)); GN_TRY(make_map_mn(&mal, g.a.lo, g.a.cols, g.a.rows, g.a.ld)); }
  else { GN_TRY(make_map(&mah, g.a.hi, g.a.rows, g.a.cols, g.a.ld, TBM)); GN_TRY(make_map(&mal, g.a.lo, g.a.rows, g.a.cols, g.a.ld, TBM)); }
  if (b3) { GN_TRY(make_map_mn3(&mbh, g.b.hi, g.b.cols, g.b.rows, g.b.ld, 128 / 32)); GN_TRY(make_map_mn3(&mbl, g.b.lo, g.b.cols, g.b.rows, g.b.ld, 128 / 32)); }
  else if (g.b.mn) { GN_TRY(make_map_mn(&mbh, g.b.hi, g.b.cols, g.b.rows, g.b.ld)); GN_TRY(make_map_mn(&mbl, g.b.lo, g.b.cols, g.b.rows, g.b.ld)); }
  else { GN_TRY(make_map(&mbh, g.b.hi, g.b.rows, g.b.cols, g.b.ld, 128)); GN_TRY(make_map(&mbl, g.b.lo, g.b.rows, g.b.cols, g.b.ld, 128)); }
  TcEpilogue ep{};
  ep.C = g.C; ep.ldc = g.ldc; ep.epi = g.accumulate ? EPI_ACCUM : EPI_STORE; ep.scalar = 1.0f;
  ep.a_mn = a3 ? 2 : (g.a.mn ? 1 : 0); ep.b_mn = b3 ? 2 : (g.b.mn ? 1 : 0);
  ep.batch = g.batch; ep.k_segments = g.k_segments; ep.k_seg_stride = g.k_seg_stride; ep.k_causal = g.k_causal;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(ceil_div(g.N, 128), ceil_div(g.M, TBM), g.batches); cfg.blockDim = dim3(64 + 32 * 4); cfg.dynamicSmemBytes = S::TOTAL - S::STG_BYTES; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 0;
  cfg.attrs = attr; cfg.numAttrs = 1;
  GN_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<128, 3, false>, mah, mal, mbh, mbl, mah, mah, mah, ep, g.M, g.N, g.K, st->err_flag));
  GN_LAUNCH_CHECK();
  return GN_OK;
}

// Reads and clears the device-side timeout flag of the stream's products.
int gemm_tcgen05_check(cudaStream_t s) {
  int* flag_dev = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    int device = 0;
    GN_CUDA(cudaGetDevice(&device));
    auto it = g_states.find(std::make_pair(device, s));
    if (it == g_states.end()) return GN_OK;
    flag_dev = it->second->err_flag;
  }
  int flag = 0;
  GN_CUDA(cudaMemcpyAsync(&flag, flag_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  if (flag) {
    cudaMemsetAsync(flag_dev, 0, sizeof(int), s);
    set_error("tcgen05 gemm: a bounded mbarrier wait ran out (pipeline stalled)");
    return GN_ERR_TIMEOUT;
  }
  return GN_OK;
}

}  // namespace gn
