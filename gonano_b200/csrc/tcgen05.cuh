// PTX wrappers for the 5th-generation tensor cores (tcgen05), tensor memory, bulk tensor copies (TMA) and
// mbarriers, shared by the kernels that run on them.  sm_100a only.  Every function has internal linkage.
#pragma once
#include <cuda.h>
#include <cstdint>

namespace gn {

namespace {

constexpr int TBM = 128;       // tile rows = UMMA M
constexpr int TBK = 32;        // floats per k-block = one 128-byte swizzle row
constexpr int UMMA_K = 8;      // tf32 MMA depth
constexpr uint32_t kSpinLimit = 1u << 22;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out (the flag is raised by the caller).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_test(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// Shared memory -> global memory through a tensor map (rows and columns outside the tensor are not written).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit_wait() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z), "r"(z), "r"(z), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row
// groups 1024 bytes apart.  Bits: [0,14) address>>4, [16,30) leading offset>>4 (1 for
// swizzled K-major), [32,46) stride offset>>4, [46,48) version 1, [61,64) layout 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// The same for an operand stored with its M (or N) index contiguous ("MN-major": the operand of a product A^T B or
// A B whose source is row-major [K, MN]).  For 32-bit elements the tensor core wants the 128-byte swizzle with
// 32-byte atoms (layout type 1; the TMA mode of the same name): rows of 128 bytes = 32 consecutive MN elements,
// one row per k, a 128 (MN) x 32 (K) tile = four 2-D TMA boxes [32 MN x 32 K] of the row-major source, 4096 bytes
// apart.  Leading offset = distance between the MN groups (4096 bytes), stride offset 512 bytes (the 4-row swizzle
// period), and one instruction's K = 8 advances the start address by 8 rows = 1024 bytes.  This form was found by
// comparing a 128 x 128 x 64 product against float64 over a handful of candidates; only this one agreed (7e-7).
constexpr uint64_t kMnDesc = ((uint64_t)(4096 >> 4) << 16) | ((uint64_t)(512 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)1 << 61);
constexpr uint32_t kMnKStep = 1024 >> 4;
// Instruction descriptor for kind::tf32, float32 accumulate, both operands K-major:
// [4,6) D format 1 = F32, [7,10) A format 2 = TF32, [10,13) B format 2, [17,23) N>>3, [24,29) M>>4.
// Bits 15 / 16 select the MN-major form of A / B.
__device__ __forceinline__ uint32_t instr_desc_tf32(int m, int n, int a_mn = 0, int b_mn = 0) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The same instruction with the A operand in tensor memory (lane = row, one 32-bit column per element of K).
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z), "r"(z), "r"(z), "r"(z)
      : "memory");
}
// Registers to tensor memory: lane i of the warp writes 32 consecutive columns of its row.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// split_tf32 with integer arithmetic: adding half a tf32 unit to the magnitude bits and clearing the low 13 bits rounds to
// nearest with ties away from zero, which is what cvt.rna.tf32.f32 does, at the full rate of the integer pipe.
__device__ __forceinline__ void split_tf32_int(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
  const float rest = x - hi;
  lo = __uint_as_float((__float_as_uint(rest) + 0x1000u) & 0xFFFFE000u);
}

}  // namespace

// Batched product on the one-tile form of the tensor-core GEMM (gemm_tcgen05.cu):
//   C_z[M, N] (+)= A_z[M, K] * B_z[N, K]^T   for z in [0, batches)
// A and B are 2-D float32 arrays given as hi/lo tf32 splits; K-major (mn = 0): rows = the m (or n) index, cols = k;
// MN-major (mn = 1): rows = k, cols = the m (or n) index.  A batch is a window of the arrays: its offsets (device
// array, one TcBatch per batch) are added to the tile coordinates in the operand's (m or n, k) index space, c_off
// (floats) to C.  The contraction may walk k_segments segments k_seg_stride 32-element blocks apart, each cut to the
// causal range: k_causal 1 = k < m0 + 128, 2 = k >= m0 (m0 the tile's first row); 0 segments = the plain K loop.
struct TcBatch { int a_m, a_k, b_n, b_k; long long c_off; };
struct TcOperand { const float* hi; const float* lo; int64_t rows, cols, ld; int mn; };
struct TcBatched {
  TcOperand a, b;
  int M, N, K;
  float* C; int64_t ldc; int accumulate;
  const TcBatch* batch; int batches;
  int k_segments, k_seg_stride, k_causal;
};
int gemm_tc_batched(const TcBatched& g, cudaStream_t s);

// Host side (gemm_tcgen05.cu): tensor maps over float32 arrays and the per-(device, stream) scratch of the attention kernels.
// K-major: a box is [32 floats x box_rows rows] of a row-major [rows, k] array (pitch ld floats), 128-byte swizzle.
int tc_make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int box_rows);
// MN-major: a box is [32 mn x 32 k] of a row-major [k, mn] array (pitch ld floats), 128-byte swizzle with 32-byte atoms.
int tc_make_map_mn(CUtensorMap* map, const float* base, int64_t mn, int64_t k, int64_t ld);
// The same as one 3-D box [32 mn x 32 k x groups] (mn a multiple of 32): the groups land 4096 bytes apart, as the tensor core reads them.
int tc_make_map_mn3(CUtensorMap* map, const float* base, int64_t mn, int64_t k, int64_t ld, int groups);
// K-major as one 3-D box [32 floats x box_rows rows x kblocks k-blocks] (k a multiple of 32): the k-blocks land one after the other.
int tc_make_map3(CUtensorMap* map, const float* base, int64_t rows, int64_t k, int64_t ld, int box_rows, int kblocks);
// Scratch of at least `floats` floats in each of `hi` and `lo`, and the error flag that gemm_tcgen05_check reads.
int tc_attention_scratch(cudaStream_t s, size_t floats, float** hi, float** lo, int** err_flag);

}  // namespace gn
