// Shared declarations for the gonano CUDA backend (sm_100a).
#pragma once
#include <atomic>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/gonano_cuda.h"

namespace gn {

// Thread-local message behind gn_last_error().
void set_error(const char* fmt, ...);
const char* get_error();

#define GN_CUDA(expr)                                                                      \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      gn::set_error("%s:%d: %s -> %s", __FILE__, __LINE__, #expr, cudaGetErrorString(e__)); \
      return GN_ERR_CUDA;                                                                  \
    }                                                                                      \
  } while (0)

#define GN_TRY(expr)                 \
  do {                               \
    int s__ = (expr);                \
    if (s__ != GN_OK) return s__;    \
  } while (0)

#define GN_REQUIRE(cond, ...)        \
  do {                               \
    if (!(cond)) {                   \
      gn::set_error(__VA_ARGS__);    \
      return GN_ERR_INVALID;         \
    }                                \
  } while (0)

// Check the launch that just happened and count it (gn_ctx_launch_count).
void count_launch();
void count_launches(int64_t n);   // kernels replayed through a CUDA graph
#define GN_LAUNCH_CHECK()          \
  do {                             \
    gn::count_launch();            \
    GN_CUDA(cudaGetLastError());   \
  } while (0)

// Streaming multiprocessors of the current device (148 on B200), queried once per device.
int num_sms();

// Function attributes (cudaFuncSetAttribute) are per device: first() is true the first time a call site runs on the
// current device, from whichever thread.
struct PerDeviceOnce {
  std::atomic<unsigned long long> done{0};
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    const unsigned long long bit = 1ull << dev;
    return (done.fetch_or(bit) & bit) == 0;
  }
};

static inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// ------------------------------------------------------------ device helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `scratch` holds at least 32 floats; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.0f;
  if (warp == 0) { t = warp_sum(t); if (lane == 0) scratch[0] = t; }
  __syncthreads();
  return scratch[0];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) { t = warp_max(t); if (lane == 0) scratch[0] = t; }
  __syncthreads();
  return scratch[0];
}
__device__ __forceinline__ double block_sum_d(double v, double* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum_d(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double t = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.0;
  if (warp == 0) { t = warp_sum_d(t); if (lane == 0) scratch[0] = t; }
  __syncthreads();
  return scratch[0];
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }
// Sigmoid evaluated in double like the reference's scalar backend
// (kernels/scalar/elementwise.go:146-150); used where a gate decides values.
__device__ __forceinline__ float sigmoid_exact(float x) { return (float)(1.0 / (1.0 + exp((double)(-x)))); }

// Programmatic dependent launch.  A kernel that feeds a product calls pdl_trigger() first thing: the product's grid
// may then be scheduled while this one still runs, and sets up (barriers, tensor memory, descriptors) in its shadow.
// The product calls pdl_wait() before it touches global memory: it returns once the triggering grid has completed
// and its writes are visible.  Both are no-ops when the next / this launch does not carry the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with programmatic stream serialization: the grid may be scheduled while the kernel in front of it on the stream
// still runs.  ONLY for kernels that call pdl_wait() before their first access to global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// hi = tf32(x) (round to nearest), lo = tf32(x - hi): the operand form of the 3xTF32 products.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  uint32_t h, l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  float rest = x - hi;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
  lo = __uint_as_float(l);
}

// ---------------------------------------------------------------- GEMM API
// C[M,N] (op)= A(M,K) * B(K,N), row-major storage with leading dimensions.
//   a_trans = 0: A(m,k) = A[m*lda + k]      a_trans = 1: A(m,k) = A[k*lda + m]
//   b_trans = 0: B(k,n) = B[k*ldb + n]      b_trans = 1: B(k,n) = B[n*ldb + k]   (weights stored [out,in])
enum GemmEpilogue {
  EPI_STORE = 0,     // C = acc
  EPI_ACCUM = 1,     // C += acc
  EPI_RESIDUAL = 2,  // C = R + acc        (R = aux, ld = ldaux; R may alias C)
  EPI_RELU2 = 3,     // aux = acc (optional), C = max(acc,0)^2
  EPI_SOFTCAP = 4,   // C = cap * tanh(acc / cap)   (cap = scalar)
  EPI_RELU2_BWD = 5, // C = acc * 2*max(aux,0)      (aux = saved pre-activation)
};
// A product left unreduced by gemm_dispatch: value(m, n) = sum over z < splits of ptr[z*stride + m*ld + n],
// added in the order z = 0, 1, ... (the same order the stand-alone reduction uses).
struct Partials {
  const float* ptr = nullptr; int splits = 0; int64_t stride = 0; int64_t ld = 0;
  __host__ __device__ bool on() const { return ptr != nullptr; }
#ifdef __CUDACC__
  __device__ __forceinline__ float at(int64_t m, int64_t n) const {
    const float* q = ptr + m * ld + n;
    float a = q[0];
    for (int z = 1; z < splits; ++z) a += q[(int64_t)z * stride];
    return a;
  }
  // Four consecutive columns (n, ld and stride multiples of 4, ptr 16-byte aligned).  The loads of
  // eight splits are issued together; the additions keep the order z = 0, 1, ...
  __device__ __forceinline__ float4 at4(int64_t m, int64_t n) const {
    const float* q = ptr + m * ld + n;
    float4 a = *reinterpret_cast<const float4*>(q);
    for (int z0 = 1; z0 < splits; z0 += 8) {
      float4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (z0 + j < splits) v[j] = *reinterpret_cast<const float4*>(q + (int64_t)(z0 + j) * stride);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (z0 + j < splits) { a.x += v[j].x; a.y += v[j].y; a.z += v[j].z; a.w += v[j].w; }
    }
    return a;
  }
#endif
};

struct GemmArgs {
  const float* A = nullptr; const float* B = nullptr; float* C = nullptr;
  int M = 0, N = 0, K = 0;
  int64_t lda = 0, ldb = 0, ldc = 0;
  int a_trans = 0, b_trans = 0;
  int epilogue = EPI_STORE;
  float* aux = nullptr; int64_t ldaux = 0;
  float scalar = 0.0f;
  int a_static = 0, b_static = 0;  // operand is a parameter tensor: its tensor-core split may be cached
  // Tensor-core path only: B holds parameters that no kernel in flight writes, so a product may request them before the
  // kernel in front of it on the stream has finished (programmatic dependent launch).
  int b_prefetch = 0;
  // Tensor-core path only: A already split by its producer (hi = tf32(x), lo = tf32(x - hi)), pitch lda.
  const float* a_hi = nullptr; const float* a_lo = nullptr;
  // Tensor-core path only: A (same pointer, pitch and shape, possibly through the other a_trans) is unchanged since the
  // previous product issued on this stream, so its split may be reused (dY feeds the weight gradient, then the data gradient).
  int a_reuse = 0;
  // Tensor-core path only: B stored [K, N] (b_trans = 0) already split by its producer, pitch ldb (read MN-major).
  const float* b_hi = nullptr; const float* b_lo = nullptr;
  // Tensor-core path only: also write the split of the output (pitch ldc) for the next product.
  float* c_hi = nullptr; float* c_lo = nullptr;
  // When set (epilogue must be EPI_STORE): the product may be left as split-K partial tiles for the
  // consumer kernel to sum; *leave says where they are (splits == 1 and ptr == C when it was not split).
  // The partial tiles live in a workspace that the next product on the stream reuses.
  Partials* leave = nullptr;
  // Grouped product over expert-major rows (kernels/backend.go:130-141): groups > 0 makes A [M, K] a stack of
  // per-group row blocks with group_counts[g] rows each (device array, sum == M), B [groups * N, K] the packed
  // per-group weights (b_trans = 1) and C [M, N] the stacked outputs.  EPI_STORE only.
  const int32_t* group_counts = nullptr; int groups = 0;
};
int gemm_simt(const GemmArgs& args, cudaStream_t stream);
// kind 0: SIMT float32.  kind 1: tcgen05 3xTF32 where the shape allows it, else SIMT.
int gemm_dispatch(const GemmArgs& args, int kind, cudaStream_t stream);
// Grouped product: tensor cores when kind == 1 and the shape allows it, else the float32 warp-per-row kernel.
int gemm_grouped_dispatch(const GemmArgs& args, int kind, cudaStream_t stream);
int gemm_default_kind();
int64_t launch_count();
// tcgen05 path housekeeping (no-ops when the library was built without it).
void gemm_invalidate_static();        // parameter storage is going away: free cached operand splits
void gemm_mark_static_stale();        // parameters changed in place: cached splits are redone (in their buffers) on next use
int gemm_check_error(cudaStream_t s); // GN_ERR_TIMEOUT when a bounded device wait ran out
void gemm_release_stream(cudaStream_t s);   // the stream is going away: free the scratch held for its products
int gemm_set_option(cudaStream_t s, const char* name, int value);
cudaStream_t tier_a_stream_or_null();       // the stream Tier A runs on (null before its first call)

}  // namespace gn
