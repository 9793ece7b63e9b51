// gn_pg_loss_backward_static: the fused policy-gradient loss for hosts that must not allocate.
//
// Some programs that embed this library own every byte of device memory themselves and hand
// out fixed budgets at start-up: a serving process whose own arena was sized to the whole
// GPU, or a control loop that cannot tolerate cudaMalloc because the call synchronises the
// whole device and may fail late, long after start-up checks have passed.  Such a caller
// cannot use gn_pg_loss_backward, which borrows a few bytes of device scratch per call for
// the per-row loss terms.  This variant keeps that scratch in a fixed array that is part of
// the library image, so the call performs no allocation of any kind: no cudaMalloc, no
// cudaFree, no staging buffers, no allocating library routine.
//
// The price of a fixed array:
//   * a hard limit of GN_STATIC_LOSS_MAX_ROWS rows per call; larger batches are refused;
//   * every GPU that loads the library holds the array (about 0.5 MB) until the process exits;
//   * all calls share it.  It still holds the previous call's values when the next one starts;
//     the cell that receives the total is cleared on every call and the per-row cells are all
//     rewritten before they are read, so stale values are never used.  Two calls that overlap on
//     the same GPU (different streams or threads) would write the same cells: do not do that.
//   * inputs and outputs must already be in device memory, since staging a host buffer would
//     need an allocation.
//
// The array's device address is looked up once per device, on the first call that runs with
// that device current; make that first call during start-up.  The call cannot run inside a stream
// capture: it synchronises the stream before it returns.  First calls on one device from several
// threads at once may each do the look-up; they store the same address, so the race is harmless.
#include <atomic>

#include "kernels.cuh"

namespace gn {
namespace {

// cell 0: the loss total; cell 1: count of out-of-range targets; cells 32..: one term per row (offset keeps the rows 256-byte aligned)
constexpr int64_t kStaticRowOffset = 32;
static __device__ __align__(256) double g_static_loss_scratch[GN_STATIC_LOSS_MAX_ROWS + kStaticRowOffset];

constexpr int kMaxDevices = 64;
std::atomic<double*> g_scratch_addr[kMaxDevices];

// The symbol name above is only a handle on the host side, not an address a kernel can use:
// the real per-device address comes from the runtime.
int static_scratch(double** out) {
  int device = 0;
  GN_CUDA(cudaGetDevice(&device));
  GN_REQUIRE(device >= 0 && device < kMaxDevices, "device ordinal %d outside [0,%d)", device, kMaxDevices);
  double* addr = g_scratch_addr[device].load(std::memory_order_acquire);
  if (!addr) {
    void* p = nullptr;
    GN_CUDA(cudaGetSymbolAddress(&p, g_static_loss_scratch));
    addr = static_cast<double*>(p);
    g_scratch_addr[device].store(addr, std::memory_order_release);
  }
  *out = addr;
  return GN_OK;
}

bool is_device_pointer(const void* p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

}  // namespace
}  // namespace gn

using namespace gn;

extern "C" int gn_pg_loss_backward_static(const float* logits, const int32_t* targets, const float* advantages, int64_t rows, int vocab,
                                          int seq_len, float norm, float softcap, float* nll, float* dlogits, double* loss, void* stream) {
  GN_REQUIRE(logits && targets && advantages && loss && vocab > 0 && seq_len > 0 && rows >= 0, "pg_loss_backward_static: bad argument");
  GN_REQUIRE(rows <= GN_STATIC_LOSS_MAX_ROWS, "pg_loss_backward_static: %lld rows exceed the fixed scratch of %d rows; split the batch or use gn_pg_loss_backward",
             (long long)rows, GN_STATIC_LOSS_MAX_ROWS);
  GN_REQUIRE(is_device_pointer(logits) && is_device_pointer(targets) && is_device_pointer(advantages) && (!nll || is_device_pointer(nll)) &&
                 (!dlogits || is_device_pointer(dlogits)),
             "pg_loss_backward_static: logits, targets, advantages, nll and dlogits must be device memory (host buffers would need staging allocations)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  double* scratch = nullptr;
  GN_TRY(static_scratch(&scratch));
  // The total and the bad-target count must start from zero; the row cells are rewritten by the kernel before the sum reads them.
  GN_CUDA(cudaMemsetAsync(scratch, 0, 2 * sizeof(double), s));
  GN_TRY(pg_loss_launch(logits, targets, advantages, rows, vocab, vocab, seq_len, norm, softcap, nll, dlogits, vocab, scratch + kStaticRowOffset, scratch, 1, s,
                        reinterpret_cast<int*>(scratch + 1)));
  int bad = 0;
  GN_CUDA(cudaMemcpyAsync(&bad, scratch + 1, sizeof(int), cudaMemcpyDeviceToHost, s));
  if (is_device_pointer(loss)) GN_CUDA(cudaMemcpyAsync(loss, scratch, sizeof(double), cudaMemcpyDeviceToDevice, s));
  else GN_CUDA(cudaMemcpyAsync(loss, scratch, sizeof(double), cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s));
  if (bad) { set_error("pg_loss_backward_static: %d targets outside {-1} and [0, %d)", bad, vocab); return GN_ERR_INVALID; }
  return GN_OK;
}

extern "C" int gn_static_loss_max_rows(void) { return GN_STATIC_LOSS_MAX_ROWS; }
