// The context behind gn_ctx: one device, one stream.
#pragma once
#include <cuda_runtime.h>

struct gn_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int gemm_kind = 1;
  bool use_graphs = true;   // replay the decode step as a CUDA graph
};
