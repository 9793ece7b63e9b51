// The context behind gn_ctx: one device, one stream.
#pragma once
#include <cuda_runtime.h>

struct gn_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int gemm_kind = 1;
  bool use_graphs = true;   // replay the decode step as a CUDA graph
  int head_chunk_rows = 16384;   // rows of logits that exist at once in the training pass (lm_head, loss and their backward run in chunks)
  int optimizer_lanes = 4;      // streams the independent tensors of an optimizer step are spread over (1..4)
  bool optimizer_graph = true;  // replay the optimizer step (all but the few AdamW scalars, whose bias correction changes every step) as a CUDA graph
  int option_generation = 0;    // bumped by every option change: captured graphs are rebuilt
  void* comm = nullptr;     // ncclComm_t of the data-parallel job (gn_ctx_comm_init), null in a single-process run
  int comm_rank = 0, comm_world = 1;
};
