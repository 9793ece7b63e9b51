// The data-parallel exchange of the RL step inside the library: one communicator per context and a SUM all-reduce of
// the model's flat gradient buffer on the context's stream.
//
// The reference is a single-process program (optimizer/optimizer.go:5-7) and has no collective; its nearest analogue
// is gradient accumulation into Tensor.Grad (tensors/tensor.go:189-194), which is why the exchange is a plain SUM:
// the 1/norm factor is already inside dlogits (trainer/rl.go:41).  A host written in the reference's language
// needs nothing but this C-ABI: rank 0 asks for an id (gn_comm_unique_id), hands its 128 bytes to the other ranks by
// whatever means it has, and every rank calls gn_ctx_comm_init.
//
// NCCL is bound at run time (dlopen of libnccl.so.2): a process that already holds a copy of the library, such as
// one that imported torch, gets that copy, and a process that never initialises a communicator never loads it.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "model_internal.cuh"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mu;

int load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle) return GN_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) { gn::set_error("cannot load libnccl.so.2: %s", dlerror()); return GN_ERR_COMM; }
  NcclApi api;
  api.handle = h;
#define GN_SYM(field, name)                                                              \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(h, name));                     \
  if (!api.field) { gn::set_error("libnccl.so.2 lacks %s", name); dlclose(h); return GN_ERR_COMM; }
  GN_SYM(GetUniqueId, "ncclGetUniqueId");
  GN_SYM(CommInitRank, "ncclCommInitRank");
  GN_SYM(CommDestroy, "ncclCommDestroy");
  GN_SYM(CommAbort, "ncclCommAbort");
  GN_SYM(AllReduce, "ncclAllReduce");
  GN_SYM(Broadcast, "ncclBroadcast");
  GN_SYM(GroupStart, "ncclGroupStart");
  GN_SYM(GroupEnd, "ncclGroupEnd");
  GN_SYM(GetErrorString, "ncclGetErrorString");
#undef GN_SYM
  g_nccl = api;
  return GN_OK;
}

#define GN_NCCL(expr)                                                                                   \
  do {                                                                                                  \
    ncclResult_t r__ = (expr);                                                                          \
    if (r__ != ncclSuccess && r__ != ncclInProgress) {                                                  \
      gn::set_error("%s:%d: %s -> %s", __FILE__, __LINE__, #expr, g_nccl.GetErrorString(r__));          \
      return GN_ERR_COMM;                                                                               \
    }                                                                                                   \
  } while (0)

}  // namespace

extern "C" {

int gn_comm_unique_id(void* id_out) {
  GN_REQUIRE(id_out, "gn_comm_unique_id: null output");
  static_assert(GN_COMM_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "the id handed across the C-ABI is NCCL's unique id");
  GN_TRY(load_nccl());
  ncclUniqueId id;
  GN_NCCL(g_nccl.GetUniqueId(&id));
  std::memcpy(id_out, id.internal, GN_COMM_ID_BYTES);
  return GN_OK;
}

int gn_ctx_comm_init(gn_ctx* c, const void* id_in, int rank, int world) {
  GN_REQUIRE(c && id_in, "gn_ctx_comm_init: null argument");
  GN_REQUIRE(world >= 1 && rank >= 0 && rank < world, "gn_ctx_comm_init: rank %d of %d", rank, world);
  GN_REQUIRE(c->comm == nullptr, "gn_ctx_comm_init: the context already has a communicator");
  GN_TRY(load_nccl());
  GN_CUDA(cudaSetDevice(c->device));
  ncclUniqueId id;
  std::memcpy(id.internal, id_in, GN_COMM_ID_BYTES);
  ncclComm_t comm = nullptr;
  GN_NCCL(g_nccl.CommInitRank(&comm, world, id, rank));
  c->comm = comm; c->comm_rank = rank; c->comm_world = world;
  return GN_OK;
}

int gn_ctx_comm_destroy(gn_ctx* c) {
  GN_REQUIRE(c, "gn_ctx_comm_destroy: null context");
  if (!c->comm) return GN_OK;
  GN_CUDA(cudaSetDevice(c->device));
  cudaStreamSynchronize(c->stream);
  ncclResult_t r = g_nccl.CommDestroy(static_cast<ncclComm_t>(c->comm));
  c->comm = nullptr; c->comm_world = 1; c->comm_rank = 0;
  if (r != ncclSuccess) { gn::set_error("ncclCommDestroy -> %s", g_nccl.GetErrorString(r)); return GN_ERR_COMM; }
  return GN_OK;
}

int gn_model_grad_allreduce(gn_model* m) {
  GN_REQUIRE(m && m->ctx, "gn_model_grad_allreduce: null model");
  gn_ctx* c = m->ctx;
  GN_CUDA(cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  GN_CUDA(cudaEventRecord(m->ev[0], s));
  if (c->comm && c->comm_world > 1)
    GN_NCCL(g_nccl.AllReduce(m->G.p, m->G.p, (size_t)m->total, ncclFloat32, ncclSum, static_cast<ncclComm_t>(c->comm), s));
  GN_CUDA(cudaEventRecord(m->ev[1], s));
  GN_CUDA(cudaStreamSynchronize(s));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1]));
  m->phase_ms["allreduce"] = ms;
  return GN_OK;
}

int gn_ctx_allreduce_max_i64(gn_ctx* c, int64_t* value) {
  GN_REQUIRE(c && value, "gn_ctx_allreduce_max_i64: null argument");
  if (!c->comm || c->comm_world <= 1) return GN_OK;
  GN_CUDA(cudaSetDevice(c->device));
  int64_t* dev = nullptr;
  GN_CUDA(cudaMalloc((void**)&dev, sizeof(int64_t)));
  cudaError_t e = cudaMemcpyAsync(dev, value, sizeof(int64_t), cudaMemcpyHostToDevice, c->stream);
  ncclResult_t r = ncclSuccess;
  if (e == cudaSuccess) r = g_nccl.AllReduce(dev, dev, 1, ncclInt64, ncclMax, static_cast<ncclComm_t>(c->comm), c->stream);
  if (e == cudaSuccess && r == ncclSuccess) e = cudaMemcpyAsync(value, dev, sizeof(int64_t), cudaMemcpyDeviceToHost, c->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  cudaFree(dev);
  if (r != ncclSuccess) { gn::set_error("ncclAllReduce -> %s", g_nccl.GetErrorString(r)); return GN_ERR_COMM; }
  if (e != cudaSuccess) { gn::set_error("gn_ctx_allreduce_max_i64: %s", cudaGetErrorString(e)); return GN_ERR_CUDA; }
  return GN_OK;
}

// The second exchange of a sharded optimizer step: every tensor is broadcast from the rank that updated it (the
// owner assignment of gn_model_optimizer_step_shard), 1/world of the bytes an all-reduce of the whole buffer moves.
int gn_model_optimizer_exchange(gn_model* m) {
  GN_REQUIRE(m && m->ctx, "gn_model_optimizer_exchange: null model");
  gn_ctx* c = m->ctx;
  GN_CUDA(cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  GN_CUDA(cudaEventRecord(m->ev[0], s));
  if (c->comm && c->comm_world > 1) {
    const std::vector<int> owner = gnm::optimizer_owners(m, c->comm_world);
    GN_NCCL(g_nccl.GroupStart());
    for (size_t i = 0; i < m->params.size(); ++i) {
      const gnm::ParamInfo& pi = m->params[i];
      ncclResult_t r = g_nccl.Broadcast(m->p(pi.offset), m->p(pi.offset), (size_t)pi.rows * pi.cols, ncclFloat32, owner[i], static_cast<ncclComm_t>(c->comm), s);
      if (r != ncclSuccess) { g_nccl.GroupEnd(); gn::set_error("ncclBroadcast -> %s", g_nccl.GetErrorString(r)); return GN_ERR_COMM; }
    }
    GN_NCCL(g_nccl.GroupEnd());
  }
  GN_CUDA(cudaMemsetAsync(m->G.p, 0, sizeof(float) * m->total, s));   // ZeroGrad (trainer/rl.go:66)
  GN_CUDA(cudaMemsetAsync(m->sacc.p, 0, sizeof(double) * (2 * m->L + 2), s));
  GN_CUDA(cudaEventRecord(m->ev[1], s));
  m->weights_dirty = true;
  GN_CUDA(cudaStreamSynchronize(s));
  float ms = 0;
  GN_CUDA(cudaEventElapsedTime(&ms, m->ev[0], m->ev[1]));
  m->phase_ms["optimizer"] += ms;
  return GN_OK;
}

}  // extern "C"
