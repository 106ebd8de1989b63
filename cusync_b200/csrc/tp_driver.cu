// Tensor-parallel layer driver below the C ABI: one rank's MLP shard (mlp_driver.cu) plus the layer's single
// exchange step, the sum all-reduce of the row-parallel output across the ranks of one node.  The reference leaves
// that collective to its caller and only times it on its own (src/ml-bench/transformer/allreduce_times.py:11-35);
// its shard shapes are mlp.cu:243-251.  Two forms of the all-reduce:
//   * this library's kernel beside the second GEMM (allreduce.cu), over memory the caller made peer-accessible;
//   * NCCL's ncclAllReduce after the layer, on a communicator created here from a caller-distributed unique id
//     (one process per GPU).  NCCL is bound at run time from the process's libnccl.so.2, so the library itself has
//     no link-time dependency on it and single-GPU users need none.
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <new>

#include "common.cuh"

namespace {

// The part of NCCL's C API used here (nccl.h; these types and enumerators are part of its stable ABI).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;                     // ncclSuccess = 0
constexpr int kNcclFloat16 = 6;               // ncclDataType_t: ncclFloat16 / ncclHalf
constexpr int kNcclSum = 0;                   // ncclRedOp_t: ncclSum

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
  bool ok;
};

const NcclApi& nccl() {
  static NcclApi api = {};
  static std::once_flag once;
  std::call_once(once, [] {
    // the copy the process already uses (a framework may have loaded its own), else the system's
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce;
  });
  return api;
}

}  // namespace

struct cusync_tp_comm {
  ncclComm_t comm;
  int world, rank;
};

extern "C" {

int cusync_tp_unique_id(void* out128) {
  if (!out128) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (!nccl().ok) return CUSYNC_ERROR_UNSUPPORTED;
  ncclUniqueId id;
  if (nccl().GetUniqueId(&id) != 0) return CUSYNC_ERROR_CUDA;
  std::memcpy(out128, &id, sizeof(id));
  return CUSYNC_SUCCESS;
}

int cusync_tp_comm_create(cusync_tp_comm_t** out, int32_t world, int32_t rank, const void* unique_id128) {
  if (!out) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  if (world < 1 || rank < 0 || rank >= world) return CUSYNC_ERROR_INVALID_ARGUMENT;
  cusync_tp_comm* c = new (std::nothrow) cusync_tp_comm();
  if (!c) return CUSYNC_ERROR_CUDA;
  c->comm = nullptr; c->world = world; c->rank = rank;
  if (world > 1) {
    if (!unique_id128) { delete c; return CUSYNC_ERROR_INVALID_ARGUMENT; }
    if (!nccl().ok) { delete c; return CUSYNC_ERROR_UNSUPPORTED; }
    ncclUniqueId id;
    std::memcpy(&id, unique_id128, sizeof(id));
    if (nccl().CommInitRank(&c->comm, world, id, rank) != 0) { delete c; return CUSYNC_ERROR_CUDA; }
  }
  *out = c;
  return CUSYNC_SUCCESS;
}

int cusync_tp_comm_destroy(cusync_tp_comm_t* c) {
  if (!c) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (c->comm) nccl().CommDestroy(c->comm);
  delete c;
  return CUSYNC_SUCCESS;
}

int cusync_tp_all_reduce(cusync_tp_comm_t* c, void* buffer, uint64_t count, cusync_stream_t stream) {
  if (!c || !buffer) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (c->world == 1) return CUSYNC_SUCCESS;
  return nccl().AllReduce(buffer, buffer, static_cast<size_t>(count), kNcclFloat16, kNcclSum, c->comm,
                          reinterpret_cast<cudaStream_t>(stream)) == 0 ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_tp_layer_run(cusync_mlp_t* mlp, cusync_tp_comm_t* comm, cusync_allreduce_plan_t* reducer, void* y,
                        uint64_t y_count, cusync_stream_t producer_stream, cusync_stream_t consumer_stream,
                        cusync_stream_t reduce_stream) {
  if (!mlp) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (reducer) return cusync_mlp_run_cusync_allreduce(mlp, reducer, producer_stream, consumer_stream, reduce_stream);
  int rc = cusync_mlp_run_cusync(mlp, producer_stream, consumer_stream);
  if (rc == CUSYNC_SUCCESS && comm && comm->world > 1) rc = cusync_tp_all_reduce(comm, y, y_count, consumer_stream);
  return rc;
}

}  // extern "C"
