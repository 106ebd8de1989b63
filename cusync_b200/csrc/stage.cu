// Stage objects of the C ABI: the device-side state a CuStage owns (schedule
// buffer, ticket counter, semaphores, started words, timeout record), the
// producer/consumer wiring, and the wait kernel.
//
// Replaces, for sm_100a: CuStage's constructor and buildScheduleBuffer
// (src/include/cusync/cusync.h:125-198), CuSync::setProducerConsumerPair
// (cusync.h:287-299) and waitKernel / invokeWaitKernel (src/cusync.cu:11-25).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

struct cusync_stage {
  cusync_stage_view_t view;      // host master copy; `iter` lives here
  bool is_producer;
  bool is_consumer;
  bool linked;
  uint32_t num_tiles;
  uint32_t num_sems;             // entries of the semaphore array this stage owns
  uint64_t blocks_launched;      // persistent-kernel blocks launched over all runs
  bool     launch_noted;         // a persistent launch was noted for the current run
  int device;
  // Producer <-> consumer links (cusync_stage_link), kept in both directions so that either side may be
  // destroyed first: the producer tells its consumers when its launch of a run has been noted.
  cusync_stage* producer;                 // consumer: the stage it waits on, or null
  std::vector<cusync_stage*>* consumers;  // producer: stages linked to it (allocated on the first link)
  uint32_t prod_target;                   // consumer: "blocks finished" count at which this run's producer is done
  uint32_t prod_target_iter;              // consumer: the run that count belongs to (0: none)
};

namespace {

// One thread spins until *sem >= value, with back-off and a time bound.
__global__ void waitKernel(const uint32_t* sem, uint32_t value, uint32_t* status, uint64_t timeout_ns) {
  if (threadIdx.x != 0) return;
  uint32_t seen = 0;
  if (!cusync::spinUntilAtLeast(sem, value, timeout_ns, &seen))
    cusync::recordTimeout(status, 3u, 0, 0, 0, 0, seen, value);
}

// The same for a counter that wraps (the 32-bit "blocks started" word counts every block of every run): done
// when the counter has reached `value` in the cyclic sense the driver's stream waits use,
// (int32_t)(*counter - value) >= 0.
__global__ void waitCounterKernel(const uint32_t* counter, uint32_t value, uint32_t* status, uint64_t timeout_ns) {
  if (threadIdx.x != 0) return;
  const uint64_t t0 = cusync::globalTimerNs();
  const uint64_t bound = timeout_ns ? timeout_ns : cusync::kDefaultSpinTimeoutNs;
  uint32_t backoff = 32;
  while (true) {
    const uint32_t v = cusync::loadAcquire(counter);
    if (static_cast<int32_t>(v - value) >= 0) return;
    if (cusync::globalTimerNs() - t0 > bound) { cusync::recordTimeout(status, 3u, 0, 0, 0, 0, v, value); return; }
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
}

// One thread per semaphore of a contiguous range; the kernel ends when every one has reached `value`.
__global__ void waitRangeKernel(const uint32_t* sems, uint32_t count, uint32_t value, uint32_t* status,
                                uint64_t timeout_ns) {
  for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
    uint32_t seen = 0;
    if (!cusync::spinUntilAtLeast(sems + i, value, timeout_ns, &seen))
      cusync::recordTimeout(status, 3u, i, 0, 0, i, seen, value);
  }
}

// Stream memory operations of the driver (cuStreamWaitValue32 / cuStreamWriteValue32): a stream waits for, or
// writes, a 32-bit word without a kernel.  A kernel would need room on an SM, and the persistent GEMM blocks leave
// none: a one-thread kernel enqueued while they are resident starts only when one of them retires.
typedef CUresult (*StreamValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

StreamValueFn stream_value_fn(const char* name) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      sym == nullptr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return reinterpret_cast<StreamValueFn>(sym);
}

// With lazy module loading the first launch of a kernel loads it onto the device, and that load can wait for
// kernels that are already running.  A wait kernel is launched exactly when a persistent producer (or an
// all-reduce kernel spinning on semaphores) is running, so its first launch would stall the host until that
// kernel ends: load the wait kernels when the first stage is created instead.
void preload_wait_kernels() {
  static bool done = false;
  if (done) return;
  cudaFuncAttributes a;
  (void)cudaFuncGetAttributes(&a, waitKernel);
  (void)cudaFuncGetAttributes(&a, waitCounterKernel);
  (void)cudaFuncGetAttributes(&a, waitRangeKernel);
  (void)cudaGetLastError();
  done = true;
}

bool policy_ok(const cusync_policy_t* p) {
  if (p == nullptr) return true;
  if (p->kind < CUSYNC_POLICY_NOSYNC || p->kind > CUSYNC_POLICY_CUSTOM) return false;
  if (p->kind == CUSYNC_POLICY_NOSYNC || p->kind == CUSYNC_POLICY_CUSTOM) return true;
  if (p->order != CUSYNC_ORDER_IDENTITY && p->order != CUSYNC_ORDER_TRANSPOSE_XY) return false;
  if (p->tile_m == 0 || p->tile_n == 0) return false;
  if (p->kind == CUSYNC_POLICY_CONV2DTILESYNC && p->p0 == 0) return false;
  if (p->kind == CUSYNC_POLICY_STRIDEDTILESYNC && (p->p0 < p->tile_n || p->p1 == 0)) return false;
  if (p->kind == CUSYNC_POLICY_CONSECUTIVETILESYNC && (p->p0 / 8) < p->tile_n) return false;
  return true;
}

// Several semaphores go to the stream as ONE batched operation (cuStreamBatchMemOp) where the driver has it:
// every separate stream memory operation is a submission of its own and a bubble between the copies or kernels
// around it.
typedef CUresult (*StreamBatchFn)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);
constexpr uint32_t kBatchOps = 64;

int stream_values(bool wait, uint32_t* semaphores, uint32_t count, uint32_t value, cusync_stream_t stream) {
  if (semaphores == nullptr || count == 0) return CUSYNC_ERROR_NOT_INITIALIZED;
  static StreamValueFn wait_fn = stream_value_fn("cuStreamWaitValue32");
  static StreamValueFn write_fn = stream_value_fn("cuStreamWriteValue32");
  static StreamBatchFn batch_fn = reinterpret_cast<StreamBatchFn>(stream_value_fn("cuStreamBatchMemOp"));
  StreamValueFn fn = wait ? wait_fn : write_fn;
  if (!fn) return CUSYNC_ERROR_UNSUPPORTED;
  CUstream cs = reinterpret_cast<CUstream>(stream);
  uint32_t done = 0;
  if (batch_fn && count > 1) {
    CUstreamBatchMemOpParams ops[kBatchOps];
    while (done < count) {
      const uint32_t n = count - done < kBatchOps ? count - done : kBatchOps;
      memset(ops, 0, sizeof(CUstreamBatchMemOpParams) * n);
      for (uint32_t i = 0; i < n; i++) {
        const CUdeviceptr addr = reinterpret_cast<CUdeviceptr>(semaphores + done + i);
        if (wait) {
          ops[i].waitValue.operation = CU_STREAM_MEM_OP_WAIT_VALUE_32;
          ops[i].waitValue.address = addr;
          ops[i].waitValue.value = value;
          ops[i].waitValue.flags = CU_STREAM_WAIT_VALUE_GEQ;
        } else {
          ops[i].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_32;
          ops[i].writeValue.address = addr;
          ops[i].writeValue.value = value;
          ops[i].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT;
        }
      }
      if (batch_fn(cs, n, ops, 0) != CUDA_SUCCESS) break;   // fall back to single operations for the rest
      done += n;
    }
  }
  for (uint32_t i = done; i < count; i++)
    if (fn(cs, reinterpret_cast<CUdeviceptr>(semaphores + i), value,
           wait ? CU_STREAM_WAIT_VALUE_GEQ : CU_STREAM_WRITE_VALUE_DEFAULT) != CUDA_SUCCESS)
      return CUSYNC_ERROR_CUDA;
  return CUSYNC_SUCCESS;
}

}  // namespace

extern "C" {

int cusync_stage_create(cusync_stage_t** out, cusync_dim3_t grid, cusync_dim3_t tile_size, int order,
                        const cusync_policy_t* in_policy, const cusync_policy_t* out_policy, int opts) {
  if (out == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  if (grid.x == 0 || grid.y == 0 || grid.z == 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const int order_kind = order & 0xff;
  const uint32_t group_rows = static_cast<uint32_t>(order) >> 8;
  if (order_kind != CUSYNC_ORDER_IDENTITY && order_kind != CUSYNC_ORDER_TRANSPOSE_XY &&
      order_kind != CUSYNC_ORDER_GROUPED_ROWS)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if ((order_kind == CUSYNC_ORDER_GROUPED_ROWS) != (group_rows != 0)) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (!policy_ok(in_policy) || !policy_ok(out_policy)) return CUSYNC_ERROR_INVALID_ARGUMENT;
  uint64_t n64 = (uint64_t)grid.x * grid.y * grid.z;
  if (n64 > (1ull << 30)) return CUSYNC_ERROR_INVALID_ARGUMENT;

  cusync_stage* s = new (std::nothrow) cusync_stage();
  if (s == nullptr) return CUSYNC_ERROR_CUDA;
  std::memset(s, 0, sizeof(*s));
  s->num_tiles = (uint32_t)n64;
  s->view.grid = grid;
  s->view.tile_size = tile_size;
  s->view.iter = 1;
  s->view.opts = opts;
  s->view.order = order;
  if (in_policy) s->view.in_policy = *in_policy;
  if (out_policy) s->view.out_policy = *out_policy;
  s->is_consumer = s->view.in_policy.kind != CUSYNC_POLICY_NOSYNC;
  s->is_producer = s->view.out_policy.kind != CUSYNC_POLICY_NOSYNC;
  s->view.timeout_ns = cusync::kDefaultSpinTimeoutNs;
  if (cudaGetDevice(&s->device) != cudaSuccess) { delete s; return CUSYNC_ERROR_CUDA; }
  preload_wait_kernels();

  // Schedule buffer: slot blockIndex(grid, block) holds block (x, y, z).  The
  // reference's two orders linearise the launch grid x-fastest; the grouped
  // order walks groups of rows.  A slot written twice or a slot out of range
  // is the invalid-linear-index error.
  std::vector<cusync_dim3_t> order_host(s->num_tiles, cusync_dim3_t{s->num_tiles, 0, 0});
  bool invalid = false;
  for (uint32_t z = 0; z < grid.z; z++)
    for (uint32_t y = 0; y < grid.y; y++)
      for (uint32_t x = 0; x < grid.x; x++) {
        uint32_t id = order_kind == CUSYNC_ORDER_GROUPED_ROWS
                          ? cusync::eval::groupedBlockIndex(group_rows, grid.x, grid.y, x, y, z)
                          : cusync::eval::blockIndex(grid.x, grid.y, x, y, z);
        if (id >= s->num_tiles || order_host[id].x != s->num_tiles) { invalid = true; continue; }
        order_host[id] = cusync_dim3_t{x, y, z};
      }

  // One allocation for the small words: ticket counter, started[2], status[8].
  uint32_t* words = nullptr;
  bool ok = cudaMalloc(&words, 16 * sizeof(uint32_t)) == cudaSuccess &&
            cudaMemset(words, 0, 16 * sizeof(uint32_t)) == cudaSuccess &&
            cudaMalloc(&s->view.tile_order, sizeof(cusync_dim3_t) * s->num_tiles) == cudaSuccess &&
            cudaMemcpy(s->view.tile_order, order_host.data(), sizeof(cusync_dim3_t) * s->num_tiles,
                       cudaMemcpyHostToDevice) == cudaSuccess;
  if (ok && s->is_producer) {
    s->num_sems = s->num_tiles;
    ok = cudaMalloc(&s->view.sems_post, sizeof(uint32_t) * s->num_sems) == cudaSuccess &&
         cudaMemset(s->view.sems_post, 0, sizeof(uint32_t) * s->num_sems) == cudaSuccess;
  }
  if (!ok) {
    cudaFree(words); cudaFree(s->view.tile_order); cudaFree(s->view.sems_post);
    delete s;
    (void)cudaGetLastError();
    return CUSYNC_ERROR_CUDA;
  }
  s->view.tile_counter = words;
  s->view.started = words + 2;
  s->view.status = words + 8;
  *out = s;
  return invalid ? CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX : CUSYNC_SUCCESS;
}

int cusync_stage_destroy(cusync_stage_t* s) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  // undo the links in both directions
  if (s->producer && s->producer->consumers) {
    std::vector<cusync_stage*>& v = *s->producer->consumers;
    for (size_t i = 0; i < v.size(); i++)
      if (v[i] == s) { v.erase(v.begin() + i); break; }
  }
  if (s->consumers) {
    for (cusync_stage* c : *s->consumers) { c->producer = nullptr; c->prod_target_iter = 0; }
    delete s->consumers;
  }
  cudaFree(s->view.tile_counter);
  cudaFree(s->view.tile_order);
  cudaFree(s->view.sems_post);   // owned by the producer; consumers only alias it
  delete s;
  return CUSYNC_SUCCESS;
}

int cusync_stage_link(cusync_stage_t* prod, cusync_stage_t* cons) {
  if (prod == nullptr || cons == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!prod->is_producer) return CUSYNC_ERROR_NOT_PRODUCER;
  if (!cons->is_consumer) return CUSYNC_ERROR_NOT_CONSUMER;
  if (prod->view.sems_post == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  cons->view.prod_grid = prod->view.grid;
  cons->view.sems_wait = prod->view.sems_post;
  cons->linked = true;
  if (cons->producer != prod) {
    if (cons->producer && cons->producer->consumers) {          // re-linked to another producer
      std::vector<cusync_stage*>& v = *cons->producer->consumers;
      for (size_t i = 0; i < v.size(); i++)
        if (v[i] == cons) { v.erase(v.begin() + i); break; }
    }
    if (!prod->consumers) prod->consumers = new (std::nothrow) std::vector<cusync_stage*>();
    if (prod->consumers) { prod->consumers->push_back(cons); cons->producer = prod; }
    else cons->producer = nullptr;
    cons->prod_target_iter = 0;
  }
  return CUSYNC_SUCCESS;
}

int cusync_stage_increment_iter(cusync_stage_t* s) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  s->view.iter += 1;
  s->launch_noted = false;
  return CUSYNC_SUCCESS;
}

int cusync_stage_set_iter(cusync_stage_t* s, uint32_t iter) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (iter != s->view.iter) s->launch_noted = false;
  s->view.iter = iter;
  return CUSYNC_SUCCESS;
}

int cusync_stage_write_tile_order(cusync_stage_t* s, const cusync_dim3_t* order, uint32_t count) {
  if (s == nullptr || order == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (count != s->num_tiles) return CUSYNC_ERROR_INVALID_ARGUMENT;
  return cudaMemcpy(s->view.tile_order, order, sizeof(cusync_dim3_t) * count, cudaMemcpyHostToDevice) == cudaSuccess
             ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_stage_reset(cusync_stage_t* s, cusync_stream_t stream) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  cudaStream_t st = (cudaStream_t)stream;
  bool ok = cudaMemsetAsync(s->view.tile_counter, 0, 16 * sizeof(uint32_t), st) == cudaSuccess;
  if (ok && s->view.sems_post)
    ok = cudaMemsetAsync(s->view.sems_post, 0, sizeof(uint32_t) * s->num_sems, st) == cudaSuccess;
  s->view.iter = 1;
  s->blocks_launched = 0;
  s->launch_noted = false;
  s->prod_target_iter = 0;
  if (s->consumers)
    for (cusync_stage* c : *s->consumers) c->prod_target_iter = 0;
  return ok ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_stage_get_view(const cusync_stage_t* s, cusync_stage_view_t* out) {
  if (s == nullptr || out == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  *out = s->view;
  // the producer's finish count, when its launch of this very run has been noted already
  out->prod_finished = nullptr;
  out->prod_finish_target = 0;
  if (s->producer && s->prod_target_iter == s->view.iter && s->producer->view.iter == s->view.iter) {
    out->prod_finished = s->producer->view.started + 2;
    out->prod_finish_target = s->prod_target;
  }
  return CUSYNC_SUCCESS;
}

int cusync_stage_set_timeout_ns(cusync_stage_t* s, uint64_t ns) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  s->view.timeout_ns = ns ? ns : cusync::kDefaultSpinTimeoutNs;
  return CUSYNC_SUCCESS;
}

int cusync_stage_note_launch(cusync_stage_t* s, uint32_t num_blocks) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  s->blocks_launched += num_blocks;
  s->launch_noted = true;
  if (s->consumers)
    for (cusync_stage* c : *s->consumers) {
      c->prod_target = static_cast<uint32_t>(s->blocks_launched & 0xffffffffull);
      c->prod_target_iter = s->view.iter;
    }
  return CUSYNC_SUCCESS;
}

int cusync_wait_kernel(uint32_t* semaphore, uint32_t given_value, cusync_stream_t stream, uint32_t* status,
                       uint64_t timeout_ns) {
  if (semaphore == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  waitKernel<<<1, 1, 0, (cudaStream_t)stream>>>(semaphore, given_value, status, timeout_ns);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_wait_kernel_range(uint32_t* semaphores, uint32_t count, uint32_t given_value, cusync_stream_t stream,
                             uint32_t* status, uint64_t timeout_ns) {
  if (semaphores == nullptr || count == 0) return CUSYNC_ERROR_NOT_INITIALIZED;
  const uint32_t threads = count < 256u ? ((count + 31u) / 32u) * 32u : 256u;
  waitRangeKernel<<<1, threads, 0, (cudaStream_t)stream>>>(semaphores, count, given_value, status, timeout_ns);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_stream_wait_values(uint32_t* semaphores, uint32_t count, uint32_t value, cusync_stream_t stream) {
  return stream_values(true, semaphores, count, value, stream);
}

int cusync_stream_write_values(uint32_t* semaphores, uint32_t count, uint32_t value, cusync_stream_t stream) {
  return stream_values(false, semaphores, count, value, stream);
}

int cusync_stage_invoke_wait_kernel(cusync_stage_t* s, cusync_stream_t stream) {
  if (s == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!s->is_producer) return CUSYNC_ERROR_NOT_PRODUCER;
  if (s->view.opts & CUSYNC_OPT_AVOID_WAIT_KERNEL) return CUSYNC_SUCCESS;
  // The device counter is 32 bits wide and wraps; both forms below compare cyclically against the low 32 bits
  // of the host's running total.
  const uint32_t launched = static_cast<uint32_t>(s->blocks_launched & 0xffffffffull);
  if (s->launch_noted && (s->view.opts & CUSYNC_OPT_STREAM_WAIT)) {
    const int rc = cusync_stream_wait_values(s->view.started + 1, 1, launched, stream);
    if (rc != CUSYNC_ERROR_UNSUPPORTED) return rc;
  }
  if (s->launch_noted) {  // persistent kernel: wait until every block of the launch is resident
    waitCounterKernel<<<1, 1, 0, (cudaStream_t)stream>>>(s->view.started + 1, launched, s->view.status,
                                                         s->view.timeout_ns);
    return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
  }
  return cusync_wait_kernel(s->view.started, s->view.iter, stream, s->view.status, s->view.timeout_ns);
}

int cusync_stage_read_tile_order(const cusync_stage_t* s, cusync_dim3_t* out, uint32_t count) {
  if (s == nullptr || out == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (count > s->num_tiles) return CUSYNC_ERROR_INVALID_ARGUMENT;
  return cudaMemcpy(out, s->view.tile_order, sizeof(cusync_dim3_t) * count, cudaMemcpyDeviceToHost) == cudaSuccess
             ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_stage_read_semaphores(const cusync_stage_t* s, uint32_t* out, uint32_t count) {
  if (s == nullptr || out == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!s->is_producer) return CUSYNC_ERROR_NOT_PRODUCER;
  if (count > s->num_sems) return CUSYNC_ERROR_INVALID_ARGUMENT;
  return cudaMemcpy(out, s->view.sems_post, sizeof(uint32_t) * count, cudaMemcpyDeviceToHost) == cudaSuccess
             ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

int cusync_stage_read_status(const cusync_stage_t* s, cusync_status_t* out) {
  if (s == nullptr || out == nullptr) return CUSYNC_ERROR_NOT_INITIALIZED;
  return cudaMemcpy(out, s->view.status, sizeof(cusync_status_t), cudaMemcpyDeviceToHost) == cudaSuccess
             ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

uint32_t cusync_stage_num_tiles(const cusync_stage_t* s) { return s ? s->num_tiles : 0; }
uint32_t cusync_stage_iter(const cusync_stage_t* s) { return s ? s->view.iter : 0; }

const char* cusync_b200_version(void) { return "cusync_b200 0.1 (sm_100a)"; }

int cusync_b200_sm_count(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

}  // extern "C"
