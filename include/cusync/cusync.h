// cusync.h -- C++ API of the B200-native CuSync library.
//
// Drop-in for the reference header of the same name
// (src/include/cusync/cusync.h): enum CuSyncError, enum Optimizations,
// class CuStage<TileOrder, InputSyncPolicy, OutputSyncPolicy, Opts> with
// grid / invokeWaitKernel / incrementIter / wait / post / tile and the getters,
// struct CuSync::setProducerConsumerPair, friend class CuSyncTest.
//
// What is behind it is new.  A CuStage is a trivially copyable value made of
//   * a handle to a stage object of the C ABI (cusync_b200.h), which owns the
//     device memory (schedule buffer, ticket counter, semaphores, started
//     words, timeout record), and
//   * a cached cusync_stage_view_t with the raw device pointers, which is what
//     the device-side methods use when the stage is passed by value to a kernel.
// Device side: post publishes with red.release.gpu (st.release.gpu under
// NoAtomicAdd); wait polls with ld.acquire.gpu, backs off with nanosleep, and
// gives up after the stage's time bound, leaving a record the host reads with
// status() -- a missed post can no longer hang the GPU.
#pragma once

#include <assert.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <type_traits>

#include <cuda_runtime_api.h>

#include "../cusync_b200.h"
#include "cusync_defines.h"

#ifndef CUDA_CHECK
#define CUDA_CHECK(cmd)                                                                      \
  do {                                                                                       \
    cudaError_t e_ = (cmd);                                                                  \
    if (e_ != cudaSuccess) {                                                                 \
      printf("Failed: Cuda error %s:%d '%s'\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
      exit(EXIT_FAILURE);                                                                    \
    }                                                                                        \
  } while (0)
#endif

#ifndef DIVUP
#define DIVUP(x, y) (((x) + (y) - 1) / (y))
#endif

#include "policies.h"
#include "tile-orders.h"
#include "wait-kernel.h"
#include "device-functions.h"

namespace cusync {

class CuSyncTest;
struct CuSync;

// Same enumerators in the same order as the reference (success is last);
// CuSyncErrorTimeout and later are additions.
enum CuSyncError {
  CuSyncErrorNotProducer = CUSYNC_ERROR_NOT_PRODUCER,
  CuSyncErrorNotConsumer = CUSYNC_ERROR_NOT_CONSUMER,
  CuSyncErrorNotInitialized = CUSYNC_ERROR_NOT_INITIALIZED,
  CuSyncErrorInvalidLinearBlockIndex = CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX,
  CuSyncErrorCUDAError = CUSYNC_ERROR_CUDA,
  CuSyncSuccess = CUSYNC_SUCCESS,
  CuSyncErrorTimeout = CUSYNC_ERROR_TIMEOUT,
  CuSyncErrorInvalidArgument = CUSYNC_ERROR_INVALID_ARGUMENT,
  CuSyncErrorUnsupported = CUSYNC_ERROR_UNSUPPORTED
};

enum Optimizations {
  NoOptimization = CUSYNC_OPT_NONE,
  NoAtomicAdd = CUSYNC_OPT_NO_ATOMIC_ADD,            // each semaphore has one poster: store instead of add
  AvoidWaitKernel = CUSYNC_OPT_AVOID_WAIT_KERNEL,    // all stages fit one wave: no wait kernel
  AvoidCustomOrder = CUSYNC_OPT_AVOID_CUSTOM_ORDER,  // take blockIdx instead of a ticket
  ReorderTileLoads = CUSYNC_OPT_REORDER_TILE_LOADS,  // load independent operands before waiting
  StreamWait = CUSYNC_OPT_STREAM_WAIT                // addition: invokeWaitKernel as a stream memory operation
};

namespace detail {
// Policy record of a policy type: built-in policies (and user policies that
// opt in) provide desc(); any other user policy is marked "custom", which the
// header-compiled device code handles and the pre-compiled kernels refuse.
template <typename P, typename = void>
struct PolicyRecord {
  static cusync_policy_t get(const P&) { return cusync_policy_t{CUSYNC_POLICY_CUSTOM, 0, 1, 1, 0, 0, 0, 0}; }
};
template <typename P>
struct PolicyRecord<P, decltype((void)std::declval<const P&>().desc())> {
  static cusync_policy_t get(const P& p) { return p.desc(); }
};
}  // namespace detail

template <typename TileOrder, typename InputSyncPolicy, typename OutputSyncPolicy, int Opts = NoOptimization>
class CuStage {
 private:
  cusync_stage_t* handle_;      // host-side owner of the device state
  cusync_stage_view_t view_;    // raw device pointers + grids, valid on the device
  int iter;                     // run counter of THIS copy, starts at 1
  InputSyncPolicy inputPolicy_;
  OutputSyncPolicy outputPolicy_;

  friend class CuSyncTest;
  friend struct CuSync;

  CUSYNC_DEVICE_HOST dim3 prodGrid() const { return dim3(view_.prod_grid.x, view_.prod_grid.y, view_.prod_grid.z); }
  CUSYNC_DEVICE_HOST dim3 ownGrid() const { return dim3(view_.grid.x, view_.grid.y, view_.grid.z); }

 public:
  // Allocates the stage's device state through the C ABI.  CUDA failures print
  // and exit, as the reference's CUDA_CHECK does.
  CuStage(dim3 grid, dim3 tileSize, InputSyncPolicy inputPolicy, OutputSyncPolicy outputPolicy)
      : handle_(nullptr), iter(1), inputPolicy_(inputPolicy), outputPolicy_(outputPolicy) {
    cusync_policy_t in = detail::PolicyRecord<InputSyncPolicy>::get(inputPolicy);
    cusync_policy_t out = detail::PolicyRecord<OutputSyncPolicy>::get(outputPolicy);
    int order = TileOrder::kOrderKind >= 0 ? TileOrder::kOrderKind : CUSYNC_ORDER_IDENTITY;
    int rc = cusync_stage_create(&handle_, cusync_dim3_t{grid.x, grid.y, grid.z},
                                 cusync_dim3_t{tileSize.x, tileSize.y, tileSize.z}, order, &in, &out, Opts);
    if (rc != CUSYNC_SUCCESS && rc != CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX) {
      printf("Failed: cusync_stage_create returned %d at %s:%d\n", rc, __FILE__, __LINE__);
      exit(EXIT_FAILURE);
    }
    if (TileOrder::kOrderKind < 0) {
      // User-defined order: build the schedule buffer from its blockIndex.
      uint32_t n = grid.x * grid.y * grid.z;
      cusync_dim3_t* order_host = new cusync_dim3_t[n];
      for (uint32_t i = 0; i < n; i++) order_host[i] = cusync_dim3_t{n, 0, 0};
      bool bad = false;
      for (uint32_t z = 0; z < grid.z; z++)
        for (uint32_t y = 0; y < grid.y; y++)
          for (uint32_t x = 0; x < grid.x; x++) {
            uint32_t id = TileOrder().blockIndex(grid, dim3(x, y, z));
            if (id >= n || order_host[id].x != n) { bad = true; continue; }
            order_host[id] = cusync_dim3_t{x, y, z};
          }
      rc = cusync_stage_write_tile_order(handle_, order_host, n);
      delete[] order_host;
      if (bad) rc = CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX;
    }
    createStatus_ = static_cast<CuSyncError>(rc);
    cusync_stage_get_view(handle_, &view_);
  }

  CUSYNC_DEVICE_HOST CuStage() : handle_(nullptr), view_(), iter(1) {}

  // Status of construction: CuSyncSuccess, or CuSyncErrorInvalidLinearBlockIndex
  // when the tile order does not number the grid's blocks 0..numTiles-1.
  CuSyncError createStatus() const { return createStatus_; }

  dim3 grid() { return ownGrid(); }

  CuSyncError invokeWaitKernel(cudaStream_t stream) {
    if (!isProducer()) return CuSyncErrorNotProducer;
    if (handle_ == nullptr) return CuSyncErrorNotInitialized;
    cusync_stage_set_iter(handle_, static_cast<uint32_t>(iter));
    return static_cast<CuSyncError>(
        cusync_stage_invoke_wait_kernel(handle_, reinterpret_cast<cusync_stream_t>(stream)));
  }

  // Every copy of a stage carries its own run counter, as in the reference:
  // increment the host objects and the by-value copies held by kernel handles.
  void incrementIter() {
    iter += 1;
    view_.iter = static_cast<uint32_t>(iter);
    if (handle_) cusync_stage_set_iter(handle_, static_cast<uint32_t>(iter));
  }

  // Additions: release the device state (the reference leaks it), re-arm after
  // an error, set the spin bound, read the timeout record.
  void destroy() { if (handle_) { cusync_stage_destroy(handle_); handle_ = nullptr; } }
  CuSyncError reset(cudaStream_t stream = 0) {
    iter = 1; view_.iter = 1;
    return static_cast<CuSyncError>(cusync_stage_reset(handle_, reinterpret_cast<cusync_stream_t>(stream)));
  }
  void setTimeoutNs(uint64_t ns) { cusync_stage_set_timeout_ns(handle_, ns); view_.timeout_ns = ns; }
  cusync_status_t status() const { cusync_status_t s{}; cusync_stage_read_status(handle_, &s); return s; }
  cusync_stage_t* handle() const { return handle_; }
  uint32_t currentIter() const { return static_cast<uint32_t>(iter); }

  CUSYNC_DEVICE_HOST bool getNoAtomicAdd() { return Opts & NoAtomicAdd; }
  CUSYNC_DEVICE_HOST bool getAvoidWaitKernel() { return Opts & AvoidWaitKernel; }
  CUSYNC_DEVICE_HOST bool getReorderTileLoads() { return Opts & ReorderTileLoads; }
  CUSYNC_DEVICE_HOST bool getAvoidCustomOrder() { return Opts & AvoidCustomOrder; }

  CUSYNC_DEVICE_HOST bool isProducer() { return !std::is_same<OutputSyncPolicy, NoSync>::value; }
  CUSYNC_DEVICE_HOST bool isConsumer() { return !std::is_same<InputSyncPolicy, NoSync>::value; }
  CUSYNC_DEVICE_HOST uint32_t numTiles() { return view_.grid.x * view_.grid.y * view_.grid.z; }

#if defined(__CUDACC__) || defined(__NVCC__)
  // Semaphore index / current value / per-run target of the wait a tile makes.
  CUSYNC_DEVICE uint32_t waitTileIndex(dim3 tile) { return inputPolicy_.tileIndex(tile, prodGrid()); }
  CUSYNC_DEVICE uint32_t waitSemValue(dim3 tile) { return loadAcquire(view_.sems_wait + waitTileIndex(tile)); }
  CUSYNC_DEVICE uint32_t expectedWaitValue(dim3 tile) { return inputPolicy_.waitValue(tile, prodGrid()); }

  // Block until the producer tile(s) this tile depends on are published.
  // `waitingThread` polls; with callSync every thread of the block learns the
  // outcome.  Returns CuSyncErrorTimeout if the bound expired.
  CUSYNC_DEVICE CuSyncError wait(dim3& tile, uint32_t waitingThread = 0, bool callSync = true) {
    if (!isConsumer()) return CuSyncErrorNotConsumer;
    if (!inputPolicy_.isSync(tile, prodGrid())) return CuSyncSuccess;
    int timedOut = 0;
    if (threadIdx.x == waitingThread && threadIdx.y == 0 && threadIdx.z == 0) {
      const uint32_t idx = inputPolicy_.tileIndex(tile, prodGrid());
      const uint32_t expected = static_cast<uint32_t>(iter) * inputPolicy_.waitValue(tile, prodGrid());
      uint32_t seen = 0;
      if (!spinUntilAtLeast(view_.sems_wait + idx, expected, view_.timeout_ns, &seen)) {
        recordTimeout(view_.status, 1u, tile.x, tile.y, tile.z, idx, seen, expected);
        timedOut = 1;
      }
    }
    if (callSync) timedOut = __syncthreads_or(timedOut);
    return timedOut ? CuSyncErrorTimeout : CuSyncSuccess;
  }

  // Publish a finished tile.  All threads' earlier global writes are ordered
  // before the release by the block barrier plus the releasing thread's fence.
  CUSYNC_DEVICE CuSyncError post(const dim3& tile, uint32_t postThread = 0) {
    if (!isProducer()) return CuSyncErrorNotProducer;
    __syncthreads();
    if (threadIdx.x == postThread && threadIdx.y == 0 && threadIdx.z == 0) {
      const uint32_t idx = outputPolicy_.tileIndex(tile, ownGrid());
      const uint32_t value = outputPolicy_.postValue(tile, ownGrid());
      __threadfence();
      if (Opts & NoAtomicAdd) storeRelease(view_.sems_post + idx, value * static_cast<uint32_t>(iter));
      else                    addRelease(view_.sems_post + idx, value);
    }
    __syncwarp();
    return CuSyncSuccess;
  }

  // Next tile of this block: a ticket into the schedule buffer, so tiles are
  // taken in tile-order whatever order the hardware starts blocks in.  Block
  // (0,0,0) of a producer also marks the kernel as started for the wait kernel.
  CUSYNC_DEVICE dim3 tile(dim3* shared_storage) {
    const bool lead = threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0;
    if (!(Opts & AvoidWaitKernel) && lead && isProducer() && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
      storeRelease(view_.started, static_cast<uint32_t>(iter));
    if ((Opts & AvoidCustomOrder) || shared_storage == nullptr) return blockIdx;
    if (lead) {
      const uint32_t ticket = atomicAdd(view_.tile_counter, 1u);
      if (ticket == numTiles() - 1) *view_.tile_counter = 0;   // last ticket re-arms the counter
      const cusync_dim3_t t = view_.tile_order[ticket];
      *shared_storage = dim3(t.x, t.y, t.z);
    }
    __syncthreads();
    return *shared_storage;
  }
#endif

 private:
  CuSyncError createStatus_ = CuSyncSuccess;
};

struct CuSync {
  // Wire a producer stage to a consumer stage: the consumer learns the
  // producer's grid and waits on the producer's semaphore array.
  template <typename Stage1, typename Stage2>
  static CuSyncError setProducerConsumerPair(Stage1& prod, Stage2& cons) {
    if (!prod.isProducer()) return CuSyncErrorNotProducer;
    if (!cons.isConsumer()) return CuSyncErrorNotConsumer;
    if (prod.handle_ == nullptr || cons.handle_ == nullptr) return CuSyncErrorNotInitialized;
    CuSyncError rc = static_cast<CuSyncError>(cusync_stage_link(prod.handle_, cons.handle_));
    if (rc == CuSyncSuccess) cusync_stage_get_view(cons.handle_, &cons.view_), cons.view_.iter = cons.iter;
    return rc;
  }
  template <typename Stage1, typename Stage2>
  static CuSyncError setProducerConsumer(Stage1& prod, Stage2& cons) { return setProducerConsumerPair(prod, cons); }
};

}  // namespace cusync
