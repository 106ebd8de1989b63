// Shared includes and small helpers of the library's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cusync_b200.h"
#include "../../include/cusync/cusync_defines.h"
#include "../../include/cusync/policy_eval.h"
#include "../../include/cusync/device-functions.h"

// Orders run r + 1 of a multi-stream chain after run r: the first stream of a run waits for the event its
// previous run recorded on its last stream (the last stage completes after every stage before it, so one
// event covers the whole chain).  The reference's loops synchronise with the host between iterations instead
// (src/ml-bench/transformer/mlp.cu:699-700).
struct RunOrder {
  cudaEvent_t done = nullptr;
  bool recorded = false;
  bool create() { return cudaEventCreateWithFlags(&done, cudaEventDisableTiming) == cudaSuccess; }
  void destroy() { if (done) cudaEventDestroy(done); done = nullptr; }
  bool begin(cusync_stream_t first) {
    return !recorded || cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(first), done, 0) == cudaSuccess;
  }
  bool end(cusync_stream_t last) {
    recorded = cudaEventRecord(done, reinterpret_cast<cudaStream_t>(last)) == cudaSuccess;
    return recorded;
  }
};
