// Shared includes and small helpers of the library's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/cusync_b200.h"
#include "../../include/cusync/cusync_defines.h"
#include "../../include/cusync/policy_eval.h"
#include "../../include/cusync/device-functions.h"

// Orders run r + 1 of a multi-stream chain after run r: the first stream of a run waits for the event its
// previous run recorded on its last stream (the last stage completes after every stage before it, so one
// event covers the whole chain).  The reference's loops synchronise with the host between iterations instead
// (src/ml-bench/transformer/mlp.cu:699-700).
// Launches `kernel` as a programmatic dependent of the kernel before it in `stream`: it may start as soon as
// every block of that kernel has called cusync::allowDependentLaunch() or exited, not when the kernel has
// finished.  Nothing of the earlier kernel's memory is visible by that alone: the dependent synchronises
// through the stage's semaphores.
#if defined(__CUDACC__)
template <typename... Params, typename... Args>
inline cudaError_t launchDependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                   Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr;
  memset(&attr, 0, sizeof(attr));
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}
#endif

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
