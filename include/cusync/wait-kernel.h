// The one non-template symbol of the reference library
// (src/include/cusync/wait-kernel.h:10): enqueue a one-thread kernel that
// returns once *semaphore >= givenValue.  Here it forwards to the C ABI, whose
// kernel backs off with nanosleep and gives up after a time bound.
#pragma once

#include <cuda_runtime_api.h>
#include <stdint.h>
#include "../cusync_b200.h"

namespace cusync {
inline void invokeWaitKernel(uint32_t* semaphore, uint32_t givenValue, cudaStream_t stream) {
  cusync_wait_kernel(semaphore, givenValue, reinterpret_cast<cusync_stream_t>(stream), nullptr, 0);
}
}  // namespace cusync
