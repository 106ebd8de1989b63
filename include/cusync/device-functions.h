// Device-side primitives of the semaphore layer, written for sm_100a:
//  * publish  = red.release.gpu (or st.release.gpu when a semaphore has a
//    single poster) -- gpu scope is enough, both kernels run on one device;
//  * observe  = ld.acquire.gpu in a loop with nanosleep back-off that gives up
//    after a time bound and leaves a record, instead of spinning forever.
// The reference's counterparts are globalVolatileLoad / globalLoad
// (src/include/cusync/device-functions.h:14-32) and the loops in
// cusync_device_defs.h:33-72.
#pragma once

#include <stdint.h>
#include "../cusync_b200.h"
#include "cusync_defines.h"

#if defined(__CUDACC__) || defined(__NVCC__)

namespace cusync {

// Default bound of a device-side spin when the stage does not set one.
static constexpr uint64_t kDefaultSpinTimeoutNs = 2000000000ull;

CUSYNC_DEVICE uint32_t loadAcquire(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

CUSYNC_DEVICE uint32_t loadRelaxed(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Acquire/release fence at device scope.  Cheaper than __threadfence(), which is the sequentially
// consistent fence: enough after relaxed semaphore probes (makes them acquiring) and before a release.
CUSYNC_DEVICE void fenceAcqRel() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

CUSYNC_DEVICE void addRelease(uint32_t* addr, uint32_t value) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" :: "l"(addr), "r"(value) : "memory");
}

CUSYNC_DEVICE void storeRelease(uint32_t* addr, uint32_t value) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(addr), "r"(value) : "memory");
}

// Tells the device that kernels launched behind this one as programmatic dependents (the launch attribute
// "programmatic stream serialization") may start: they do once every block of this grid has said so or has
// exited, which is to say once every block of this grid is resident or done.  That is the guarantee the
// reference's wait kernel gives a consumer (cusync_device_defs.h:78-83, waitKernel), given by the launch
// hardware instead of a polling kernel.  Without such a dependent behind the grid it does nothing.
CUSYNC_DEVICE void allowDependentLaunch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A producer block's last act: counts itself finished (after its posts) in the stage's third "started" word.
CUSYNC_DEVICE void countBlockFinished(uint32_t* started) { addRelease(started + 2, 1u); }

// Whether the producer kernel of this run has finished altogether: its "blocks finished" word has reached the
// count the host computed when it launched the producer (a counter over all runs: wrapped difference).  An
// acquire: when true, everything the producer wrote and posted is visible to this thread.
CUSYNC_DEVICE bool producerFinished(const uint32_t* finished, uint32_t target) {
  return finished != nullptr && static_cast<int32_t>(loadAcquire(finished) - target) >= 0;
}

CUSYNC_DEVICE uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Names kept from the reference for code that calls them directly.
CUSYNC_DEVICE uint32_t globalVolatileLoad(volatile uint32_t* addr) { return loadAcquire((const uint32_t*)addr); }
CUSYNC_DEVICE uint32_t globalLoad(volatile uint32_t* addr) { return loadRelaxed((const uint32_t*)addr); }

// First timeout wins the record; later ones leave it alone.
CUSYNC_DEVICE void recordTimeout(uint32_t* status, uint32_t where, uint32_t tx, uint32_t ty, uint32_t tz,
                                 uint32_t idx, uint32_t seen, uint32_t expected) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0u, (uint32_t)CUSYNC_ERROR_TIMEOUT) == 0u) {
    status[1] = where; status[2] = tx; status[3] = ty; status[4] = tz;
    status[5] = idx; status[6] = seen; status[7] = expected;
    __threadfence();
  }
}

// Bit a block sets in every semaphore of its stage when it gives up (a bounded wait expired), so that nothing
// downstream waits for posts that will not come: a ">= value" comparison is then satisfied, the plain unsigned
// one of spinUntilAtLeast as well as the cyclic one of the driver's stream memory operations
// ((int32_t)(*addr - value) >= 0), as long as counts stay below 2^30.  Work released this way reads unfinished
// data: the host finds CUSYNC_ERROR_TIMEOUT in the stage's status and has to reset the chain's stages.
static constexpr uint32_t kAbortedSemaphoreBit = 0x40000000u;

// Called by all `nthreads` threads of a block on its abort path; `sems` may be null (not a producer).
CUSYNC_DEVICE void releaseWaitersOnAbort(uint32_t* sems, uint32_t count, uint32_t tid, uint32_t nthreads) {
  if (sems == nullptr) return;
  for (uint32_t i = tid; i < count; i += nthreads) atomicOr(sems + i, kAbortedSemaphoreBit);
  __threadfence();
}

// Spin until *sem >= expected.  Returns false (after recording why) when the
// bound expires.  Called by ONE thread; the caller broadcasts the outcome.
CUSYNC_DEVICE bool spinUntilAtLeast(const uint32_t* sem, uint32_t expected, uint64_t timeoutNs,
                                    uint32_t* seenOut) {
  uint32_t v = loadAcquire(sem);
  if (v >= expected) { *seenOut = v; return true; }
  const uint64_t t0 = globalTimerNs();
  const uint64_t bound = timeoutNs ? timeoutNs : kDefaultSpinTimeoutNs;
  uint32_t backoff = 32;
  while (true) {
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
    v = loadAcquire(sem);
    if (v >= expected) { *seenOut = v; return true; }
    if (globalTimerNs() - t0 > bound) { *seenOut = v; return false; }
  }
}

}  // namespace cusync

#endif  // __CUDACC__
