// Sum all-reduce of a row-parallel layer's output that runs BESIDE the GEMM that produces it: the one exchange
// step of a tensor-parallel MLP / attention shard (the reference only ever times this collective on its own,
// src/ml-bench/transformer/allreduce_times.py:11-35, and runs it after the layer).
//
// A small persistent kernel (a handful of blocks on SMs the GEMMs leave free) walks the 128-row tiles of the
// fp16 matrix Y[rows, cols] in order.  For tile t
//   1. a watcher thread waits until THIS rank's producer has published the tile (the RowSync semaphore of the
//      second GEMM, the same bounded ld.acquire spin every CuSync wait uses), then adds 1 to the tile's ready
//      counter on EVERY rank (one multimem.red through the NVSwitch, or one red per peer);
//   2. the worker warps wait until the local ready counter shows that all ranks have published tile t;
//   3. rank r reduces rows [r, r + 1) * tile_rows / world of the tile: with NVLS one multimem.ld_reduce (the
//      switch adds the ranks' copies, fp32 accumulation) and one multimem.st (the switch writes the sum into
//      every rank's copy) per 16 bytes; without it plain peer loads from every rank, an fp32 sum in rank order,
//      and plain peer stores to every rank.
// A final counter handshake makes every rank's stores visible everywhere before any rank's kernel ends.
// No TMA, no bulk copies, no multicast LOADS of the cluster kind: multimem.* and ordinary loads/stores only.
// Every wait is bounded; on expiry the kernel records why, stops reducing and returns.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <new>

#include "common.cuh"

namespace {

constexpr int kMaxWorld = 8;
constexpr int kWorkers = 480;                     // worker threads per block
constexpr int kThreads = kWorkers + 32;           // ... plus one more warp: the watcher (it has work in block 0 only)
constexpr int kWatcherWarp = kWorkers / 32;
constexpr int kFlagHeader = 8;                    // [0] done counter, [1..7] spare; then one ready counter per row tile

struct ArParams {
  int32_t rank, world;
  int32_t rows, cols, tile_rows, num_tiles;
  long long ld;
  __half* bufs[kMaxWorld];
  __half* mc_buf;                  // multicast address of the matrix, or null
  uint32_t* flags[kMaxWorld];
  uint32_t* mc_flags;              // multicast address of the flag words, or null
  const uint32_t* row_sems;        // this rank's producer semaphores, one per row tile; null = rows already complete
  uint32_t sem_target;
  uint32_t epoch;                  // run number, from 1: counters only grow
  uint32_t* status;                // cusync_status_t on the device
  unsigned long long timeout_ns;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f16x8(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// The same two, executed only where `on` holds.  The condition lives inside the statement (a branch over the one
// instruction), so the compiler sees straight-line code with fixed registers.  A guard predicate on the
// instruction itself was not enough: `@p multimem.st` was observed to store with p false.
__device__ __forceinline__ void multimem_ld_reduce_f16x8_if(bool on, const void* mc, uint4& v) {
  // (outputs only: the registers are cleared inside the statement, then loaded where the condition holds)
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 a;\n\tsetp.eq.u32 p, %5, 0;\n\tmov.b64 a, %4;\n\t"   // inputs read before any output is written
      "mov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\tmov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t"
      "@p bra SKIP_LD;\n\t"
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [a];\n\t"
      "SKIP_LD:\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc), "r"(on ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void multimem_st_f16x8_if(bool on, void* mc, const uint4& v) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, %5, 0;\n\t"
      "@p bra SKIP_ST;\n\t"
      "multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};\n\t"
      "SKIP_ST:\n\t}"
      ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(on ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_v4(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Bounded spin until *p >= expected (system scope).  Returns false when the bound expired or the block aborts.
__device__ __forceinline__ bool spin_sys(const uint32_t* p, uint32_t expected, unsigned long long timeout_ns,
                                         volatile uint32_t* abort, uint32_t* seen) {
  uint32_t v = ld_acquire_sys(p);
  if (v >= expected) { *seen = v; return true; }
  const unsigned long long t0 = cusync::globalTimerNs();
  uint32_t backoff = 64;
  while (true) {
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
    v = ld_acquire_sys(p);
    if (v >= expected) { *seen = v; return true; }
    if (*abort || cusync::globalTimerNs() - t0 > timeout_ns) { *seen = v; return false; }
  }
}

__device__ __forceinline__ void add8(float (&acc)[8], uint4 v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 f = __half22float2(h[i]);
    acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
  }
}

// In-switch sum of `vecs` 16-byte pieces starting at the multicast address `base`, written back to every rank.
// Rounds of one chunk of kUnroll * kWorkers pieces per block; what is left after the last full round is shared
// out equally among the blocks and done in one more pass.  Inside a chunk a thread's pieces are kWorkers pieces
// apart, a compile-time distance, so that one base register serves all of its kUnroll loads in flight.
constexpr int kUnroll = 24;
constexpr uint32_t kChunkVecs = kUnroll * kWorkers;
__device__ __forceinline__ void multicast_reduce_span(__half* base, uint32_t vecs, uint32_t block, uint32_t blocks,
                                                      uint32_t tid) {
  const uint32_t full_rounds = vecs / (blocks * kChunkVecs);
  for (uint32_t r = 0; r < full_rounds; r++) {
    __half* const p0 = base + (static_cast<size_t>(r * blocks + block) * kChunkVecs + tid) * 8;
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) v[u] = multimem_ld_reduce_f16x8(p0 + static_cast<size_t>(u) * kWorkers * 8);
#pragma unroll
    for (int u = 0; u < kUnroll; u++) multimem_st_f16x8(p0 + static_cast<size_t>(u) * kWorkers * 8, v[u]);
  }
  const uint32_t rest0 = full_rounds * blocks * kChunkVecs;
  if (rest0 == vecs) return;
  // the rest (fewer than `blocks` chunks): an equal share per block, at most one chunk, whole groups of kWorkers
  const uint32_t share = ((vecs - rest0 + blocks - 1) / blocks + kWorkers - 1) / kWorkers * kWorkers;
  const uint32_t begin = rest0 + block * share;
  const uint32_t end = begin + share < vecs ? begin + share : vecs;
  if (begin >= end) return;
  __half* const p0 = base + (static_cast<size_t>(begin) + tid) * 8;
  const uint32_t mine = begin + tid < end ? (end - begin - tid + kWorkers - 1) / kWorkers : 0u;   // this thread's pieces
  // (the conditions are inside the asm statements: for the compiler this is straight-line code with fixed
  // registers, which C++ branches around the individual pieces were not)
  uint4 v[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; u++) {
    multimem_ld_reduce_f16x8_if(static_cast<uint32_t>(u) < mine, p0 + static_cast<size_t>(u) * kWorkers * 8, v[u]);
  }
#pragma unroll
  for (int u = 0; u < kUnroll; u++)
    multimem_st_f16x8_if(static_cast<uint32_t>(u) < mine, p0 + static_cast<size_t>(u) * kWorkers * 8, v[u]);
}

template <bool kMulticast>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) cusync_allreduce_rows_kernel(const ArParams p) {
  __shared__ volatile uint32_t s_abort;
  if (threadIdx.x == 0) s_abort = 0u;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* const my_flags = p.flags[p.rank];

  if (blockIdx.x == 0 && warp == kWatcherWarp) {
    // ---- watcher: publish this rank's finished row tiles to every rank -------------------------------
    for (int t = lane; t < p.num_tiles; t += 32) {
      if (p.row_sems) {
        uint32_t seen = 0;
        if (!cusync::spinUntilAtLeast(p.row_sems + t, p.sem_target, p.timeout_ns, &seen)) {
          cusync::recordTimeout(p.status, 1u, static_cast<uint32_t>(t) * p.tile_rows, 0u, 0u, static_cast<uint32_t>(t),
                                seen, p.sem_target);
          s_abort = 1u;
          continue;       // not published: the other ranks' bounded waits run out as well
        }
      }
      fence_sys();        // the producer's stores (acquired at gpu scope) before the system-scope signal
      if (kMulticast) multimem_red_add_release_sys(p.mc_flags + kFlagHeader + t, 1u);
      else
        for (int w = 0; w < p.world; w++) red_add_release_sys(p.flags[(p.rank + w) % p.world] + kFlagHeader + t, 1u);
    }
    return;
  }
  if (warp == kWatcherWarp) return;      // the extra warp of the other blocks has nothing to do

  // ---- workers ---------------------------------------------------------------------------------------
  const int vec_per_row = p.cols / 8;
  const uint32_t block_workers = kWorkers;
  const uint32_t worker = blockIdx.x * kWorkers + threadIdx.x;
  const uint32_t num_workers = gridDim.x * kWorkers;
  const bool contiguous = p.ld == p.cols;
  bool ok = true;
  for (int t = 0; t < p.num_tiles && ok; t++) {
    // all ranks have published tile t
    int warp_ok = 1;
    if (lane == 0) {
      uint32_t seen = 0;
      if (!spin_sys(my_flags + kFlagHeader + t, p.epoch * static_cast<uint32_t>(p.world), p.timeout_ns, &s_abort, &seen)) {
        cusync::recordTimeout(p.status, 2u, static_cast<uint32_t>(t) * p.tile_rows, 0u, 0u, static_cast<uint32_t>(t), seen,
                              p.epoch * static_cast<uint32_t>(p.world));
        s_abort = 1u;
        warp_ok = 0;
      }
    }
    warp_ok = __shfl_sync(0xffffffffu, warp_ok, 0);
    __syncwarp();         // lane 0's acquire is ordered before the other lanes' loads of the tile
    if (!warp_ok) { ok = false; break; }
    // this rank's share of the tile: a contiguous range of its rows
    const int row0 = t * p.tile_rows;
    const int rows_in = p.rows - row0 < p.tile_rows ? p.rows - row0 : p.tile_rows;
    const int r_begin = row0 + static_cast<int>(static_cast<long long>(rows_in) * p.rank / p.world);
    const int r_end = row0 + static_cast<int>(static_cast<long long>(rows_in) * (p.rank + 1) / p.world);
    const uint32_t vecs = static_cast<uint32_t>(r_end - r_begin) * static_cast<uint32_t>(vec_per_row);
    if (kMulticast) {
      // Latency-bound: a multimem.ld_reduce is a round trip through the switch of a few microseconds, so every
      // thread of the 512 keeps 24 of them in flight (192 KB per block: most of the register file) before it
      // turns to the stores.  A matrix with padded rows is walked row by row.
      __half* const slice = p.mc_buf + static_cast<size_t>(r_begin) * p.ld;
      const int spans = contiguous ? 1 : r_end - r_begin;
      const uint32_t span_vecs = contiguous ? vecs : static_cast<uint32_t>(vec_per_row);
      for (int r = 0; r < spans; r++)
        multicast_reduce_span(slice + static_cast<size_t>(r) * p.ld, span_vecs, blockIdx.x, gridDim.x, threadIdx.x);
    } else {
      for (uint32_t i = worker; i < vecs; i += num_workers) {
        const size_t off = static_cast<size_t>(r_begin + i / vec_per_row) * p.ld + static_cast<size_t>(i % vec_per_row) * 8;
        uint4 in[kMaxWorld];
#pragma unroll
        for (int w = 0; w < kMaxWorld; w++)
          if (w < p.world) in[w] = ld_relaxed_sys_v4(p.bufs[w] + off);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < kMaxWorld; w++)
          if (w < p.world) add8(acc, in[w]);               // rank order: the same sum on every rank and run
        uint4 out;
        __half2* h = reinterpret_cast<__half2*>(&out);
#pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
#pragma unroll
        for (int w = 0; w < kMaxWorld; w++)
          if (w < p.world) st_relaxed_sys_v4(p.bufs[(p.rank + w) % p.world] + off, out);
      }
    }
  }
  // ---- every rank's stores are in place before any rank's kernel ends -----------------------------------
  fence_sys();
  asm volatile("bar.sync 1, %0;" ::"r"(block_workers) : "memory");
  if (threadIdx.x == 0) {
    if (kMulticast) multimem_red_add_release_sys(p.mc_flags, 1u);
    else
      for (int w = 0; w < p.world; w++) red_add_release_sys(p.flags[(p.rank + w) % p.world], 1u);
    const uint32_t expected = p.epoch * static_cast<uint32_t>(p.world) * gridDim.x;
    uint32_t seen = 0;
    if (!s_abort && !spin_sys(my_flags, expected, p.timeout_ns, &s_abort, &seen))
      cusync::recordTimeout(p.status, 3u, 0u, 0u, 0u, 0u, seen, expected);
  }
}

}  // namespace

struct cusync_allreduce_plan {
  ArParams params;
  int num_ctas;
  uint32_t* status;      // device
};

extern "C" {

uint32_t cusync_allreduce_flag_words(int32_t rows, int32_t tile_rows) {
  if (rows <= 0 || tile_rows <= 0) return 0;
  return static_cast<uint32_t>(kFlagHeader + (rows + tile_rows - 1) / tile_rows);
}

int cusync_allreduce_plan_create(cusync_allreduce_plan_t** out, const cusync_allreduce_desc_t* desc) {
  if (!out || !desc) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_allreduce_desc_t& d = *desc;
  if (d.world < 1 || d.world > kMaxWorld || d.rank < 0 || d.rank >= d.world) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.rows <= 0 || d.cols <= 0 || !d.buffers || !d.flags) return CUSYNC_ERROR_INVALID_ARGUMENT;
  // 16-byte pieces: whole groups of 8 halves per row, aligned rows
  if (d.cols % 8 || d.ld % 8 || d.ld < d.cols) return CUSYNC_ERROR_UNSUPPORTED;
  const int tile_rows = d.tile_rows > 0 ? d.tile_rows : 128;
  if (d.num_ctas < 0 || d.num_ctas % 2) return CUSYNC_ERROR_INVALID_ARGUMENT;      // whole block pairs (one TPC each)
  cusync_allreduce_plan* pl = new (std::nothrow) cusync_allreduce_plan();
  if (!pl) return CUSYNC_ERROR_CUDA;
  std::memset(pl, 0, sizeof(*pl));
  ArParams& p = pl->params;
  p.rank = d.rank; p.world = d.world;
  p.rows = d.rows; p.cols = d.cols; p.ld = d.ld; p.tile_rows = tile_rows;
  p.num_tiles = (d.rows + tile_rows - 1) / tile_rows;
  for (int w = 0; w < d.world; w++) {
    if (!d.buffers[w] || !d.flags[w] || (reinterpret_cast<uintptr_t>(d.buffers[w]) & 15u)) { delete pl; return CUSYNC_ERROR_INVALID_ARGUMENT; }
    p.bufs[w] = static_cast<__half*>(d.buffers[w]);
    p.flags[w] = d.flags[w];
  }
  p.mc_buf = static_cast<__half*>(d.multicast_buffer);
  p.mc_flags = d.multicast_flags;
  if ((p.mc_buf == nullptr) != (p.mc_flags == nullptr)) { delete pl; return CUSYNC_ERROR_INVALID_ARGUMENT; }
  p.timeout_ns = d.timeout_ns ? d.timeout_ns : cusync::kDefaultSpinTimeoutNs;
  p.epoch = 1;
  pl->num_ctas = d.num_ctas ? d.num_ctas : 4;
  if (cudaMalloc(&pl->status, 8 * sizeof(uint32_t)) != cudaSuccess || cudaMemset(pl->status, 0, 8 * sizeof(uint32_t)) != cudaSuccess) {
    (void)cudaGetLastError();
    cudaFree(pl->status);
    delete pl;
    return CUSYNC_ERROR_CUDA;
  }
  p.status = pl->status;
  // Load the kernel now: its launches come while other persistent kernels may be running (see stage.cu).
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, cusync_allreduce_rows_kernel<true>) != cudaSuccess) (void)cudaGetLastError();
  if (cudaFuncGetAttributes(&attr, cusync_allreduce_rows_kernel<false>) != cudaSuccess) (void)cudaGetLastError();
  *out = pl;
  return CUSYNC_SUCCESS;
}

int cusync_allreduce_plan_destroy(cusync_allreduce_plan_t* pl) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  cudaFree(pl->status);
  delete pl;
  return CUSYNC_SUCCESS;
}

int cusync_allreduce_run(cusync_allreduce_plan_t* pl, const uint32_t* row_semaphores, uint32_t value, cusync_stream_t stream) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  ArParams p = pl->params;
  p.row_sems = row_semaphores;
  p.sem_target = value;
  if (p.mc_buf) cusync_allreduce_rows_kernel<true><<<pl->num_ctas, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  else          cusync_allreduce_rows_kernel<false><<<pl->num_ctas, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  if (cudaGetLastError() != cudaSuccess) return CUSYNC_ERROR_CUDA;
  pl->params.epoch += 1;         // counted only when the launch went out: every rank must run equally often
  return CUSYNC_SUCCESS;
}

int cusync_allreduce_read_status(const cusync_allreduce_plan_t* pl, cusync_status_t* out) {
  if (!pl || !out) return CUSYNC_ERROR_NOT_INITIALIZED;
  return cudaMemcpy(out, pl->status, sizeof(cusync_status_t), cudaMemcpyDeviceToHost) == cudaSuccess ? CUSYNC_SUCCESS
                                                                                                      : CUSYNC_ERROR_CUDA;
}

uint32_t cusync_allreduce_plan_num_ctas(const cusync_allreduce_plan_t* pl) { return pl ? static_cast<uint32_t>(pl->num_ctas) : 0; }

}  // extern "C"
