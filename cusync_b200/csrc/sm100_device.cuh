// Device-side building blocks shared by the sm_100a kernels of this directory: PTX wrappers (mbarrier, TMA,
// tcgen05 / tensor memory), shared-memory and instruction descriptors, the kernel parameter block, the barrier
// block, bounded waits, epilogue math and the store / split-K epilogue helpers.  Everything has internal linkage:
// the file is included by the one translation unit that holds the kernels (gemm_sm100.cu).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace {

constexpr int kBlockM = 128;        // UMMA M
constexpr int kBlockK = 64;         // one 128-byte swizzle row of fp16
constexpr int kUmmaK = 16;
constexpr int kThreads = 384;
constexpr int kEpilogueWarps = 8;    // two per TMEM lane quarter: keeps every scheduler fed during the epilogue
constexpr int kSchedSlots = 8;
constexpr int kEpilogueWarp0 = 4;
constexpr int kLookahead = 32;      // semaphores probed ahead of a consumer wait (a whole row of producer tiles here)
constexpr int kStoreCols = 64;      // columns per TMA store box (128 bytes)
constexpr uint32_t kSmemLimit = 232448;  // 227 KB

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrive on a barrier of any CTA of the cluster, given its shared::cluster address.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders this thread's generic-proxy accesses to GLOBAL memory (a semaphore acquire) before its later async-proxy
// ones (TMA reads of what the semaphore guards).  The form without a state space also covers shared memory, and
// a loader thread with TMA copies into shared memory in flight then waits for those: measured 680 cycles per
// fence beside streaming loads against 4 to 150 for this one.
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
// Element-wise add of a shared-memory box into global memory, done by the TMA unit at the L2.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for tcgen05.mma: 128-byte swizzle, Blackwell
// descriptor version 1.  Offsets are given in bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;   // descriptor version
  d |= 2ull << 61;   // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16: D = f32, A = B = f16, A K-major.
__host__ __device__ constexpr uint32_t make_idesc(int umma_n, bool b_mn_major) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(umma_n >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
}

// ---------------------------------------------------------------------------
// Kernel parameters
// ---------------------------------------------------------------------------
// One work unit of the CTA-pair kernel: K slice `slice` of `nslices` of the pair tile (x = N tile, y = pair row).
// Tiles of the last, partial wave may be cut into more slices than the others (see setup_pair).  A split tile
// owns `nslices` consecutive 256 x 256 fp32 slots of the workspace, starting at slot ws_tile * nslices.
struct PairUnit { uint32_t x, y, slice_of, ws_tile; };   // slice_of = slice | nslices << 16

struct GemmParams {
  int32_t m, n, k;
  int32_t tiles_n, tiles_m, num_tiles;
  int32_t num_k_blocks;
  int32_t epilogue;
  int32_t b_kmajor;            // 1: B given as [n,k] row-major
  int32_t b_chunked3d;         // [k,n] B: all 64-column chunks of a tile come with one 3-D TMA box
  int32_t is_producer, is_consumer;
  uint32_t b_lbo, b_sbo, b_kstep;  // B shared-memory descriptor: leading / stride offsets, bytes per UMMA K step
  void* d; long long ldd;          // output matrix (split-K finalisation stores it without TMA)
  int32_t split_k;                 // K slices per output tile (grid.z of the stage); 1 = none
  int32_t k_blocks_per_split;      // ring stages per slice
  float* splitk_ws;                // fp32 [tiles_m * 128, n] partial sums, all zero between launches
  uint32_t* splitk_arrivals;       // per (m, n) tile: slices that have added their part
  // 3x3 convolution as implicit GEMM (CONV kernels): NHWC input [conv_n, conv_h, conv_w, conv_c]; an M tile
  // is conv_rows whole image rows (conv_rows * conv_w <= 128 output pixels); K walks channel chunks of 64
  // outermost and the nine filter taps innermost.
  int32_t conv_n, conv_h, conv_w, conv_c, conv_rows, conv_tiles_per_image;
  const PairUnit* pair_order;      // CTA-pair kernel: schedule over work units (256-row pair tile x K slice)
  int32_t num_pairs;
  unsigned long long* trace;       // optional per-tile timeline: 4 words per ticket (see cusync_gemm_plan_set_trace)
  uint32_t trace_capacity;
  // B operand produced by an earlier stage (CTA-pair kernel): rows [128 r, 128 r + 128) of the B matrix as given
  // (n rows of [n,k], k rows of [k,n]) are complete when b_sems[b_sem_first + r * b_sem_stride] has reached
  // iter * b_sem_value.  Null: B holds weights and is never waited for.
  const uint32_t* b_sems;
  uint32_t b_sem_first, b_sem_stride, b_sem_value;
  cusync_stage_view_t stage;   // by-value copy, like params_.custage in the reference
};

template <int BN, bool DUAL>
struct Cfg {
  static constexpr int kNumB = DUAL ? 2 : 1;
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kNumB * kBBytes;
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;   // one 32-row x 128-byte buffer per epilogue warp
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kStages =
      ((int)kSmemLimit - 1024 /*alignment slack*/ - kStagingBytes - kBarrierBytes) / kStageBytes > 8
          ? 8
          : ((int)kSmemLimit - 1024 - kStagingBytes - kBarrierBytes) / kStageBytes;
  static constexpr int kAccCols = BN * kNumB;               // fp32 columns per accumulator buffer
  // two accumulator buffers, rounded up to a power of two (tcgen05.alloc's granularity)
  static constexpr int kTmemCols = 2 * kAccCols <= 32 ? 32 : 2 * kAccCols <= 64 ? 64 : 2 * kAccCols <= 128 ? 128
                                   : 2 * kAccCols <= 256 ? 256 : 512;
  static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarrierBytes;
  static_assert(kTmemCols <= 512, "accumulators exceed tensor memory");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns must be a power of two");
  static_assert(kSmemBytes <= kSmemLimit, "shared memory over budget");
  static_assert(kStages >= 3, "pipeline too shallow");
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sched_full[kSchedSlots];
  uint64_t sched_empty[kSchedSlots];
  uint64_t drain;
  uint64_t post;                        // epilogue warps -> the posting thread
  uint64_t post_slot[kSchedSlots];      // slab kernel: the same, one barrier per schedule slot
  uint64_t splitk_counted;              // posting thread -> epilogue warps: arrival counted, `splitk_last` valid
  uint64_t splitk_done;                 // epilogue warps -> posting thread: finalisation stored
  uint32_t splitk_last;
  uint32_t pad0;
  int32_t sched_tile[kSchedSlots][8];   // {n tile, m tile, valid, ticket, k slice, k slices of the tile, -, -}
  unsigned long long sched_time[kSchedSlots];   // globaltimer at the ticket draw (tracing only)
  uint32_t tmem_base;
  volatile uint32_t abort;
};
static_assert(sizeof(Barriers) <= 1024, "barrier block too large");

struct WaitCtx {
  volatile uint32_t* abort;
  uint32_t* status;
  uint64_t timeout_ns;
};

// Bounded mbarrier wait.  Returns false when the block is aborting or the
// bound expired (then it raises the abort flag itself).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = cusync::globalTimerNs();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 31u) == 0u) {
      if (*ctx.abort) return false;
      if (cusync::globalTimerNs() - t0 > ctx.timeout_ns) {
        *ctx.abort = 1u;
        cusync::recordTimeout(ctx.status, 2u, blockIdx.x, threadIdx.x, parity, smem_u32(bar), 0u, 0u);
        return false;
      }
    }
  }
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Epilogue of one warp for one tile: its 32 accumulator rows (TMEM lanes of `t_row`), every second
// 64-column chunk starting at `half`: tcgen05.ld -> fp32 epilogue math -> fp16 -> swizzled staging
// buffer -> TMA store.  `row0` is the matrix row of the warp's first lane.
template <int BN, bool DUAL>
__device__ __forceinline__ void epilogue_store_rows(const GemmParams& p, const CUtensorMap* tmD, uint8_t* buf,
                                                    uint32_t t_row, int n_off, int row0, int half, int lane) {
  const bool rows_in = row0 < p.m;                      // else this warp's 32 rows are all padding
#pragma unroll 1
  for (int c = half; c < BN / kStoreCols && rows_in; c += 2) {
    if (n_off + c * kStoreCols >= p.n) break;           // chunk entirely past the matrix edge
    // The store that last read this warp's buffer must be done reading it.
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
    uint32_t packed[32];
    if (!DUAL) {
      uint32_t v[64];
      tmem_ld_32x32b_x32(t_row + c * 64, v);
      tmem_ld_32x32b_x32(t_row + c * 64 + 32, v + 32);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j++) {
        float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
        if (p.epilogue == CUSYNC_EPILOGUE_GELU_ERF) { x0 = gelu_erf(x0); x1 = gelu_erf(x1); }
        else if (p.epilogue == CUSYNC_EPILOGUE_RELU) { x0 = fmaxf(x0, 0.0f); x1 = fmaxf(x1, 0.0f); }
        packed[j] = pack_half2(x0, x1);
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        uint32_t a[32], b[32];
        tmem_ld_32x32b_x32(t_row + c * 64 + h * 32, a);
        tmem_ld_32x32b_x32(t_row + BN + c * 64 + h * 32, b);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j++) {
          float g0 = silu(__uint_as_float(a[2 * j])) * __uint_as_float(b[2 * j]);
          float g1 = silu(__uint_as_float(a[2 * j + 1])) * __uint_as_float(b[2 * j + 1]);
          packed[h * 16 + j] = pack_half2(g0, g1);
        }
      }
    }
    // Row `lane` of the 32 x 64 chunk, 16-byte pieces XOR-swizzled by row so
    // the layout is the one a 128-byte-swizzle tensor map expects.
    uint8_t* row = buf + lane * 128;
#pragma unroll
    for (int q = 0; q < 8; q++) {
      uint4 val = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      *reinterpret_cast<uint4*>(row + ((q ^ (lane & 7)) << 4)) = val;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmD, buf, n_off + c * kStoreCols, row0);
      tma_store_commit();
    }
  }
}


// Split-K, phase 1: one warp adds its 32 accumulator rows (every second 64-column span from `half`, in two
// 32-column boxes) into the fp32 workspace: tcgen05.ld -> swizzled staging buffer -> TMA reduce-add.  The
// workspace map covers exactly m rows and n columns, so padding rows and columns are clipped by the TMA.
template <int BN>
__device__ __forceinline__ void splitk_accumulate_rows(const GemmParams& p, const CUtensorMap* tmWS, uint8_t* buf,
                                                       uint32_t t_row, int n_off, int row0, int half, int lane) {
  if (row0 >= p.m) return;
#pragma unroll 1
  for (int c = half; c < BN / kStoreCols; c += 2) {
#pragma unroll 1
    for (int h = 0; h < 2; h++) {
      const int col0 = n_off + c * kStoreCols + h * 32;
      if (col0 >= p.n) return;
      if (lane == 0) tma_store_wait_read<0>();     // the previous box has left this warp's staging buffer
      __syncwarp();
      uint32_t v[32];
      tmem_ld_32x32b_x32(t_row + c * 64 + h * 32, v);
      tmem_ld_wait();
      uint8_t* row = buf + lane * 128;             // 32 fp32 = 128 bytes per row, 16-byte pieces XOR-swizzled
#pragma unroll
      for (int q = 0; q < 8; q++)
        *reinterpret_cast<uint4*>(row + ((q ^ (lane & 7)) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_reduce_add_2d(tmWS, buf, col0, row0);
        tma_store_commit();
      }
    }
  }
}

// Split-K, phase 2 (only in the block that brought the last slice): the 256 epilogue threads read the
// summed tile back, zero it for the next launch, apply the epilogue and store fp16.
template <int BN>
__device__ __forceinline__ void splitk_finalize_tile(const GemmParams& p, __half* d, int64_t ldd, int n_off, int m_off,
                                                     int tid) {
  const int rows = p.m - m_off < kBlockM ? p.m - m_off : kBlockM;
  constexpr int kVecPerRow = BN / 4;
  constexpr int kThreadsE = kEpilogueWarps * 32;
  constexpr int kBatch = 8;                 // loads in flight per thread: the reads are L2 round trips
  const int total = rows * kVecPerRow;
  for (int base = tid; base < total; base += kThreadsE * kBatch) {
    float4 x[kBatch];
    float4* src[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
      const int i = base + j * kThreadsE;
      const int r = i / kVecPerRow, c = (i % kVecPerRow) * 4;
      const bool in = i < total && n_off + c < p.n;
      src[j] = in ? reinterpret_cast<float4*>(p.splitk_ws + static_cast<size_t>(m_off + r) * p.n + n_off + c) : nullptr;
      if (in) x[j] = __ldcg(src[j]);
    }
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
      if (src[j] == nullptr) continue;
      const int i = base + j * kThreadsE;
      const int r = i / kVecPerRow, c = (i % kVecPerRow) * 4;
      __stcg(src[j], make_float4(0.f, 0.f, 0.f, 0.f));
      float4 v = x[j];
      if (p.epilogue == CUSYNC_EPILOGUE_GELU_ERF) { v.x = gelu_erf(v.x); v.y = gelu_erf(v.y); v.z = gelu_erf(v.z); v.w = gelu_erf(v.w); }
      else if (p.epilogue == CUSYNC_EPILOGUE_RELU) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
      *reinterpret_cast<uint2*>(d + static_cast<size_t>(m_off + r) * ldd + n_off + c) =
          make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
    }
  }
}

// CTA-pair kernel, split tiles.  Every K slice of a split tile owns a 256 x 256 fp32 slot of the workspace
// (first the leader CTA's 128 rows, then the peer's).  Inside a CTA's part the order is the one the epilogue
// warps produce and consume: 32-row x 32-column boxes, box (row quarter, column block) at float4 index
// ((quarter * 8 + block) * 8 + q) * 32 + lane for columns [4q, 4q + 4) of row `lane` of the box, so that both
// the slices' stores and the finaliser's loads are 512 contiguous bytes per warp instruction.
constexpr int kPairBN = 256;                                // tile width of the pair kernel
constexpr int kPairSlotVec4 = 2 * kBlockM * kPairBN / 4;    // float4 per slot

// Phase 1: one warp stores its 32 accumulator rows (every second 64-column span from `half`) straight from
// registers: plain stores that L2 takes at write bandwidth (reduce-adds of all slices into one tile were
// bound by the L2's atomic rate, and staging through shared memory by the per-box round trip).
template <int BN>
__device__ __forceinline__ void pair_store_partial_rows(float4* cta_part, uint32_t t_row, int quarter, int half, int lane) {
#pragma unroll 1
  for (int c = half; c < BN / kStoreCols; c += 2) {
    uint32_t v[64];
    tmem_ld_32x32b_x32(t_row + c * 64, v);
    tmem_ld_32x32b_x32(t_row + c * 64 + 32, v + 32);
    tmem_ld_wait();
    float4* dst = cta_part + ((quarter * 8 + c * 2) * 8) * 32 + lane;
#pragma unroll
    for (int j = 0; j < 16; j++)
      __stcg(dst + j * 32, make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
  }
  __threadfence();     // every lane's stores are ordered before the arrival count that follows
}

// Phase 2 (only in the CTA that counted the last slice): each warp adds up the slices' slots for its own rows
// and column spans, in slice order (so the sum does not depend on which slice came last), then does what the
// unsplit epilogue does: epilogue math -> fp16 -> swizzled staging buffer -> TMA store.
template <int BN>
__device__ __forceinline__ void pair_finalize_partials(const GemmParams& p, const CUtensorMap* tmD, uint8_t* buf,
                                                       const float4* cta_part0, uint32_t nslices, int n_off, int row0,
                                                       int quarter, int half, int lane) {
  const bool rows_in = row0 < p.m;
#pragma unroll 1
  for (int c = half; c < BN / kStoreCols && rows_in; c += 2) {
    if (n_off + c * kStoreCols >= p.n) break;
    float acc[64];
#pragma unroll
    for (int j = 0; j < 64; j++) acc[j] = 0.f;
    const float4* src = cta_part0 + ((quarter * 8 + c * 2) * 8) * 32 + lane;
#pragma unroll 1
    for (uint32_t sl = 0; sl < nslices; sl++, src += kPairSlotVec4) {
      float4 x[16];
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = __ldcg(src + j * 32);
#pragma unroll
      for (int j = 0; j < 16; j++) { acc[4 * j] += x[j].x; acc[4 * j + 1] += x[j].y; acc[4 * j + 2] += x[j].z; acc[4 * j + 3] += x[j].w; }
    }
    if (lane == 0) tma_store_wait_read<0>();     // the store that last read this warp's buffer is done with it
    __syncwarp();
    uint32_t packed[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
      float x0 = acc[2 * j], x1 = acc[2 * j + 1];
      if (p.epilogue == CUSYNC_EPILOGUE_GELU_ERF) { x0 = gelu_erf(x0); x1 = gelu_erf(x1); }
      else if (p.epilogue == CUSYNC_EPILOGUE_RELU) { x0 = fmaxf(x0, 0.0f); x1 = fmaxf(x1, 0.0f); }
      packed[j] = pack_half2(x0, x1);
    }
    uint8_t* row = buf + lane * 128;
#pragma unroll
    for (int q = 0; q < 8; q++)
      *reinterpret_cast<uint4*>(row + ((q ^ (lane & 7)) << 4)) =
          make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmD, buf, n_off + c * kStoreCols, row0);
      tma_store_commit();
    }
  }
  if (lane == 0) tma_store_wait_all();           // the tile is in memory before the caller publishes it
}

// Split-K epilogue of one tile for one epilogue warp; returns false if a bounded wait expired.
// Every slice adds its part; the block that counts the last arrival finalises and publishes the tile
// (the reference posts from the last K slice only, gemm/kernel/cusyncgemm.h:374-392).
template <int BN>
__device__ __forceinline__ bool splitk_epilogue(const GemmParams& p, const CUtensorMap* tmWS, uint8_t* buf,
                                                Barriers* bars, const WaitCtx& ctx, uint32_t t_row,
                                                int n_off, int m_off, int quarter, int half, int ew, int lane,
                                                uint32_t phase, uint32_t split_phase, uint32_t nslices,
                                                uint64_t* tmem_empty_local, uint32_t tmem_empty_cluster,
                                                __half* d, int64_t ldd, bool* is_last,
                                                float4* ws_part0 = nullptr, uint32_t slice = 0,
                                                const CUtensorMap* tmD = nullptr) {
  // ws_part0 (CTA-pair kernel): this CTA's part of the tile's first workspace slot; slice `slice` stores
  // into the slot `slice` slots further on.  Without it the slices reduce-add into one [m, n] tile.
  if (ws_part0) { if (m_off < p.m) pair_store_partial_rows<BN>(ws_part0 + static_cast<size_t>(slice) * kPairSlotVec4, t_row, quarter, half, lane); }
  else splitk_accumulate_rows<BN>(p, tmWS, buf, t_row, n_off, m_off + quarter * 32, half, lane);
  // accumulator buffer is free for the MMA warp again
  tc_fence_before();
  __syncwarp();
  bool lane0_ok = true;
  if (lane == 0) {
    if (tmem_empty_local) mbar_arrive(tmem_empty_local); else mbar_arrive_cluster(tmem_empty_cluster);
    tma_store_wait_all();            // this warp's reduce-adds have been performed ...
    __threadfence();                 // ... and are ordered before the arrival count
    // (a warp that ran ahead must not arrive while the previous tile's phase of `post` is still open)
    if (!mbar_wait(&bars->post, phase ^ 1u, ctx)) lane0_ok = false;
    mbar_arrive(&bars->post);
  }
  bool ok = lane0_ok;
  if (ew == 0 && lane == 0) {
    if (!mbar_wait(&bars->post, phase, ctx)) ok = false;
    else if (m_off >= p.m) bars->splitk_last = 0u;     // a pair's second half past the last row tile
    else {
      const uint32_t tile = static_cast<uint32_t>(m_off / kBlockM) * static_cast<uint32_t>(p.tiles_n) +
                            static_cast<uint32_t>(n_off / BN);
      __threadfence();
      const uint32_t before = atomicAdd(p.splitk_arrivals + tile, 1u);
      const uint32_t last = before == nslices - 1u ? 1u : 0u;
      if (last) { p.splitk_arrivals[tile] = 0u; __threadfence(); }   // re-armed for the next launch
      bars->splitk_last = last;
    }
    mbar_arrive(&bars->splitk_counted);
  }
  if (!mbar_wait(&bars->splitk_counted, split_phase, ctx)) ok = false;
  const bool last = ok && bars->splitk_last != 0u;
  __syncwarp();
  if (last) {
    if (ws_part0) pair_finalize_partials<BN>(p, tmD, buf, ws_part0, nslices, n_off, m_off + quarter * 32, quarter, half, lane);
    else splitk_finalize_tile<BN>(p, d, ldd, n_off, m_off, ew * 32 + lane);
  }
  __syncwarp();
  if (lane == 0) { __threadfence(); mbar_arrive(&bars->splitk_done); }
  *is_last = last;
  return ok;
}

}  // namespace
