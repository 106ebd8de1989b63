// Tile-synchronised GEMM for sm_100a: D = epilogue(A * B), fp16 operands, fp32
// accumulation in tensor memory, fp16 output.
//
// Replaces the reference's CuSync-augmented CUTLASS 2.x GEMM
// (gemm/kernel/cusyncgemm.h:207-399 and the main loops in
// gemm/threadblock/cusyncmma_multistage.h:943-1200, which are mma.sync +
// cp.async) with a persistent, warp-specialised kernel:
//
//   warp 0  lane 0   tile scheduler + TMA loader.  Draws a ticket from the
//                    stage's counter, looks the tile up in the schedule buffer
//                    (CuStage::tile, cusync_device_defs.h:77-103), and streams
//                    K-blocks of A and B into a shared-memory ring.  The
//                    CONSUMER WAIT sits here: before the TMA load of an A
//                    K-block whose producer tile is not known to be finished,
//                    it evaluates the input policy and spins on the semaphore
//                    (CuStage::wait, cusync_device_defs.h:33-50).  B (weights)
//                    is issued before the wait, which is the reference's
//                    ReorderTileLoads optimisation (cusyncmma_multistage.h:1076-1084).
//   warp 1  lane 0   issues tcgen05.mma (128 x BN x 16, kind::f16) into one of
//                    two TMEM accumulator buffers.
//   warp 2           allocates / frees tensor memory.
//   warps 4-11       epilogue: tcgen05.ld -> fp32 math (GELU / ReLU / SiLU*mul)
//                    -> fp16 -> swizzled shared staging -> TMA store.  After
//                    the stores have fully completed, ONE thread publishes the
//                    tile with red.release.gpu (CuStage::post,
//                    cusync_device_defs.h:55-72).
//
// No TMA multicast is used anywhere.  Every wait in the kernel is bounded: on
// expiry the waiter records why in the stage's status words, raises a
// block-wide abort flag, and the block drains its copies, frees its tensor
// memory and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"

namespace {

constexpr int kBlockM = 128;        // UMMA M
constexpr int kBlockK = 64;         // one 128-byte swizzle row of fp16
constexpr int kUmmaK = 16;
constexpr int kThreads = 384;
constexpr int kEpilogueWarps = 8;    // two per TMEM lane quarter: keeps every scheduler fed during the epilogue
constexpr int kSchedSlots = 8;
constexpr int kEpilogueWarp0 = 4;
constexpr int kLookahead = 8;       // semaphores probed ahead of a consumer wait
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
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
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
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
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

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int BN, bool DUAL, bool CONV = false>
__global__ void __launch_bounds__(kThreads, 1)
cusync_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmD,
                   const __grid_constant__ CUtensorMap tmWS, const GemmParams p) {
  using C = Cfg<BN, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle patterns repeat every 1024 bytes: align the ring to that.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(staging + C::kStagingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const cusync_stage_view_t& st = p.stage;
  WaitCtx ctx{&bars->abort, st.status, 2 * st.timeout_ns + 1000000000ull};

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; i++) { mbar_init(&bars->tmem_full[i], 1); mbar_init(&bars->tmem_empty[i], kEpilogueWarps); }
    for (int i = 0; i < kSchedSlots; i++) { mbar_init(&bars->sched_full[i], 1); mbar_init(&bars->sched_empty[i], 1 + kEpilogueWarps); }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->post, kEpilogueWarps);
    mbar_init(&bars->splitk_counted, 1);
    mbar_init(&bars->splitk_done, kEpilogueWarps);
    bars->abort = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    // "Kernel started" words the wait kernel polls: [0] follows the reference
    // (block 0 stores iter, cusync_device_defs.h:78-83); [1] counts resident blocks.
    if (p.is_producer) {
      if (blockIdx.x == 0) cusync::storeRelease(st.started, st.iter);
      cusync::addRelease(st.started + 1, 1u);
    }
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA); prefetch_tensormap(&tmB); prefetch_tensormap(&tmD);
    if (DUAL) prefetch_tensormap(&tmB2);
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // =====================================================================
    // Scheduler + TMA loader
    // =====================================================================
    if (lane == 0) {
      uint32_t fills = 0, sched_it = 0;
      bool ok = true;
      const uint32_t total_draws = static_cast<uint32_t>(p.num_tiles) + gridDim.x;
      const uint32_t wait_target = p.is_consumer ? st.iter * cusync::eval::waitValue(st.in_policy) : 0u;
      // Distance along K between two sync points of the input policy (0: it syncs once per tile).
      uint32_t sync_stride = 0;
      if (p.is_consumer) {
        const int kind = st.in_policy.kind;
        if (kind == CUSYNC_POLICY_TILESYNC || kind == CUSYNC_POLICY_STRIDEDTILESYNC) sync_stride = st.in_policy.tile_n;
        else if (kind == CUSYNC_POLICY_CONV2DTILESYNC) sync_stride = st.in_policy.tile_n * st.in_policy.p0;
      }
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
        const uint32_t ticket = atomicAdd(st.tile_counter, 1u);
        // Every block draws exactly one ticket past the end, so the draw
        // numbered total_draws-1 is the launch's last: it re-arms the counter
        // (the reference resets on the last tile, cusync_device_defs.h:87-90).
        if (ticket == total_draws - 1u) atomicExch(st.tile_counter, 0u);
        const bool valid = ticket < static_cast<uint32_t>(p.num_tiles);
        cusync_dim3_t t = {0, 0, 0};
        if (valid) t = st.tile_order[ticket];
        bars->sched_tile[slot][0] = static_cast<int32_t>(t.x);
        bars->sched_tile[slot][1] = static_cast<int32_t>(t.y);
        bars->sched_tile[slot][2] = valid ? 1 : 0;
        bars->sched_tile[slot][3] = static_cast<int32_t>(ticket);
        bars->sched_tile[slot][4] = static_cast<int32_t>(t.z);
        if (p.trace) bars->sched_time[slot] = cusync::globalTimerNs();
        mbar_arrive(&bars->sched_full[slot]);
        sched_it++;
        if (!valid) break;

        const int n_off = static_cast<int>(t.x) * BN;
        // Row offset of the tile: 128 matrix rows, or for a convolution conv_rows image rows of output pixels.
        const int m_off = CONV ? static_cast<int>(t.y) * p.conv_rows * p.conv_w : static_cast<int>(t.y) * kBlockM;
        const int img = CONV ? static_cast<int>(t.y) / p.conv_tiles_per_image : 0;
        const int h0 = CONV ? (static_cast<int>(t.y) % p.conv_tiles_per_image) * p.conv_rows : 0;
        // K slice of this work unit (the whole K walk without split-K)
        const int kb_begin = static_cast<int>(t.z) * p.k_blocks_per_split;
        const int kb_end = kb_begin + p.k_blocks_per_split < p.num_k_blocks ? kb_begin + p.k_blocks_per_split
                                                                           : p.num_k_blocks;
        uint32_t ready_end = 0;   // K offset below which this tile's producer tiles are known finished
        long long wait_empty = 0;
        for (int kb = kb_begin; kb < kb_end; kb++) {
          const uint32_t s = fills % C::kStages, ph = (fills / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u, ctx)) { ok = false; break; }
          if (p.trace) wait_empty += clock64() - c0;
          uint8_t* sa = ring + s * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          // A convolution's A box holds conv_rows * conv_w pixel rows of 128 bytes, not the full 128.
          mbar_expect_tx(&bars->full[s], CONV ? static_cast<uint32_t>(p.conv_rows * p.conv_w * 128 + C::kNumB * C::kBBytes)
                                              : static_cast<uint32_t>(C::kStageBytes));
          const int k_off = kb * kBlockK;
          // Convolution: K block kb is channel chunk kb / 9, filter tap (r, s) = kb % 9; the filter is
          // [k_out][r][s][c], so its K offset is tap * C + chunk * 64.
          const int tap = CONV ? kb % 9 : 0, chunk = CONV ? kb / 9 : 0;
          // Weights first: they never depend on the producer kernel.
          if (CONV) {
            tma_load_2d(sb, &tmB, &bars->full[s], tap * p.conv_c + chunk * kBlockK, n_off);
          } else if (p.b_kmajor) {
            tma_load_2d(sb, &tmB, &bars->full[s], k_off, n_off);
            if (DUAL) tma_load_2d(sb + C::kBBytes, &tmB2, &bars->full[s], k_off, n_off);
          } else if (p.b_chunked3d) {
            // one box {64 columns, kBlockK rows, BN/64 chunks}: a TMA instruction costs the issuing
            // thread over a hundred cycles, so fewer and larger boxes keep the loader ahead of the MMAs
            tma_load_3d(sb, &tmB, &bars->full[s], 0, k_off, n_off / 64);
            if (DUAL) tma_load_3d(sb + C::kBBytes, &tmB2, &bars->full[s], 0, k_off, n_off / 64);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; j++)
              tma_load_2d(sb + j * (kBlockK * 128), &tmB, &bars->full[s], n_off + j * 64, k_off);
            if (DUAL) {
#pragma unroll
              for (int j = 0; j < BN / 64; j++)
                tma_load_2d(sb + C::kBBytes + j * (kBlockK * 128), &tmB2, &bars->full[s], n_off + j * 64, k_off);
            }
          }
          // Consumer wait, at the load of the dependent A K-block.
          if (p.is_consumer) {
            const uint32_t tz = kb == kb_begin ? 1u : 0u;
            if (static_cast<uint32_t>(k_off) >= ready_end &&
                cusync::eval::isSync(st.in_policy, static_cast<uint32_t>(k_off), tz)) {
              const uint32_t idx = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(k_off), st.prod_grid.x,
                                                           st.prod_grid.y);
              uint32_t seen = 0;
              // Convolution: the tile's own semaphore and those of its two halo neighbours are probed
              // together first (one memory round trip instead of three); only what is still missing is
              // then waited for.
              bool conv_all_ready = false;
              if (CONV) {
                const int tin = static_cast<int>(t.y) % p.conv_tiles_per_image;
                const int span = p.conv_rows * p.conv_w;
                const uint32_t i_up = tin > 0 ? cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off - span),
                                                    static_cast<uint32_t>(k_off), st.prod_grid.x, st.prod_grid.y) : idx;
                const uint32_t i_dn = tin + 1 < p.conv_tiles_per_image
                                          ? cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off + span),
                                                static_cast<uint32_t>(k_off), st.prod_grid.x, st.prod_grid.y) : idx;
                const uint32_t v0 = cusync::loadRelaxed(st.sems_wait + idx);
                const uint32_t v1 = cusync::loadRelaxed(st.sems_wait + i_up);
                const uint32_t v2 = cusync::loadRelaxed(st.sems_wait + i_dn);
                conv_all_ready = v0 >= wait_target && v1 >= wait_target && v2 >= wait_target;
                if (conv_all_ready) __threadfence();
              }
              if (!conv_all_ready &&
                  !cusync::spinUntilAtLeast(st.sems_wait + idx, wait_target, st.timeout_ns, &seen)) {
                bars->abort = 1u;
                cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_off), tz,
                                      idx, seen, wait_target);
                // The stage was armed: give it its A bytes anyway so the
                // barrier completes and the drain below terminates.
                if (CONV) tma_load_4d(sa, &tmA, &bars->full[s], chunk * kBlockK, tap % 3 - 1, h0 + tap / 3 - 1, img);
                else      tma_load_2d(sa, &tmA, &bars->full[s], k_off, m_off);
                fills++;
                ok = false;
                break;
              }
              // Look ahead: probe the semaphores of the next producer tiles along K with independent
              // relaxed loads (one memory round trip for all of them) and remember how far the
              // finished prefix reaches, so later K-blocks skip the wait.  The relaxed loads are
              // made acquiring by the fence that follows.
              if (sync_stride) {
                uint32_t vals[kLookahead];
#pragma unroll
                for (int j = 0; j < kLookahead; j++) {
                  const uint32_t kk = static_cast<uint32_t>(k_off) + (j + 1) * sync_stride;
                  vals[j] = kk < static_cast<uint32_t>(p.k)
                                ? cusync::loadRelaxed(st.sems_wait + cusync::eval::tileIndex(st.in_policy,
                                      static_cast<uint32_t>(m_off), kk, st.prod_grid.x, st.prod_grid.y))
                                : 0u;
                }
                uint32_t ahead = 0;
#pragma unroll
                for (int j = 0; j < kLookahead; j++) {
                  if (ahead == static_cast<uint32_t>(j) && vals[j] >= wait_target) ahead++;
                }
                ready_end = static_cast<uint32_t>(k_off) + (ahead + 1) * sync_stride;
                if (ahead) __threadfence();
              }
              // A 3x3 stencil also reads the image rows just above and below the tile: they belong to
              // the neighbouring producer tiles of the same image, which the reference's policy does
              // not wait for (it relies on tile order); wait for them as well.
              if (CONV && !conv_all_ready) {
                bool halo_ok = true;
                for (int dm = -1; dm <= 1 && halo_ok; dm += 2) {
                  const int nb = static_cast<int>(t.y) % p.conv_tiles_per_image + dm;
                  if (nb < 0 || nb >= p.conv_tiles_per_image) continue;
                  const uint32_t nidx = cusync::eval::tileIndex(
                      st.in_policy, static_cast<uint32_t>(m_off + dm * p.conv_rows * p.conv_w),
                      static_cast<uint32_t>(k_off), st.prod_grid.x, st.prod_grid.y);
                  if (!cusync::spinUntilAtLeast(st.sems_wait + nidx, wait_target, st.timeout_ns, &seen)) {
                    bars->abort = 1u;
                    cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_off), 2u,
                                          nidx, seen, wait_target);
                    halo_ok = false;
                  }
                }
                if (!halo_ok) {
                  tma_load_4d(sa, &tmA, &bars->full[s], chunk * kBlockK, tap % 3 - 1, h0 + tap / 3 - 1, img);
                  fills++;
                  ok = false;
                  break;
                }
              }
              // Order the acquire (generic proxy) before the TMA read (async proxy).
              fence_proxy_async();
            }
          }
          // Convolution: the box {64 channels, W pixels, conv_rows rows, 1 image} shifted by the tap; the
          // TMA zero-fills what falls outside the image, which is the padding.
          if (CONV) tma_load_4d(sa, &tmA, &bars->full[s], chunk * kBlockK, tap % 3 - 1, h0 + tap / 3 - 1, img);
          else      tma_load_2d(sa, &tmA, &bars->full[s], k_off, m_off);
          fills++;
        }
        if (p.trace && ticket < p.trace_capacity) p.trace[8ull * ticket + 5] = static_cast<unsigned long long>(wait_empty);
      }
      if (!ok) {
        // Abort path: wait (bounded) for every copy still in flight before the
        // block's shared memory goes away.
        bars->abort = 1u;
        const uint32_t live = fills < static_cast<uint32_t>(C::kStages) ? fills : static_cast<uint32_t>(C::kStages);
        for (uint32_t j = 0; j < live; j++) {
          const uint32_t f = fills - 1u - j;
          const uint32_t s = f % C::kStages, ph = (f / C::kStages) & 1u;
          const uint64_t t0 = cusync::globalTimerNs();
          while (!mbar_try_wait(&bars->full[s], ph)) {
            if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // =====================================================================
    // MMA issuer
    // =====================================================================
    if (lane == 0) {
      // Dual-B tiles sit back to back in the ring (second operand right after the first, same chunking), so
      // while both fit one instruction they are multiplied as a single 2*BN-wide B: accumulator columns
      // [0, BN) are A*B, [BN, 2BN) are A*B2.
      constexpr bool kFusedDual = DUAL && 2 * BN <= 256;
      const uint32_t idesc = make_idesc(kFusedDual ? 2 * BN : BN, !p.b_kmajor);
      const uint32_t b_lbo = p.b_lbo, b_sbo = p.b_sbo, b_kstep = p.b_kstep;
      uint32_t drains = 0, sched_it = 0, acc_it = 0;
      bool ok = true;
      bool issued = false;
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
        const int valid = bars->sched_tile[slot][2];
        const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
        const int slice = bars->sched_tile[slot][4];
        mbar_arrive(&bars->sched_empty[slot]);
        sched_it++;
        if (!valid) break;
        const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
        const long long t_tile0 = p.trace ? clock64() : 0;
        if (!mbar_wait(&bars->tmem_empty[acc], aph ^ 1u, ctx)) { ok = false; break; }
        tc_fence_after();
        const long long t_acc = p.trace ? clock64() : 0;
        long long wait_full = 0;
        const uint32_t d_tmem = tmem_base + acc * C::kAccCols;
        const int kb_first = slice * p.k_blocks_per_split;
        const int kb_count = kb_first + p.k_blocks_per_split < p.num_k_blocks ? p.k_blocks_per_split
                                                                             : p.num_k_blocks - kb_first;
        for (int kb = 0; kb < kb_count; kb++) {
          const uint32_t s = drains % C::kStages, ph = (drains / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait(&bars->full[s], ph, ctx)) { ok = false; break; }
          if (p.trace) wait_full += clock64() - c0;
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + s * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; kk++) {
            const uint64_t adesc = make_smem_desc(sa + kk * 32, 16u, 1024u);
            const uint64_t bdesc = make_smem_desc(sb + kk * b_kstep, b_lbo, b_sbo);
            const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
            umma_f16(d_tmem, adesc, bdesc, idesc, accumulate);
            if (DUAL && !kFusedDual) {
              const uint64_t b2desc = make_smem_desc(sb + C::kBBytes + kk * b_kstep, b_lbo, b_sbo);
              umma_f16(d_tmem + BN, adesc, b2desc, idesc, accumulate);
            }
          }
          umma_commit(&bars->empty[s]);   // frees the ring slot when these MMAs retire
          issued = true;
          drains++;
        }
        if (!ok) break;
        umma_commit(&bars->tmem_full[acc]);
        if (p.trace && ticket < p.trace_capacity) {
          p.trace[8ull * ticket + 4] = static_cast<unsigned long long>(wait_full);
          p.trace[8ull * ticket + 6] = static_cast<unsigned long long>(clock64() - t_tile0);
          p.trace[8ull * ticket + 7] = static_cast<unsigned long long>(t_acc - t_tile0);
        }
        acc_it++;
      }
      if (!ok && issued) {
        // Let outstanding MMAs retire before tensor memory is released.
        umma_commit(&bars->drain);
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(&bars->drain, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // =====================================================================
    // Epilogue
    // =====================================================================
    const int ew = warp - kEpilogueWarp0;
    const int quarter = ew & 3;                        // == warp % 4: the TMEM lanes this warp may read
    const int half = ew >> 2;                          // which 64-column chunks of the tile it takes
    uint8_t* buf = staging + ew * (32 * 128);
    uint32_t sched_it = 0, acc_it = 0, post_it = 0;
    bool ok = true;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_n = bars->sched_tile[slot][0];
      const int tile_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
      const unsigned long long t_draw = p.trace ? bars->sched_time[slot] : 0ull;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->sched_empty[slot]);
      sched_it++;
      if (!valid) break;
      const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
      if (!mbar_wait(&bars->tmem_full[acc], aph, ctx)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_mma_done = p.trace ? cusync::globalTimerNs() : 0ull;
      const int n_off = tile_n * BN, m_off = CONV ? tile_m * p.conv_rows * p.conv_w : tile_m * kBlockM;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kAccCols;

      if (CONV) {
        // One output pixel per lane: its BN channels are contiguous in NHWC, so each lane stores its own
        // 128-byte pieces directly.  Rows past conv_rows * conv_w are padding of the 128-row MMA.
        const int row = quarter * 32 + lane;
        const bool row_in = row < p.conv_rows * p.conv_w;
#pragma unroll 1
        for (int c = half; c < BN / kStoreCols; c += 2) {
          uint32_t v[64];
          tmem_ld_32x32b_x32(t_row + c * 64, v);
          tmem_ld_32x32b_x32(t_row + c * 64 + 32, v + 32);
          tmem_ld_wait();
          if (row_in) {
            __half* dst = static_cast<__half*>(p.d) + static_cast<size_t>(m_off + row) * p.ldd + n_off + c * 64;
#pragma unroll
            for (int q = 0; q < 8; q++) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; e++) {
                float x0 = __uint_as_float(v[8 * q + 2 * e]), x1 = __uint_as_float(v[8 * q + 2 * e + 1]);
                if (p.epilogue == CUSYNC_EPILOGUE_RELU) { x0 = fmaxf(x0, 0.0f); x1 = fmaxf(x1, 0.0f); }
                w[e] = pack_half2(x0, x1);
              }
              *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
        acc_it++;
        if (p.is_producer) {
          // every lane's stores are ordered before lane 0's fence by the warp barrier above
          if (lane == 0) {
            __threadfence();
            // Epilogue warps run at their own pace: one that is a tile ahead must not arrive on `post`
            // while the previous tile's phase is still open (its arrival would close that phase early).
            if (!mbar_wait(&bars->post, (post_it & 1u) ^ 1u, ctx)) ok = false;
            mbar_arrive(&bars->post);
            if (ew == 0) {
              if (!mbar_wait(&bars->post, post_it & 1u, ctx)) ok = false;
              else {
                const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                             static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
                const uint32_t pv = cusync::eval::postValue(st.out_policy);
                __threadfence();
                if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
                else                                    cusync::addRelease(st.sems_post + idx, pv);
              }
            }
          }
          post_it++;
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
          uint32_t smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          unsigned long long* rec = p.trace + 8ull * ticket;
          rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
          rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
        }
        continue;
      }
      if (!DUAL && p.split_k > 1) {
        // Split-K: add this slice's part; the block that brings the last slice finalises and posts.
        bool last = false;
        ok = splitk_epilogue<BN>(p, &tmWS, buf, bars, ctx, t_row, n_off, m_off, quarter, half, ew, lane, post_it & 1u,
                                 post_it & 1u, static_cast<uint32_t>(p.split_k), &bars->tmem_empty[acc], 0u,
                                 static_cast<__half*>(p.d), p.ldd, &last);
        acc_it++;
        if (ew == 0 && lane == 0) {
          if (!mbar_wait(&bars->splitk_done, post_it & 1u, ctx)) ok = false;
          else if (last && p.is_producer) {
            const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                         static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
            const uint32_t pv = cusync::eval::postValue(st.out_policy);
            __threadfence();
            if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
            else                                    cusync::addRelease(st.sems_post + idx, pv);
          }
        }
        post_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        continue;
      }
      epilogue_store_rows<BN, DUAL>(p, &tmD, buf, t_row, n_off, m_off + quarter * 32, half, lane);
      // Accumulator buffer is free for the MMA warp again.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
      acc_it++;

      if (p.is_producer) {
        // Publish the tile only after every store of it has fully completed:
        // each warp's issuing lane waits for its own bulk stores, then arrives
        // on `post`; the first epilogue warp's lane collects the four arrivals
        // (bounded) and performs the single release.
        if (lane == 0) {
          tma_store_wait_all();
          __threadfence();
          // Epilogue warps run at their own pace: one that is a tile ahead must not arrive on `post`
          // while the previous tile's phase is still open (its arrival would close that phase early).
          if (!mbar_wait(&bars->post, (post_it & 1u) ^ 1u, ctx)) ok = false;
          mbar_arrive(&bars->post);
          if (ew == 0) {
            if (!mbar_wait(&bars->post, post_it & 1u, ctx)) ok = false;
            else {
              const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
              const uint32_t pv = cusync::eval::postValue(st.out_policy);
              __threadfence();
              if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
              else                                    cusync::addRelease(st.sems_post + idx, pv);
            }
          }
        }
        post_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long* rec = p.trace + 8ull * ticket;
        rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
        rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // Teardown (normal and abort paths alike).
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}


// ---------------------------------------------------------------------------
// 3x3 convolution, 64 -> 64 channels: the slab kernel
// ---------------------------------------------------------------------------
// The implicit-GEMM path above fetches one shifted copy of the input rows per filter tap (nine TMA boxes and
// nine barrier round trips per tile) and re-reads the 3x3 filter for every tile.  For the layer the conv chain
// is measured on (C = K = 64, src/ml-bench/volta_conv2d/ resnet sizes) both fit on chip:
//
//   * the whole filter (9 taps x 64 x 64 fp16 = 72 KB) is loaded ONCE per CTA and stays in shared memory;
//   * per tile ONE 4-D TMA box brings the input slab: conv_rows + 2 image rows of W + 2 pixels (the halo is the
//     box's out-of-range part, zero-filled = the padding), 64 channels = one 128-byte swizzle row per pixel;
//   * the MMA's M index runs over the slab's pixels in memory order (padded width W + 2), so tap (r, s) is the
//     same slab read from (r * (W + 2) + s) pixel rows further on: 36 tcgen05.mma per tile, back to back, with a
//     shared-memory descriptor whose start address moves by whole 128-byte rows (the 128-byte swizzle is a
//     function of the shared-memory address, so a start that is not a multiple of 8 rows needs nothing else;
//     the descriptor's base-offset field stays 0 - setting it to the start row's phase gave wrong products).
//     M rows that fall on the two padding columns of a slab row, or past conv_rows rows, are computed and dropped.
//
// Tile shape, stage grid, semaphores and policies are those of the general path: one tile = conv_rows whole image
// rows, waits on its own and the two neighbouring producer tiles, posts once.
//
// The scheduler keeps three tickets in flight: the ticket draw, the schedule look-up and the semaphore probes of
// a tile are three dependent memory round trips (about 2 us), as long as a whole tile's math here, so each is
// issued one tile ahead of the next.  Every CTA therefore draws exactly three tickets past the end.
constexpr int kSlabStages = 4;
constexpr int kSlabBytes = 256 * 128;          // room for 256 pixel rows: the last tap reads up to row 2(W+2)+2+127
constexpr int kSlabFilterBytes = 9 * 64 * 128; // nine taps of [64 n][64 c]
constexpr int kSlabBN = 64;
constexpr uint32_t kSlabSmemBytes = 1024 + kSlabStages * kSlabBytes + kSlabFilterBytes + 1024;
constexpr int kSlabTicketsAhead = 3;
constexpr int kSlabIssuers = 2;                // threads that issue MMAs, alternating tiles

__global__ void __launch_bounds__(kThreads, 1)
cusync_conv3x3_slab_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmF,
                           const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slabs = smem;
  uint8_t* filt = smem + kSlabStages * kSlabBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(filt + kSlabFilterBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const cusync_stage_view_t& st = p.stage;
  WaitCtx ctx{&bars->abort, st.status, 2 * st.timeout_ns + 1000000000ull};
  const int wp = p.conv_w + 2;                         // padded slab width
  uint64_t* filt_full = &bars->splitk_counted;         // (split-K is not used by this kernel)
  // Four accumulators, one per slab stage: tile j of this CTA uses slab j % 4 and accumulator j % 4, and is
  // issued by MMA thread j % 2 (see below).  Their barriers live in the upper half of the ring's arrays.
  uint64_t* acc_full = &bars->full[kSlabStages];
  uint64_t* acc_empty = &bars->empty[kSlabStages];

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlabStages; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < kSlabStages; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpilogueWarps); }
    for (int i = 0; i < kSchedSlots; i++) { mbar_init(&bars->sched_full[i], 1); mbar_init(&bars->sched_empty[i], kSlabIssuers + kEpilogueWarps + 1); }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->splitk_done, 1);     // the second MMA thread's drain barrier
    for (int i = 0; i < kSchedSlots; i++) mbar_init(&bars->post_slot[i], kEpilogueWarps);
    mbar_init(filt_full, 1);
    bars->abort = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    if (p.is_producer) {
      if (blockIdx.x == 0) cusync::storeRelease(st.started, st.iter);
      cusync::addRelease(st.started + 1, 1u);
    }
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmX); prefetch_tensormap(&tmF); }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, kSlabStages * kSlabBN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // =====================================================================
    // Scheduler + TMA loader
    // =====================================================================
    if (lane == 0) {
      // The filter: nine boxes {64 c, 64 n}, tap t at K offset t * C of the [k_out][r][s][c] matrix.
      mbar_expect_tx(filt_full, kSlabFilterBytes);
      for (int tap = 0; tap < 9; tap++) tma_load_2d(filt + tap * (64 * 128), &tmF, filt_full, tap * p.conv_c, 0);

      const uint32_t num_tiles = static_cast<uint32_t>(p.num_tiles);
      const uint32_t total_draws = num_tiles + kSlabTicketsAhead * gridDim.x;
      const uint32_t wait_target = p.is_consumer ? st.iter * cusync::eval::waitValue(st.in_policy) : 0u;
      const int span = p.conv_rows * p.conv_w;           // output pixels per tile
      uint32_t fills = 0, sched_it = 0;
      bool ok = true;

      // Pipeline registers: tickets of the tiles i, i+1, i+2; schedule entries of i and i+1; probes of i.
      uint32_t tk0 = atomicAdd(st.tile_counter, 1u);
      uint32_t tk1 = atomicAdd(st.tile_counter, 1u);
      uint32_t tk2 = atomicAdd(st.tile_counter, 1u);
      uint32_t y0 = tk0 < num_tiles ? st.tile_order[tk0].y : 0u;
      uint32_t y1 = tk1 < num_tiles ? st.tile_order[tk1].y : 0u;
      uint32_t pr0 = 0, pr1 = 0, pr2 = 0;                // semaphore values seen for tile i: own, above, below
      auto sem_indices = [&](uint32_t ty, uint32_t* own, uint32_t* up, uint32_t* dn) {
        const int tin = static_cast<int>(ty) % p.conv_tiles_per_image;
        const uint32_t m_off = ty * static_cast<uint32_t>(span);
        *own = cusync::eval::tileIndex(st.in_policy, m_off, 0u, st.prod_grid.x, st.prod_grid.y);
        *up = tin > 0 ? cusync::eval::tileIndex(st.in_policy, m_off - span, 0u, st.prod_grid.x, st.prod_grid.y) : *own;
        *dn = tin + 1 < p.conv_tiles_per_image
                  ? cusync::eval::tileIndex(st.in_policy, m_off + span, 0u, st.prod_grid.x, st.prod_grid.y) : *own;
      };
      if (p.is_consumer && tk0 < num_tiles) {
        uint32_t a, b, c;
        sem_indices(y0, &a, &b, &c);
        pr0 = cusync::loadRelaxed(st.sems_wait + a); pr1 = cusync::loadRelaxed(st.sems_wait + b);
        pr2 = cusync::loadRelaxed(st.sems_wait + c);
      }
      while (ok) {
        const bool valid = tk0 < num_tiles;
        const long long lc0 = p.trace ? clock64() : 0;
        // Tile i's dependencies first: the fence that makes its (earlier) probes acquiring would otherwise
        // also wait for the loads issued below for later tiles.
        bool waited_ok = true;
        if (valid && p.is_consumer) {
          if (pr0 < wait_target || pr1 < wait_target || pr2 < wait_target) {
            // not finished when probed: wait (bounded) for the tile itself and its two halo neighbours
            uint32_t idx[3];
            sem_indices(y0, &idx[0], &idx[1], &idx[2]);
            for (int j = 0; j < 3 && waited_ok; j++) {
              uint32_t seen = 0;
              if (!cusync::spinUntilAtLeast(st.sems_wait + idx[j], wait_target, st.timeout_ns, &seen)) {
                bars->abort = 1u;
                cusync::recordTimeout(st.status, 1u, y0 * static_cast<uint32_t>(span), 0u, static_cast<uint32_t>(j), idx[j],
                                      seen, wait_target);
                waited_ok = false;
              }
            }
          } else {
            cusync::fenceAcqRel();  // makes the relaxed probes acquiring
          }
          fence_proxy_async();     // acquire (generic proxy) before the TMA read (async proxy)
        }
        const long long lc1 = p.trace ? clock64() : 0;
        uint32_t tk3 = 0, y2 = 0, pn0 = 0, pn1 = 0, pn2 = 0;
        if (valid) {
          // issue, for later tiles: the draw of i+3, the schedule entry of i+2, the probes of i+1
          tk3 = atomicAdd(st.tile_counter, 1u);
          y2 = tk2 < num_tiles ? st.tile_order[tk2].y : 0u;
          if (p.is_consumer && tk1 < num_tiles) {
            uint32_t a, b, c;
            sem_indices(y1, &a, &b, &c);
            pn0 = cusync::loadRelaxed(st.sems_wait + a); pn1 = cusync::loadRelaxed(st.sems_wait + b);
            pn2 = cusync::loadRelaxed(st.sems_wait + c);
          }
        } else {
          // the three tickets in hand are this block's draws past the end; the launch's last draw re-arms
          // the counter (the reference resets on the last tile, cusync_device_defs.h:87-90)
          if (tk0 == total_draws - 1u || tk1 == total_draws - 1u || tk2 == total_draws - 1u)
            atomicExch(st.tile_counter, 0u);
        }
        const long long lc2 = p.trace ? clock64() : 0;
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
        bars->sched_tile[slot][0] = 0;
        bars->sched_tile[slot][1] = static_cast<int32_t>(y0);
        bars->sched_tile[slot][2] = valid ? 1 : 0;
        bars->sched_tile[slot][3] = static_cast<int32_t>(tk0);
        if (p.trace) bars->sched_time[slot] = cusync::globalTimerNs();
        mbar_arrive(&bars->sched_full[slot]);
        sched_it++;
        if (!valid) break;
        if (!waited_ok) { ok = false; break; }

        const int img = static_cast<int>(y0) / p.conv_tiles_per_image;
        const int h0 = (static_cast<int>(y0) % p.conv_tiles_per_image) * p.conv_rows;
        const long long lc3 = p.trace ? clock64() : 0;
        const uint32_t s = fills % kSlabStages, ph = (fills / kSlabStages) & 1u;
        if (!mbar_wait(&bars->empty[s], ph ^ 1u, ctx)) { ok = false; break; }
        const long long lc4 = p.trace ? clock64() : 0;
        const uint32_t slab_bytes = static_cast<uint32_t>((p.conv_rows + 2) * wp * 128);
        mbar_expect_tx(&bars->full[s], slab_bytes);
        // box {64 channels, W + 2 pixels, conv_rows + 2 rows, 1 image} from pixel (-1, h0 - 1)
        tma_load_4d(slabs + s * kSlabBytes, &tmX, &bars->full[s], 0, -1, h0 - 1, img);
        fills++;
        if (p.trace && tk0 < p.trace_capacity) {
          // loader's cycles for this tile: dependencies | prefetch issue | schedule slot | free slab | TMA issue
          auto cap = [](long long v) { return static_cast<unsigned long long>(v < 0 ? 0 : (v > 4095 ? 4095 : v)); };
          p.trace[8ull * tk0 + 5] = cap(lc1 - lc0) | (cap(lc2 - lc1) << 12) | (cap(lc3 - lc2) << 24) |
                                    (cap(lc4 - lc3) << 36) | (cap(clock64() - lc4) << 48);
        }
        tk0 = tk1; tk1 = tk2; tk2 = tk3; y0 = y1; y1 = y2; pr0 = pn0; pr1 = pn1; pr2 = pn2;
      }
      if (!ok) {
        bars->abort = 1u;
        // wait (bounded) for the copies in flight before the block's shared memory goes away
        const uint32_t live = fills < static_cast<uint32_t>(kSlabStages) ? fills : static_cast<uint32_t>(kSlabStages);
        for (uint32_t j = 0; j < live; j++) {
          const uint32_t f = fills - 1u - j;
          const uint32_t s = f % kSlabStages, ph = (f / kSlabStages) & 1u;
          const uint64_t t0 = cusync::globalTimerNs();
          while (!mbar_try_wait(&bars->full[s], ph)) {
            if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
          }
        }
      }
      // the filter copy must have landed too
      {
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(filt_full, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // =====================================================================
    // MMA issuers.  A 128 x 64 x 16 MMA keeps the tensor pipe busy for about a third of the time one thread
    // needs to issue it, so two threads issue: warp 1 the CTA's even tiles, warp 3 the odd ones, each into
    // its own accumulators.  Both walk the whole schedule ring to stay in step.
    // =====================================================================
    if (lane == 0) {
      const uint32_t me = warp == 1 ? 0u : 1u;
      const uint32_t idesc = make_idesc(kSlabBN, false);
      uint32_t drains = 0, sched_it = 0;
      bool ok = mbar_wait(filt_full, 0u, ctx);
      bool issued = false;
      const uint32_t filt_addr = smem_u32(filt);
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
        const int valid = bars->sched_tile[slot][2];
        const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
        mbar_arrive(&bars->sched_empty[slot]);
        sched_it++;
        if (!valid) break;
        const uint32_t s = drains % kSlabStages, ph = (drains / kSlabStages) & 1u;   // slab and accumulator of tile j
        const bool mine = (drains & 1u) == me;
        if (!mine) { drains++; continue; }
        const uint32_t acc = s;
        const long long t_tile0 = p.trace ? clock64() : 0;
        if (!mbar_wait(&acc_empty[acc], ph ^ 1u, ctx)) { ok = false; break; }
        const long long t_acc = p.trace ? clock64() : 0;
        if (!mbar_wait(&bars->full[s], ph, ctx)) { ok = false; break; }
        const long long t_full = p.trace ? clock64() : 0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kSlabBN;
        const uint32_t slab_addr = smem_u32(slabs + s * kSlabBytes);
#pragma unroll 1
        for (int tap = 0; tap < 9; tap++) {
          const uint32_t a_row = static_cast<uint32_t>((tap / 3) * wp + tap % 3);     // first pixel row of this tap
          const uint32_t a_addr = slab_addr + a_row * 128u;
          const uint32_t b_addr = filt_addr + static_cast<uint32_t>(tap) * (64u * 128u);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; kk++) {
            const uint64_t adesc = make_smem_desc(a_addr + kk * 32, 16u, 1024u);
            const uint64_t bdesc = make_smem_desc(b_addr + kk * 32, 16u, 1024u);
            umma_f16(d_tmem, adesc, bdesc, idesc, (tap > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bars->empty[s]);
        umma_commit(&acc_full[acc]);
        issued = true;
        drains++;
        if (p.trace && ticket < p.trace_capacity) {
          p.trace[8ull * ticket + 4] = static_cast<unsigned long long>(t_full - t_acc);
          p.trace[8ull * ticket + 6] = static_cast<unsigned long long>(clock64() - t_tile0);
          p.trace[8ull * ticket + 7] = static_cast<unsigned long long>(t_acc - t_tile0);
        }
      }
      if (!ok && issued) {
        uint64_t* drain = me ? &bars->splitk_done : &bars->drain;
        umma_commit(drain);
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(drain, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // =====================================================================
    // Epilogue: lane = one M row = one slab pixel; warp (quarter, half) takes 32 of its 64 channels
    // =====================================================================
    const int ew = warp - kEpilogueWarp0;
    const int quarter = ew & 3;
    const int half = ew >> 2;
    uint32_t sched_it = 0, acc_it = 0, post_it = 0;
    bool ok = true;
    const int mrow = quarter * 32 + lane;
    const int prow = mrow / wp, pcol = mrow % wp;       // image row within the tile, column
    const bool px_in = prow < p.conv_rows && pcol < p.conv_w;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
      const unsigned long long t_draw = p.trace ? bars->sched_time[slot] : 0ull;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->sched_empty[slot]);
      sched_it++;
      if (!valid) break;
      const uint32_t acc = acc_it % kSlabStages, aph = (acc_it / kSlabStages) & 1u;
      if (!mbar_wait(&acc_full[acc], aph, ctx)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_mma_done = p.trace ? cusync::globalTimerNs() : 0ull;
      const int m_off = tile_m * p.conv_rows * p.conv_w;      // first output pixel of the tile
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kSlabBN + half * 32, v);
      tmem_ld_wait();
      if (px_in) {
        __half* dst = static_cast<__half*>(p.d) + static_cast<size_t>(m_off + prow * p.conv_w + pcol) * p.ldd + half * 32;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            float x0 = __uint_as_float(v[8 * q + 2 * e]), x1 = __uint_as_float(v[8 * q + 2 * e + 1]);
            if (p.epilogue == CUSYNC_EPILOGUE_RELU) { x0 = fmaxf(x0, 0.0f); x1 = fmaxf(x1, 0.0f); }
            w[e] = pack_half2(x0, x1);
          }
          *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      acc_it++;
      if (p.is_producer) {
        // Hand the tile to the posting thread (warp 2) and go on: the warp barrier above orders every lane's
        // stores before lane 0's arrival, the arrival (release) before the poster's wait (acquire), and the
        // poster's fence + release publish them device-wide.  The barrier belongs to the tile's schedule
        // slot, which the poster gives back only after it has posted: no warp can be a phase ahead on it.
        if (lane == 0) mbar_arrive(&bars->post_slot[slot]);
      }
      if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long* rec = p.trace + 8ull * ticket;
        rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
        rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
      }
    }
  }

  else if (warp == 2 && lane == 0) {
    // =====================================================================
    // Poster: publishes each finished tile (CuStage::post, cusync_device_defs.h:55-72) so that the epilogue
    // warps do not sit out the device-wide fence.  Walks the schedule ring like everybody else.
    // =====================================================================
    uint32_t sched_it = 0;
    bool ok = true;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      sched_it++;
      if (!valid || !p.is_producer) {
        mbar_arrive(&bars->sched_empty[slot]);
        if (!valid) break;
        continue;
      }
      {
        if (!mbar_wait(&bars->post_slot[slot], sph, ctx)) { ok = false; break; }
        const uint32_t m_off = static_cast<uint32_t>(tile_m * p.conv_rows * p.conv_w);
        const uint32_t idx = cusync::eval::tileIndex(st.out_policy, m_off, 0u, st.grid.x, st.grid.y);
        const uint32_t pv = cusync::eval::postValue(st.out_policy);
        cusync::fenceAcqRel();
        if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
        else                                    cusync::addRelease(st.sems_post + idx, pv);
        mbar_arrive(&bars->sched_empty[slot]);      // only now may the slot (and its post barrier) be reused
      }
    }
  }

  // Teardown (normal and abort paths alike).
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kSlabStages * kSlabBN);
  }
}


// ---------------------------------------------------------------------------
// CTA-pair variant: tcgen05.mma.cta_group::2
// ---------------------------------------------------------------------------
// Two CTAs of a cluster (the two SMs of a TPC) compute one 256 x 256 output tile.  CTA r owns rows
// [r*128, r*128+128) of it: it loads its own A rows and HALF of the B tile (128 of the 256 columns),
// and holds its 128 x 256 accumulator in its own tensor memory.  The leader (rank 0) issues one
// M=256 MMA per K step that reads A and the B halves from both CTAs' shared memory.  Per CTA and
// K-block that is 32 KB from L2 instead of 48 KB, and the ring holds six K-blocks instead of four.
// No multicast loads: the only cluster-wide traffic is mbarrier signalling (TMA completion on the
// leader's barrier, tcgen05.commit to both CTAs, remote arrives) and the scheduler's tile broadcast.
// Semaphores stay per 128-row tile: each CTA waits for, and posts, its own rows.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on a LOCAL barrier that a peer CTA may have signalled.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = cusync::globalTimerNs();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
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
// TMA load whose completion may be signalled on the peer CTA's barrier (`bar_cluster_addr` is a
// shared::cluster address); the data lands in this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair when the MMAs retire.
__device__ __forceinline__ void umma_commit_pair_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair_local(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// K depth of one ring stage of the pair kernel: two 64-element swizzle chunks.  A barrier wait, a commit and
// each MMA issue cost the issuing thread of the order of a hundred cycles whatever the MMA's size, so a stage
// carries eight MMAs (and two TMA boxes) per wait/commit instead of four to stay under the tensor time.
constexpr int kPairBlockK = 128;
constexpr int kPairChunkBytes = kBlockM * 128;     // one 64-deep chunk of 128 rows
struct PairCfg {
  static constexpr int kABytes = kBlockM * kPairBlockK * 2;            // this CTA's 128 A rows
  static constexpr int kBHalfBytes = (kPairBN / 2) * kPairBlockK * 2;  // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBHalfBytes;
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kStages = ((int)kSmemLimit - 1024 - kStagingBytes - kBarrierBytes) / kStageBytes;
  static constexpr int kAccCols = kPairBN;
  static constexpr int kTmemCols = 2 * kAccCols;
  static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarrierBytes;
  static_assert(kStages >= 3 && kStages <= 8, "ring depth out of range");
  static_assert(kSmemBytes <= kSmemLimit, "shared memory over budget");
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
cusync_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmWS,
                        const GemmParams p) {
  using C = PairCfg;
  constexpr int BN = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(staging + C::kStagingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader: draws tickets, issues the MMAs
  const bool leader = rank == 0;
  const cusync_stage_view_t& st = p.stage;
  WaitCtx ctx{&bars->abort, st.status, 2 * st.timeout_ns + 1000000000ull};

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; i++) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 2 * kEpilogueWarps);           // leader's: epilogue warps of both CTAs
    }
    for (int i = 0; i < kSchedSlots; i++) {
      mbar_init(&bars->sched_full[i], 1);
      mbar_init(&bars->sched_empty[i], 2 * (1 + kEpilogueWarps));    // leader's: MMA + peer loader + all epilogue warps
    }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->post, kEpilogueWarps);
    mbar_init(&bars->splitk_counted, 1);
    mbar_init(&bars->splitk_done, kEpilogueWarps);
    bars->abort = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    if (p.is_producer) {
      if (blockIdx.x == 0) cusync::storeRelease(st.started, st.iter);
      cusync::addRelease(st.started + 1, 1u);
    }
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmA); prefetch_tensormap(&tmB); prefetch_tensormap(&tmD); }
  if (warp == 2) {
    tmem_alloc_pair(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // Cluster addresses of the leader's barriers that the peer signals.
  const uint32_t leader_full0 = map_to_cta(smem_u32(&bars->full[0]), 0);
  const uint32_t leader_tmem_empty0 = map_to_cta(smem_u32(&bars->tmem_empty[0]), 0);
  const uint32_t leader_sched_empty0 = map_to_cta(smem_u32(&bars->sched_empty[0]), 0);

  if (warp == 0) {
    // =====================================================================
    // Scheduler (leader) + TMA loader (both CTAs)
    // =====================================================================
    if (lane == 0) {
      uint32_t fills = 0, sched_it = 0;
      bool ok = true;
      const uint32_t total_draws = static_cast<uint32_t>(p.num_pairs) + gridDim.x / 2;
      const uint32_t wait_target = p.is_consumer ? st.iter * cusync::eval::waitValue(st.in_policy) : 0u;
      uint32_t sync_stride = 0;
      if (p.is_consumer) {
        const int kind = st.in_policy.kind;
        if (kind == CUSYNC_POLICY_TILESYNC || kind == CUSYNC_POLICY_STRIDEDTILESYNC) sync_stride = st.in_policy.tile_n;
        else if (kind == CUSYNC_POLICY_CONV2DTILESYNC) sync_stride = st.in_policy.tile_n * st.in_policy.p0;
      }
      const uint32_t peer_sched_tile0 = map_to_cta(smem_u32(&bars->sched_tile[0][0]), 1);
      const uint32_t peer_sched_time0 = map_to_cta(smem_u32(&bars->sched_time[0]), 1);
      const uint32_t peer_sched_full0 = map_to_cta(smem_u32(&bars->sched_full[0]), 1);
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        int32_t tn, tpm, valid, tz_slice = 0, nslices = 1;
        if (leader) {
          if (!mbar_wait_cluster(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
          const uint32_t ticket = atomicAdd(st.tile_counter, 1u);
          if (ticket == total_draws - 1u) atomicExch(st.tile_counter, 0u);   // last draw of the launch
          valid = ticket < static_cast<uint32_t>(p.num_pairs) ? 1 : 0;
          PairUnit t = {0, 0, 1u << 16, 0};
          if (valid) t = p.pair_order[ticket];
          tn = static_cast<int32_t>(t.x); tpm = static_cast<int32_t>(t.y);
          tz_slice = static_cast<int32_t>(t.slice_of & 0xffffu); nslices = static_cast<int32_t>(t.slice_of >> 16);
          const unsigned long long now = p.trace ? cusync::globalTimerNs() : 0ull;
          bars->sched_tile[slot][0] = tn; bars->sched_tile[slot][1] = tpm;
          bars->sched_tile[slot][2] = valid; bars->sched_tile[slot][3] = static_cast<int32_t>(ticket);
          bars->sched_tile[slot][4] = tz_slice; bars->sched_tile[slot][5] = nslices;
          bars->sched_tile[slot][6] = static_cast<int32_t>(t.ws_tile);
          bars->sched_time[slot] = now;
          // the same record into the peer's ring, then signal both
          const uint32_t pt = peer_sched_tile0 + slot * 32;
          st_cluster_u32(pt, static_cast<uint32_t>(tn)); st_cluster_u32(pt + 4, static_cast<uint32_t>(tpm));
          st_cluster_u32(pt + 8, static_cast<uint32_t>(valid)); st_cluster_u32(pt + 12, ticket);
          st_cluster_u32(pt + 16, static_cast<uint32_t>(tz_slice)); st_cluster_u32(pt + 20, static_cast<uint32_t>(nslices));
          st_cluster_u32(pt + 24, t.ws_tile);
          st_cluster_u32(peer_sched_time0 + slot * 8, static_cast<uint32_t>(now));
          st_cluster_u32(peer_sched_time0 + slot * 8 + 4, static_cast<uint32_t>(now >> 32));
          mbar_arrive(&bars->sched_full[slot]);
          mbar_arrive_cluster(peer_sched_full0 + slot * 8);
        } else {
          if (!mbar_wait_cluster(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
          tn = bars->sched_tile[slot][0]; tpm = bars->sched_tile[slot][1]; valid = bars->sched_tile[slot][2];
          tz_slice = bars->sched_tile[slot][4]; nslices = bars->sched_tile[slot][5];
          mbar_arrive_cluster(leader_sched_empty0 + slot * 8);
        }
        sched_it++;
        if (!valid) break;

        const int n_off = tn * BN;
        const int m_off = tpm * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;   // this CTA's 128 rows
        const int nb_off = n_off + static_cast<int>(rank) * (BN / 2);               // this CTA's half of B
        uint32_t ready_end = 0;
        long long wait_empty = 0;
        const int kb_per_slice = (p.num_k_blocks + nslices - 1) / nslices;
        const int kb_begin = tz_slice * kb_per_slice;
        const int kb_end = kb_begin + kb_per_slice < p.num_k_blocks ? kb_begin + kb_per_slice : p.num_k_blocks;
        for (int kb = kb_begin; kb < kb_end; kb++) {
          const uint32_t s = fills % C::kStages, ph = (fills / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait_cluster(&bars->empty[s], ph ^ 1u, ctx)) { ok = false; break; }
          if (p.trace) wait_empty += clock64() - c0;
          uint8_t* sa = ring + s * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          const uint32_t full_addr = leader_full0 + s * 8;
          // The leader's barrier collects the bytes of both CTAs.
          if (leader) mbar_expect_tx(&bars->full[s], 2 * C::kStageBytes);
          const int k_base = kb * kPairBlockK;
          // B half: one 3-D box.  [k,n] weights: {64 columns, 128 k rows, 2 column chunks};
          // [n,k] weights: {64 k, 128 n rows, 2 k chunks}.
          if (p.b_kmajor) tma_load_3d_pair(sb, &tmB, full_addr, 0, nb_off, k_base / 64);
          else            tma_load_3d_pair(sb, &tmB, full_addr, 0, k_base, nb_off / 64);
          // The stage spans two 64-deep K chunks; each may open a new producer tile.
#pragma unroll 1
          for (int sub = 0; sub < kPairBlockK / kBlockK && ok; sub++) {
          const int k_off = k_base + sub * kBlockK;
          if (p.is_consumer && m_off < p.m && k_off < p.k) {
            const uint32_t tz = (kb == kb_begin && sub == 0) ? 1u : 0u;
            if (static_cast<uint32_t>(k_off) >= ready_end &&
                cusync::eval::isSync(st.in_policy, static_cast<uint32_t>(k_off), tz)) {
              const uint32_t idx = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(k_off), st.prod_grid.x,
                                                           st.prod_grid.y);
              uint32_t seen = 0;
              if (!cusync::spinUntilAtLeast(st.sems_wait + idx, wait_target, st.timeout_ns, &seen)) {
                bars->abort = 1u;
                cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_off), tz,
                                      idx, seen, wait_target);
                ok = false;
                break;
              }
              if (sync_stride) {
                uint32_t vals[kLookahead];
#pragma unroll
                for (int j = 0; j < kLookahead; j++) {
                  const uint32_t kk = static_cast<uint32_t>(k_off) + (j + 1) * sync_stride;
                  vals[j] = kk < static_cast<uint32_t>(p.k)
                                ? cusync::loadRelaxed(st.sems_wait + cusync::eval::tileIndex(st.in_policy,
                                      static_cast<uint32_t>(m_off), kk, st.prod_grid.x, st.prod_grid.y))
                                : 0u;
                }
                uint32_t ahead = 0;
#pragma unroll
                for (int j = 0; j < kLookahead; j++) {
                  if (ahead == static_cast<uint32_t>(j) && vals[j] >= wait_target) ahead++;
                }
                ready_end = static_cast<uint32_t>(k_off) + (ahead + 1) * sync_stride;
                if (ahead) __threadfence();
              }
              fence_proxy_async();
            }
          }
          }
          // A: {64 k, 128 rows, 2 k chunks}.  Issued on the abort path too, so that the armed barrier
          // completes and the drain below terminates.
          tma_load_3d_pair(sa, &tmA, full_addr, 0, m_off, k_base / 64);
          fills++;
          if (!ok) break;
        }
        if (p.trace) {
          const uint32_t tk = static_cast<uint32_t>(bars->sched_tile[slot][3]);
          if (2 * tk + rank < p.trace_capacity)
            p.trace[8ull * (2 * tk + rank) + 5] = static_cast<unsigned long long>(wait_empty);
        }
      }
      if (!ok) {
        bars->abort = 1u;
        if (leader) {
          // wait (bounded) for the copies of both CTAs that were armed on this CTA's barriers
          const uint32_t live = fills < static_cast<uint32_t>(C::kStages) ? fills : static_cast<uint32_t>(C::kStages);
          for (uint32_t j = 0; j < live; j++) {
            const uint32_t f = fills - 1u - j;
            const uint32_t s = f % C::kStages, ph = (f / C::kStages) & 1u;
            const uint64_t t0 = cusync::globalTimerNs();
            while (!mbar_try_wait_cluster(&bars->full[s], ph)) {
              if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
            }
          }
        } else {
          // the peer's copies complete on the leader's barriers, which it cannot wait on: give
          // them time to land before this CTA's shared memory goes away
          const uint64_t t0 = cusync::globalTimerNs();
          while (cusync::globalTimerNs() - t0 < 100000ull) __nanosleep(1000);
        }
      }
    }
  } else if (warp == 1) {
    // =====================================================================
    // MMA issuer (leader only)
    // =====================================================================
    if (lane == 0 && leader) {
      // instruction descriptor: M = 256 across the pair, N = 256
      const uint32_t idesc = (1u << 4) | ((p.b_kmajor ? 0u : 1u) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>((2 * kBlockM) >> 4) << 24);
      const uint32_t b_lbo = p.b_lbo, b_sbo = p.b_sbo, b_kstep = p.b_kstep;
      uint32_t drains = 0, sched_it = 0, acc_it = 0;
      bool ok = true, issued = false;
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
        const int valid = bars->sched_tile[slot][2];
        const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
        const int slice = bars->sched_tile[slot][4];
        const int nslices = bars->sched_tile[slot][5];
        mbar_arrive(&bars->sched_empty[slot]);
        sched_it++;
        if (!valid) break;
        const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
        const long long t_tile0 = p.trace ? clock64() : 0;
        if (!mbar_wait_cluster(&bars->tmem_empty[acc], aph ^ 1u, ctx)) { ok = false; break; }
        tc_fence_after();
        const long long t_acc = p.trace ? clock64() : 0;
        long long wait_full = 0;
        const uint32_t d_tmem = tmem_base + acc * C::kAccCols;
        const int kb_per_slice = (p.num_k_blocks + nslices - 1) / nslices;
        const int kb_first = slice * kb_per_slice;
        const int kb_count = kb_first + kb_per_slice < p.num_k_blocks ? kb_per_slice : p.num_k_blocks - kb_first;
        for (int kb = 0; kb < kb_count; kb++) {
          const uint32_t s = drains % C::kStages, ph = (drains / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait_cluster(&bars->full[s], ph, ctx)) { ok = false; break; }
          if (p.trace) wait_full += clock64() - c0;
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + s * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int kk = 0; kk < kPairBlockK / kUmmaK; kk++) {
            // K-major operands: 64-deep chunks of 128 rows, 32 bytes per K step inside a chunk.
            // [k,n] B: 2048 bytes (16 rows) per K step, column chunks one leading offset apart.
            const uint32_t a_off = (kk >> 2) * kPairChunkBytes + (kk & 3) * 32;
            const uint32_t b_off = p.b_kmajor ? a_off : kk * b_kstep;
            const uint64_t adesc = make_smem_desc(sa + a_off, 16u, 1024u);
            const uint64_t bdesc = make_smem_desc(sb + b_off, b_lbo, b_sbo);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair_both(&bars->empty[s]);     // frees the ring slot in both CTAs
          issued = true;
          drains++;
        }
        if (!ok) break;
        umma_commit_pair_both(&bars->tmem_full[acc]);
        if (p.trace && 2 * ticket < p.trace_capacity) {
          p.trace[8ull * (2 * ticket) + 4] = static_cast<unsigned long long>(wait_full);
          p.trace[8ull * (2 * ticket) + 6] = static_cast<unsigned long long>(clock64() - t_tile0);
          p.trace[8ull * (2 * ticket) + 7] = static_cast<unsigned long long>(t_acc - t_tile0);
        }
        acc_it++;
      }
      if (!ok && issued) {
        umma_commit_pair_local(&bars->drain);
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(&bars->drain, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // =====================================================================
    // Epilogue (both CTAs, each for its own 128 rows)
    // =====================================================================
    const int ew = warp - kEpilogueWarp0;
    const int quarter = ew & 3;
    const int half = ew >> 2;
    uint8_t* buf = staging + ew * (32 * 128);
    uint32_t sched_it = 0, acc_it = 0, post_it = 0, split_it = 0;
    bool ok = true;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait_cluster(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_n = bars->sched_tile[slot][0];
      const int pair_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      const uint32_t nslices = static_cast<uint32_t>(bars->sched_tile[slot][5]);
      const uint32_t ws_slot = static_cast<uint32_t>(bars->sched_tile[slot][6]) * nslices;   // the tile's first slot
      const uint32_t slice = static_cast<uint32_t>(bars->sched_tile[slot][4]);
      const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
      const unsigned long long t_draw = bars->sched_time[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_sched_empty0 + slot * 8);
      sched_it++;
      if (!valid) break;
      const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
      if (!mbar_wait_cluster(&bars->tmem_full[acc], aph, ctx)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_mma_done = p.trace ? cusync::globalTimerNs() : 0ull;
      const int n_off = tile_n * BN;
      const int m_off = pair_m * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kAccCols;

      if (nslices > 1u) {
        // One K slice of the tile: add it to the workspace; the pair that brings the last slice finalises.
        // `post` is also used by unsplit tiles, the two split-K barriers only here: separate phase counters.
        bool last = false;
        ok = splitk_epilogue<BN>(p, &tmWS, buf, bars, ctx, t_row, n_off, m_off, quarter, half, ew, lane, post_it & 1u,
                                 split_it & 1u, nslices, nullptr, leader_tmem_empty0 + acc * 8,
                                 static_cast<__half*>(p.d), p.ldd, &last,
                                 reinterpret_cast<float4*>(p.splitk_ws) + static_cast<size_t>(ws_slot) * kPairSlotVec4 +
                                     rank * (kPairSlotVec4 / 2),
                                 slice, &tmD);
        acc_it++;
        if (ew == 0 && lane == 0) {
          if (!mbar_wait(&bars->splitk_done, split_it & 1u, ctx)) ok = false;
          else if (last && p.is_producer) {
            const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                         static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
            const uint32_t pv = cusync::eval::postValue(st.out_policy);
            __threadfence();
            if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
            else                                    cusync::addRelease(st.sems_post + idx, pv);
          }
        }
        post_it++;
        split_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (p.trace && ew == 0 && lane == 0 && 2 * ticket + rank < p.trace_capacity) {
          uint32_t smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          unsigned long long* rec = p.trace + 8ull * (2 * ticket + rank);
          rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
          rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
        }
        continue;
      }
      epilogue_store_rows<BN, false>(p, &tmD, buf, t_row, n_off, m_off + quarter * 32, half, lane);

      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tmem_empty0 + acc * 8);
      acc_it++;

      if (p.is_producer && m_off < p.m) {     // a pair's second half may lie past the last row tile
        if (lane == 0) {
          tma_store_wait_all();
          __threadfence();
          // Epilogue warps run at their own pace: one that is a tile ahead must not arrive on `post`
          // while the previous tile's phase is still open (its arrival would close that phase early).
          if (!mbar_wait(&bars->post, (post_it & 1u) ^ 1u, ctx)) ok = false;
          mbar_arrive(&bars->post);
          if (ew == 0) {
            if (!mbar_wait(&bars->post, post_it & 1u, ctx)) ok = false;
            else {
              const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
              const uint32_t pv = cusync::eval::postValue(st.out_policy);
              __threadfence();
              if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
              else                                    cusync::addRelease(st.sems_post + idx, pv);
            }
          }
        }
        post_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      if (p.trace && ew == 0 && lane == 0 && 2 * ticket + rank < p.trace_capacity) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long* rec = p.trace + 8ull * (2 * ticket + rank);
        rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
        rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // Teardown: nobody may leave while the peer can still signal its barriers or read its operands.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || sym == nullptr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// 2-D fp16 tensor map over a row-major [rows, cols] matrix with leading
// dimension ld (elements); box = box_cols x box_rows, 128-byte swizzle.
bool make_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
              uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 3-D view of a row-major [k, n] fp16 matrix whose n is a multiple of 64: {64 columns, k rows, n/64 column
// chunks}; a box of {64, box_rows, box_chunks} lands in shared memory chunk after chunk, each chunk being
// box_rows rows of 128 swizzled bytes -- the layout the MN-major UMMA descriptor walks with its leading offset.
bool make_map_chunked(CUtensorMap* out, const void* base, uint64_t k, uint64_t n, uint64_t ld, uint32_t box_rows,
                      uint32_t box_chunks) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  if (n % 64 != 0) return false;
  cuuint64_t dims[3] = {64, k, n / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, box_rows, box_chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// NHWC fp16 activation [n, h, w, c] as a 4-D tensor {c, w, h, n}; box = {64 channels, w pixels, box_rows image
// rows, 1 image}, 128-byte swizzle.  In shared memory that is box_rows * w rows of 128 bytes: the K-major
// operand layout, one output pixel per row.
bool make_map_nhwc(CUtensorMap* out, const void* base, uint64_t n, uint64_t h, uint64_t w, uint64_t c,
                   uint32_t box_rows, uint32_t box_w = 0) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {c, w, h, n};
  cuuint64_t strides[3] = {c * 2, w * c * 2, h * w * c * 2};
  cuuint32_t box[4] = {64, box_w ? box_w : static_cast<cuuint32_t>(w), box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// fp32 workspace of split-K: [rows, cols] row-major, boxes of 32 columns (128 bytes) x 32 rows.
bool make_map_f32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                         const GemmParams);

struct KernelEntry { KernelFn fn; uint32_t smem; };

template <int BN, bool DUAL>
KernelEntry entry() { return KernelEntry{cusync_gemm_kernel<BN, DUAL>, Cfg<BN, DUAL>::kSmemBytes}; }

bool select_kernel(int tile_n, bool dual, KernelEntry* out) {
  if (!dual) {
    switch (tile_n) {
      case 64:  *out = entry<64, false>(); return true;
      case 128: *out = entry<128, false>(); return true;
      case 256: *out = entry<256, false>(); return true;
      default: return false;
    }
  }
  switch (tile_n) {
    case 64:  *out = entry<64, true>(); return true;
    case 128: *out = entry<128, true>(); return true;
    default: return false;
  }
}

}  // namespace

struct cusync_gemm_plan {
  cusync_gemm_desc_t desc;
  CUtensorMap tmA, tmB, tmB2, tmD, tmWS;
  GemmParams params;
  KernelEntry kernel;
  int tile_n;
  uint32_t num_ctas;
  cusync_stage_t* own_stage;   // created when the caller passes no stage
  cusync_stage_t* stage;
  bool pair;                   // CTA-pair kernel (tcgen05 cta_group::2, 256 x 256 tiles per pair)
  bool conv_slab;              // 3x3 convolution on the slab kernel (64 -> 64 channels)
  PairUnit* pair_order;        // device: schedule over pair work units
  int split_k;
  int tail_split;              // K slices of the tiles of the last, partial wave (pair kernel); 1 = none
  size_t ws_slots;             // pair kernel: 256 x 256 fp32 workspace slots, one per (split tile, slice)
  float* splitk_ws;            // device: fp32 partial sums [tiles_m * 128, n], zero between launches
  uint32_t* splitk_arrivals;   // device: per-tile slice counters, zero between launches
};

namespace {

// K slices per output tile when the caller leaves the choice open: enough to give every SM (or SM pair) a
// work unit when the tile grid alone cannot, as long as a slice keeps at least 1024 of K.
int auto_split_k(int m, int n, int k, int tile_n, bool dual, bool pair, int sms) {
  if (dual || sms <= 0) return 1;
  const int tiles_n = (n + tile_n - 1) / tile_n, tiles_m = (m + kBlockM - 1) / kBlockM;
  const int units = pair ? tiles_n * ((tiles_m + 1) / 2) : tiles_n * tiles_m;
  const int capacity = pair ? sms / 2 : sms;
  // Worth its fp32 workspace traffic only while the tile grid leaves more than half of the machine idle.
  if (2 * units > capacity) return 1;
  int max_split = k / 1024;
  if (max_split > 16) max_split = 16;
  // rounds of work units the machine runs, in units of an unsplit tile's time, plus a few per cent per extra
  // slice for the workspace traffic
  int best = 1;
  double best_cost = 1e30;
  for (int split = 1; split <= max_split; split++) {
    const int rounds = (units * split + capacity - 1) / capacity;
    const double cost = static_cast<double>(rounds) / split * (1.0 + 0.04 * (split - 1));
    if (cost < best_cost - 1e-9) { best_cost = cost; best = split; }
  }
  return best;
}

// Whether cusync_gemm_plan_create picks the CTA-pair kernel when the caller leaves the choice open.
bool pair_by_default(int m, int tile_n, bool dual) {
  return !dual && tile_n == kPairBN && m > kBlockM;
}

// Pair mode: schedule over 256-row pair tiles (the stage's order applied to the pair grid), and the
// number of clusters that can be resident at once.
int setup_pair(cusync_gemm_plan* pl, const cusync_stage_view_t& view, uint32_t cta_cap) {
  GemmParams& p = pl->params;
  const uint32_t pair_rows = static_cast<uint32_t>((p.tiles_m + 1) / 2);
  const uint32_t tiles_n = static_cast<uint32_t>(p.tiles_n);
  const uint32_t split = static_cast<uint32_t>(pl->split_k);
  const uint32_t num_units = pair_rows * tiles_n * split;   // pair tile x uniform K slice, slice outermost
  std::vector<PairUnit> order(num_units, PairUnit{num_units, 0, 0, 0});
  const int kind = view.order & 0xff;
  uint32_t group = static_cast<uint32_t>(view.order) >> 8;
  group = group > 1 ? group / 2 : 1;   // a group of R 128-row tiles is R/2 pair rows
  for (uint32_t z = 0; z < split; z++)
    for (uint32_t y = 0; y < pair_rows; y++)
      for (uint32_t x = 0; x < tiles_n; x++) {
        const uint32_t id = kind == CUSYNC_ORDER_GROUPED_ROWS
                                ? cusync::eval::groupedBlockIndex(group, tiles_n, pair_rows, x, y, z)
                                : cusync::eval::blockIndex(tiles_n, pair_rows, x, y, z);
        if (id >= num_units || order[id].x != num_units) return CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX;
        order[id] = PairUnit{x, y, z | (split << 16), y * tiles_n + x};
      }

  // How many 2-CTA clusters fit on the device at once (one CTA per SM).
  int max_clusters = 0;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * num_units, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, cusync_gemm_pair_kernel, &cfg) != cudaSuccess || max_clusters <= 0) {
    (void)cudaGetLastError();
    max_clusters = cusync_b200_sm_count() / 2;
    if (max_clusters <= 0) max_clusters = 74;
  }
  uint32_t capacity = static_cast<uint32_t>(max_clusters);
  if (cta_cap / 2 >= 1 && capacity > cta_cap / 2) capacity = cta_cap / 2;

  // Tail split: the tiles left over after the last full wave of `capacity` pair tiles would keep only some
  // of the pairs busy for a whole tile's time.  Cut each of them into K slices (the same fp32 workspace
  // and last-arrival finalisation as uniform split-K), so that the tail is spread over all pairs.
  pl->tail_split = 1;
  pl->ws_slots = split > 1 ? static_cast<size_t>(pair_rows) * tiles_n * split : 0;
  if (split == 1 && pl->desc.tail_split != 1) {
    const uint32_t tail = num_units % capacity;
    int best = 1;
    if (pl->desc.tail_split > 1) best = tail ? pl->desc.tail_split : 1;
    // Left to choose (0), the tail is not split: on B200 the split tail measured slower at every GPT-3 MLP
    // shape (the main loop is bound by L2 -> SM operand traffic and the power cap, so idle SM pairs in the
    // last wave are not free throughput, and the extra fp32 round trip through the workspace is not paid back).
    if (best > 1) {
      // whole ring stages per slice; no slice may be left empty by the rounding
      const int per = (p.num_k_blocks + best - 1) / best;
      best = (p.num_k_blocks + per - 1) / per;
    }
    if (best > 1 && tail) {
      std::vector<PairUnit> cut(order.begin(), order.begin() + (num_units - tail));
      for (uint32_t i = num_units - tail; i < num_units; i++)
        for (uint32_t sl = 0; sl < static_cast<uint32_t>(best); sl++)
          cut.push_back(PairUnit{order[i].x, order[i].y, sl | (static_cast<uint32_t>(best) << 16), i - (num_units - tail)});
      order.swap(cut);
      pl->tail_split = best;
      pl->ws_slots = static_cast<size_t>(tail) * best;
    }
  }
  const uint32_t num_pairs = static_cast<uint32_t>(order.size());
  if (cudaMalloc(&pl->pair_order, sizeof(PairUnit) * num_pairs) != cudaSuccess ||
      cudaMemcpy(pl->pair_order, order.data(), sizeof(PairUnit) * num_pairs, cudaMemcpyHostToDevice) != cudaSuccess) {
    (void)cudaGetLastError();
    return CUSYNC_ERROR_CUDA;
  }
  p.pair_order = pl->pair_order;
  p.num_pairs = static_cast<int32_t>(num_pairs);
  uint32_t clusters = num_pairs < capacity ? num_pairs : capacity;
  pl->num_ctas = 2 * clusters;
  return CUSYNC_SUCCESS;
}

int build_maps(cusync_gemm_plan* pl) {
  const cusync_gemm_desc_t& d = pl->desc;
  const bool dual = d.epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL;
  if (pl->pair) {
    // Pair kernel: every operand box is 3-D, {64 contiguous elements, 128 rows, 2 chunks of 64}.
    // A [m,k] and [n,k] weights are chunked along k; [k,n] weights along n.
    bool okp = make_map_chunked(&pl->tmA, d.a, d.m, d.k, d.lda, kBlockM, kPairBlockK / 64);
    if (d.b_layout == CUSYNC_B_ROW_MAJOR_NK) okp = okp && make_map_chunked(&pl->tmB, d.b, d.n, d.k, d.ldb, kPairBN / 2, kPairBlockK / 64);
    else                                     okp = okp && make_map_chunked(&pl->tmB, d.b, d.k, d.n, d.ldb, kPairBlockK, kPairBN / 2 / 64);
    pl->tmB2 = pl->tmB;
    okp = okp && make_map(&pl->tmD, d.d, d.m, d.n, d.ldd, kStoreCols, 32);
    return okp ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
  }
  bool ok = make_map(&pl->tmA, d.a, d.m, d.k, d.lda, kBlockK, kBlockM);
  if (d.b_layout == CUSYNC_B_ROW_MAJOR_NK) {
    const uint32_t b_rows = pl->pair ? pl->tile_n / 2 : pl->tile_n;   // a pair CTA loads half of the B tile
    ok = ok && make_map(&pl->tmB, d.b, d.n, d.k, d.ldb, kBlockK, b_rows);
    if (dual) ok = ok && make_map(&pl->tmB2, d.b2, d.n, d.k, d.ldb, kBlockK, b_rows);
  } else if (pl->params.b_chunked3d) {
    const uint32_t chunks = static_cast<uint32_t>(pl->pair ? pl->tile_n / 2 : pl->tile_n) / 64;
    ok = ok && make_map_chunked(&pl->tmB, d.b, d.k, d.n, d.ldb, kBlockK, chunks);
    if (dual) ok = ok && make_map_chunked(&pl->tmB2, d.b2, d.k, d.n, d.ldb, kBlockK, chunks);
  } else {
    ok = ok && make_map(&pl->tmB, d.b, d.k, d.n, d.ldb, 64, kBlockK);
    if (dual) ok = ok && make_map(&pl->tmB2, d.b2, d.k, d.n, d.ldb, 64, kBlockK);
  }
  if (!dual) pl->tmB2 = pl->tmB;
  ok = ok && make_map(&pl->tmD, d.d, d.m, d.n, d.ldd, kStoreCols, 32);
  return ok ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// Allocation-free GEMM entry point
// ---------------------------------------------------------------------------
// Some hosts of this library may not allocate device memory when they call it:
// a serving runtime that handed the whole device to its own arena and forbids
// cudaMalloc from plug-ins; a latency-critical loop in which cudaMalloc/cudaFree
// would serialise with every stream of the device; a process that is already at
// its memory limit.  The regular path (cusync_gemm_plan_create) allocates a
// stage -- schedule buffer, ticket counter, status words -- with cudaMalloc.
// cusync_gemm_run_noalloc runs the same un-synchronised GEMM kernel with that
// scratch taken from the fixed array below instead.  The array is part of the
// library image: every GPU that loads the library holds these ~97 KB until the
// process exits, whether or not the entry point is ever called.
constexpr uint32_t kNoAllocMaxTiles = 8192;   // 128 x tile_n output tiles per call, at most

struct NoAllocScratch {
  uint32_t words[64];                          // [0] ticket counter, [2..3] started, [8..15] status record
  cusync_dim3_t tile_order[kNoAllocMaxTiles];  // schedule buffer
};

static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

// Re-arms the shared scratch for one call: zero ticket counter and status
// words (they keep the previous call's contents), write the row-major
// schedule.  Device code may name the array directly.
__global__ void noalloc_prepare_kernel(uint32_t tiles_n, uint32_t num_tiles) {
  NoAllocScratch* sc = reinterpret_cast<NoAllocScratch*>(g_noalloc_scratch);
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < 64) sc->words[i] = 0u;
  if (i < num_tiles) sc->tile_order[i] = cusync_dim3_t{i % tiles_n, i / tiles_n, 0u};
}

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
NoAllocScratch* g_noalloc_device_ptr[kNoAllocMaxDevices] = {};

// Device address of the scratch array on the CURRENT device.  In host code the
// array's name is only a handle for the runtime, never an address a kernel
// can use, so the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached.
int noalloc_scratch_for_current_device(NoAllocScratch** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    (void)cudaGetLastError();
    return CUSYNC_ERROR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_device_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return CUSYNC_ERROR_CUDA;
    }
    g_noalloc_device_ptr[dev] = static_cast<NoAllocScratch*>(ptr);
  }
  *out = g_noalloc_device_ptr[dev];
  return CUSYNC_SUCCESS;
}

}  // namespace

extern "C" int cusync_gemm_run_noalloc(const cusync_gemm_desc_t* desc, cusync_stream_t stream) {
  if (desc == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const cusync_gemm_desc_t& d = *desc;
  if (d.stage != nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;   // stages own allocated memory
  if (d.m <= 0 || d.n <= 0 || d.k <= 0 || d.a == nullptr || d.b == nullptr || d.d == nullptr)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.epilogue < CUSYNC_EPILOGUE_NONE || d.epilogue > CUSYNC_EPILOGUE_SILU_MUL_DUAL)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  const bool dual = d.epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL;
  if (dual && d.b2 == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.b_layout != CUSYNC_B_ROW_MAJOR_KN && d.b_layout != CUSYNC_B_ROW_MAJOR_NK) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (!aligned16(d.a) || !aligned16(d.b) || !aligned16(d.d) || (dual && !aligned16(d.b2)))
    return CUSYNC_ERROR_UNSUPPORTED;
  if (d.lda % 8 || d.ldb % 8 || d.ldd % 8 || d.lda < d.k || d.ldd < d.n) return CUSYNC_ERROR_UNSUPPORTED;
  if (d.b_layout == CUSYNC_B_ROW_MAJOR_NK ? d.ldb < d.k : d.ldb < d.n) return CUSYNC_ERROR_UNSUPPORTED;

  cusync_gemm_plan pl;                       // on the stack: tensor maps travel as kernel parameters
  std::memset(&pl, 0, sizeof(pl));
  pl.desc = d;
  pl.tile_n = d.tile_n ? d.tile_n : cusync_gemm_default_tile_n(d.m, d.n, d.k, d.epilogue);
  if (!select_kernel(pl.tile_n, dual, &pl.kernel)) return CUSYNC_ERROR_UNSUPPORTED;
  GemmParams& p = pl.params;
  p.m = d.m; p.n = d.n; p.k = d.k;
  const int64_t tiles_n = (static_cast<int64_t>(d.n) + pl.tile_n - 1) / pl.tile_n;
  const int64_t tiles_m = (static_cast<int64_t>(d.m) + kBlockM - 1) / kBlockM;
  if (tiles_n * tiles_m > static_cast<int64_t>(kNoAllocMaxTiles))
    return CUSYNC_ERROR_EXCEEDS_STATIC_SCRATCH;   // more output tiles than the fixed schedule buffer holds
  p.tiles_n = static_cast<int32_t>(tiles_n);
  p.tiles_m = static_cast<int32_t>(tiles_m);
  p.num_tiles = p.tiles_n * p.tiles_m;
  p.num_k_blocks = (d.k + kBlockK - 1) / kBlockK;
  p.split_k = 1; p.k_blocks_per_split = p.num_k_blocks;
  p.d = d.d; p.ldd = d.ldd;
  p.epilogue = d.epilogue;
  p.b_kmajor = d.b_layout == CUSYNC_B_ROW_MAJOR_NK ? 1 : 0;
  if (p.b_kmajor) { p.b_lbo = 16; p.b_sbo = 1024; p.b_kstep = 32; }
  else            { p.b_lbo = kBlockK * 128; p.b_sbo = 1024; p.b_kstep = kUmmaK * 128; }

  NoAllocScratch* scratch = nullptr;
  int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != CUSYNC_SUCCESS) return rc;
  rc = build_maps(&pl);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (cudaFuncSetAttribute(reinterpret_cast<const void*>(pl.kernel.fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(pl.kernel.smem)) != cudaSuccess) {
    (void)cudaGetLastError();
    return CUSYNC_ERROR_CUDA;
  }

  cusync_stage_view_t& v = p.stage;          // a NoSync stage view over the static scratch
  v.grid = cusync_dim3_t{static_cast<uint32_t>(p.tiles_n), static_cast<uint32_t>(p.tiles_m), 1};
  v.tile_size = cusync_dim3_t{1, 1, 1};
  v.iter = 1;
  v.order = CUSYNC_ORDER_TRANSPOSE_XY;
  v.in_policy.tile_m = v.in_policy.tile_n = v.out_policy.tile_m = v.out_policy.tile_n = 1;
  v.tile_order = scratch->tile_order;
  v.tile_counter = &scratch->words[0];
  v.started = &scratch->words[2];
  v.status = &scratch->words[8];
  v.timeout_ns = cusync::kDefaultSpinTimeoutNs;
  p.is_producer = 0; p.is_consumer = 0;

  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  const uint32_t cap = d.max_ctas > 0 ? static_cast<uint32_t>(d.max_ctas) : static_cast<uint32_t>(sms);
  const uint32_t ctas = static_cast<uint32_t>(p.num_tiles) < cap ? static_cast<uint32_t>(p.num_tiles) : cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint32_t prep_threads = p.num_tiles > 64 ? static_cast<uint32_t>(p.num_tiles) : 64u;
  noalloc_prepare_kernel<<<(prep_threads + 255) / 256, 256, 0, st>>>(static_cast<uint32_t>(p.tiles_n),
                                                                     static_cast<uint32_t>(p.num_tiles));
  pl.kernel.fn<<<ctas, kThreads, pl.kernel.smem, st>>>(pl.tmA, pl.tmB, pl.tmB2, pl.tmD, pl.tmD, p);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

extern "C" {

int cusync_gemm_default_tile_n(int32_t m, int32_t n, int32_t k, int32_t epilogue) {
  (void)k;
  if (epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL) return m <= 128 ? 64 : 128;
  // Every MMA issue costs the issuing thread about as much whatever its width, so wide tiles it is, also for
  // a single row of tiles; split-K then spreads the weight stream over all SMs.
  if (n % 256 == 0 || n >= 2048) return 256;
  return m <= 128 ? 64 : 128;
}

int cusync_gemm_default_split_k(int32_t m, int32_t n, int32_t k, int32_t epilogue, int32_t tile_n, int32_t cta_pair) {
  const bool dual = epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL;
  if (tile_n <= 0) tile_n = cusync_gemm_default_tile_n(m, n, k, epilogue);
  const bool pair_ok = !dual && tile_n == kPairBN && k % 64 == 0;
  const bool pair = cta_pair == 2 || (cta_pair == 0 && pair_ok && pair_by_default(m, tile_n, dual));
  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  return auto_split_k(m, n, k, tile_n, dual, pair, sms);
}

int cusync_gemm_plan_create(cusync_gemm_plan_t** out, const cusync_gemm_desc_t* desc) {
  if (out == nullptr || desc == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_gemm_desc_t& d = *desc;
  if (d.m <= 0 || d.n <= 0 || d.k <= 0 || d.a == nullptr || d.b == nullptr || d.d == nullptr)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  const bool dual = d.epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL;
  if (d.epilogue < CUSYNC_EPILOGUE_NONE || d.epilogue > CUSYNC_EPILOGUE_SILU_MUL_DUAL)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (dual && d.b2 == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  // TMA needs 16-byte aligned bases and row pitches; fp16 => multiples of 8 elements.
  if (!aligned16(d.a) || !aligned16(d.b) || !aligned16(d.d) || (dual && !aligned16(d.b2)))
    return CUSYNC_ERROR_UNSUPPORTED;
  if (d.lda % 8 || d.ldb % 8 || d.ldd % 8 || d.lda < d.k || d.ldd < d.n) return CUSYNC_ERROR_UNSUPPORTED;
  if (d.b_layout == CUSYNC_B_ROW_MAJOR_NK ? d.ldb < d.k : d.ldb < d.n) return CUSYNC_ERROR_UNSUPPORTED;
  if (d.b_layout != CUSYNC_B_ROW_MAJOR_KN && d.b_layout != CUSYNC_B_ROW_MAJOR_NK)
    return CUSYNC_ERROR_INVALID_ARGUMENT;

  cusync_gemm_plan* pl = new (std::nothrow) cusync_gemm_plan();
  if (!pl) return CUSYNC_ERROR_CUDA;
  std::memset(pl, 0, sizeof(*pl));
  pl->desc = d;
  pl->tile_n = d.tile_n ? d.tile_n : cusync_gemm_default_tile_n(d.m, d.n, d.k, d.epilogue);
  if (!select_kernel(pl->tile_n, dual, &pl->kernel)) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  if (d.cta_pair < 0 || d.cta_pair > 2) { delete pl; return CUSYNC_ERROR_INVALID_ARGUMENT; }
  // The pair kernel fetches operands in 64-element chunks of whole rows: K, and N of [k,n] weights, must be
  // multiples of 64 (a ragged last chunk would read past the end of a row).
  const bool pair_ok = !dual && pl->tile_n == kPairBN && d.k % 64 == 0 &&
                       (d.b_layout == CUSYNC_B_ROW_MAJOR_NK || d.n % 64 == 0);
  if (d.cta_pair == 2 && !pair_ok) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  pl->pair = d.cta_pair == 2 || (d.cta_pair == 0 && pair_ok && pair_by_default(d.m, pl->tile_n, dual));
  if (pl->pair) pl->kernel = KernelEntry{nullptr, PairCfg::kSmemBytes};

  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  if (d.split_k < 0 || d.split_k > 64 || (dual && d.split_k > 1)) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  if (d.tail_split < 0 || d.tail_split > 16) { delete pl; return CUSYNC_ERROR_INVALID_ARGUMENT; }
  pl->split_k = d.split_k > 0 ? d.split_k : auto_split_k(d.m, d.n, d.k, pl->tile_n, dual, pl->pair, sms);

  GemmParams& p = pl->params;
  p.m = d.m; p.n = d.n; p.k = d.k;
  p.d = d.d; p.ldd = d.ldd;
  p.tiles_n = (d.n + pl->tile_n - 1) / pl->tile_n;
  p.tiles_m = (d.m + kBlockM - 1) / kBlockM;
  p.num_k_blocks = pl->pair ? (d.k + kPairBlockK - 1) / kPairBlockK : (d.k + kBlockK - 1) / kBlockK;
  // Slices of whole ring stages; drop slices that rounding left empty.
  p.k_blocks_per_split = (p.num_k_blocks + pl->split_k - 1) / pl->split_k;
  pl->split_k = (p.num_k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
  if (d.split_k > 0 && pl->split_k != d.split_k) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  p.split_k = pl->split_k;
  p.num_tiles = p.tiles_n * p.tiles_m * pl->split_k;
  p.epilogue = d.epilogue;
  p.b_kmajor = d.b_layout == CUSYNC_B_ROW_MAJOR_NK ? 1 : 0;
  // [k,n] weights whose n is a whole number of 64-column chunks are fetched with one 3-D box per K-block
  // (a ragged last chunk would read past the end of a row, so such matrices keep one 2-D box per chunk).
  p.b_chunked3d = (!p.b_kmajor && d.n % 64 == 0 && pl->tile_n > 64) ? 1 : 0;
  if (p.b_kmajor) {
    // K-major, 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart; one UMMA K step
    // (16 fp16) is 32 B along the row.  The leading offset is unused for swizzled K-major operands.
    p.b_lbo = 16; p.b_sbo = 1024; p.b_kstep = 32;
  } else {
    // MN-major ([k,n] row-major), 128-byte swizzle: each TMA box holds 64 columns x kBlockK rows;
    // 64-column groups are one box (kBlockK * 128 B) apart, 8-row K groups 1024 B apart, and one
    // UMMA K step is 16 rows = 2048 B.
    p.b_lbo = (pl->pair ? kPairBlockK : kBlockK) * 128; p.b_sbo = 1024; p.b_kstep = kUmmaK * 128;
  }

  pl->stage = d.stage;
  if (pl->stage == nullptr) {
    cusync_dim3_t grid = {static_cast<uint32_t>(p.tiles_n), static_cast<uint32_t>(p.tiles_m),
                          static_cast<uint32_t>(pl->split_k)};
    cusync_dim3_t ts = {1, 1, 1};
    int rc = cusync_stage_create(&pl->own_stage, grid, ts, CUSYNC_ORDER_TRANSPOSE_XY, nullptr, nullptr,
                                 CUSYNC_OPT_NONE);
    if (rc != CUSYNC_SUCCESS) { delete pl; return rc; }
    pl->stage = pl->own_stage;
  }
  cusync_stage_view_t view;
  cusync_stage_get_view(pl->stage, &view);
  // The stage's grid is the tile grid (N tiles, M tiles, K slices), as
  // CuSyncGemmHorizontalThreadblockSwizzle lays it out.
  if (view.grid.x != static_cast<uint32_t>(p.tiles_n) || view.grid.y != static_cast<uint32_t>(p.tiles_m) ||
      view.grid.z != static_cast<uint32_t>(pl->split_k)) {
    if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
    delete pl;
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  }
  if (view.in_policy.kind != CUSYNC_POLICY_NOSYNC && view.sems_wait == nullptr) {
    if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
    delete pl;
    return CUSYNC_ERROR_NOT_INITIALIZED;   // consumer not wired to a producer yet
  }

  uint32_t cap = d.max_ctas > 0 ? static_cast<uint32_t>(d.max_ctas) : static_cast<uint32_t>(sms);
  pl->num_ctas = static_cast<uint32_t>(p.num_tiles) < cap ? static_cast<uint32_t>(p.num_tiles) : cap;

  int rc = CUSYNC_SUCCESS;
  const void* kernel_fn = pl->pair ? reinterpret_cast<const void*>(cusync_gemm_pair_kernel)
                                   : reinterpret_cast<const void*>(pl->kernel.fn);
  if (rc == CUSYNC_SUCCESS &&
      cudaFuncSetAttribute(kernel_fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(pl->kernel.smem)) != cudaSuccess) {
    (void)cudaGetLastError();
    rc = CUSYNC_ERROR_CUDA;
  }
  pl->tail_split = 1;
  if (rc == CUSYNC_SUCCESS && pl->pair) rc = setup_pair(pl, view, cap);
  if (rc == CUSYNC_SUCCESS && (pl->split_k > 1 || pl->tail_split > 1)) {
    // 1-CTA kernel: one [m, n] fp32 tile set that the slices reduce-add into and the finaliser zeroes again;
    // CTA-pair kernel: one 256 x 256 slot per slice of every split tile (needs no zeroing).
    const size_t ws_bytes = pl->pair ? pl->ws_slots * (2 * kBlockM) * kPairBN * sizeof(float)
                                     : static_cast<size_t>(p.tiles_m) * kBlockM * static_cast<size_t>(d.n) * sizeof(float);
    const size_t cnt_bytes = static_cast<size_t>(p.tiles_m) * p.tiles_n * sizeof(uint32_t);
    if (cudaMalloc(&pl->splitk_ws, ws_bytes) != cudaSuccess || cudaMemset(pl->splitk_ws, 0, ws_bytes) != cudaSuccess ||
        cudaMalloc(&pl->splitk_arrivals, cnt_bytes) != cudaSuccess ||
        cudaMemset(pl->splitk_arrivals, 0, cnt_bytes) != cudaSuccess) {
      (void)cudaGetLastError();
      rc = CUSYNC_ERROR_CUDA;
    }
    p.splitk_ws = pl->splitk_ws;
    p.splitk_arrivals = pl->splitk_arrivals;
    if (rc == CUSYNC_SUCCESS) {
      // (the pair kernel writes its slots with plain stores and needs no map)
      if (!pl->pair && !make_map_f32(&pl->tmWS, pl->splitk_ws, d.m, d.n, d.n)) rc = CUSYNC_ERROR_CUDA;
    }
  }
  if (rc == CUSYNC_SUCCESS) rc = build_maps(pl);
  if (rc != CUSYNC_SUCCESS) {
    if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
    cudaFree(pl->pair_order); cudaFree(pl->splitk_ws); cudaFree(pl->splitk_arrivals);
    delete pl;
    return rc;
  }
  *out = pl;
  return CUSYNC_SUCCESS;
}

int cusync_gemm_plan_destroy(cusync_gemm_plan_t* pl) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  cudaFree(pl->pair_order); cudaFree(pl->splitk_ws); cudaFree(pl->splitk_arrivals);
  if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
  delete pl;
  return CUSYNC_SUCCESS;
}

int cusync_gemm_plan_update(cusync_gemm_plan_t* pl, const void* a, const void* b, const void* b2, void* d) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (a) pl->desc.a = a;
  if (b) pl->desc.b = b;
  if (b2) pl->desc.b2 = b2;
  if (d) { pl->desc.d = d; pl->params.d = d; }
  if (!aligned16(pl->desc.a) || !aligned16(pl->desc.b) || !aligned16(pl->desc.d)) return CUSYNC_ERROR_UNSUPPORTED;
  return build_maps(pl);
}

uint32_t cusync_gemm_plan_num_ctas(const cusync_gemm_plan_t* pl) { return pl ? pl->num_ctas : 0; }

int cusync_gemm_plan_tail_split(const cusync_gemm_plan_t* pl) { return pl && pl->tail_split > 1 ? pl->tail_split : 1; }

int cusync_gemm_plan_set_trace(cusync_gemm_plan_t* pl, void* device_buffer, uint32_t capacity_tiles) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  pl->params.trace = static_cast<unsigned long long*>(device_buffer);
  pl->params.trace_capacity = device_buffer ? capacity_tiles : 0;
  return CUSYNC_SUCCESS;
}

int cusync_gemm_run(cusync_gemm_plan_t* pl, cusync_stream_t stream) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  GemmParams p = pl->params;
  cusync_stage_get_view(pl->stage, &p.stage);   // picks up the current iter
  p.is_producer = p.stage.out_policy.kind != CUSYNC_POLICY_NOSYNC;
  p.is_consumer = p.stage.in_policy.kind != CUSYNC_POLICY_NOSYNC;
  if (p.is_producer) cusync_stage_note_launch(pl->stage, pl->num_ctas);
  if (pl->conv_slab)
    cusync_conv3x3_slab_kernel<<<pl->num_ctas, kThreads, kSlabSmemBytes, reinterpret_cast<cudaStream_t>(stream)>>>(
        pl->tmA, pl->tmB, p);
  else if (pl->pair)
    cusync_gemm_pair_kernel<<<pl->num_ctas, kThreads, pl->kernel.smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        pl->tmA, pl->tmB, pl->tmD, pl->tmWS, p);
  else
    pl->kernel.fn<<<pl->num_ctas, kThreads, pl->kernel.smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        pl->tmA, pl->tmB, pl->tmB2, pl->tmD, pl->tmWS, p);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

// ---------------------------------------------------------------------------
// 3x3 convolution (implicit GEMM on the same kernel)
// ---------------------------------------------------------------------------
int cusync_conv2d_tile_rows(int32_t w) {
  if (w <= 0 || w > kBlockM) return 0;
  return kBlockM / w;     // whole image rows per 128-pixel M tile
}

int cusync_conv2d_plan_create(cusync_conv2d_plan_t** out, const cusync_conv2d_desc_t* desc) {
  if (out == nullptr || desc == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_conv2d_desc_t& d = *desc;
  if (d.n <= 0 || d.h <= 0 || d.w <= 0 || d.c <= 0 || d.k <= 0 || !d.x || !d.filter || !d.y)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.epilogue != CUSYNC_EPILOGUE_NONE && d.epilogue != CUSYNC_EPILOGUE_RELU) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.r != 3 || d.s != 3 || d.stride != 1 || d.pad != 1) return CUSYNC_ERROR_UNSUPPORTED;
  // channels in whole 64-element K chunks / 64-wide N tiles; an M tile is whole image rows
  const int rows = cusync_conv2d_tile_rows(d.w);
  if (d.c % 64 || d.k % 64 || rows == 0 || d.h % rows) return CUSYNC_ERROR_UNSUPPORTED;
  if (!aligned16(d.x) || !aligned16(d.filter) || !aligned16(d.y)) return CUSYNC_ERROR_UNSUPPORTED;

  cusync_gemm_plan* pl = new (std::nothrow) cusync_gemm_plan();
  if (!pl) return CUSYNC_ERROR_CUDA;
  std::memset(pl, 0, sizeof(*pl));
  pl->tile_n = 64;
  pl->split_k = 1;
  pl->kernel = KernelEntry{cusync_gemm_kernel<64, false, true>, Cfg<64, false>::kSmemBytes};
  GemmParams& p = pl->params;
  p.m = d.n * d.h * d.w; p.n = d.k; p.k = 9 * d.c;
  p.d = d.y; p.ldd = d.k;
  p.tiles_n = d.k / 64;
  p.conv_n = d.n; p.conv_h = d.h; p.conv_w = d.w; p.conv_c = d.c;
  p.conv_rows = rows; p.conv_tiles_per_image = d.h / rows;
  p.tiles_m = d.n * p.conv_tiles_per_image;
  p.num_tiles = p.tiles_n * p.tiles_m;
  p.num_k_blocks = 9 * (d.c / 64);
  p.split_k = 1; p.k_blocks_per_split = p.num_k_blocks;
  p.epilogue = d.epilogue;
  p.b_kmajor = 1;                                  // filter [k_out][r][s][c] is an [n, k] matrix
  p.b_lbo = 16; p.b_sbo = 1024; p.b_kstep = 32;

  pl->stage = d.stage;
  if (pl->stage == nullptr) {
    cusync_dim3_t grid = {static_cast<uint32_t>(p.tiles_n), static_cast<uint32_t>(p.tiles_m), 1};
    cusync_dim3_t ts = {1, 1, 1};
    int rc = cusync_stage_create(&pl->own_stage, grid, ts, CUSYNC_ORDER_TRANSPOSE_XY, nullptr, nullptr, CUSYNC_OPT_NONE);
    if (rc != CUSYNC_SUCCESS) { delete pl; return rc; }
    pl->stage = pl->own_stage;
  }
  cusync_stage_view_t view;
  cusync_stage_get_view(pl->stage, &view);
  int rc = CUSYNC_SUCCESS;
  if (view.grid.x != static_cast<uint32_t>(p.tiles_n) || view.grid.y != static_cast<uint32_t>(p.tiles_m) || view.grid.z != 1)
    rc = CUSYNC_ERROR_INVALID_ARGUMENT;
  else if (view.in_policy.kind != CUSYNC_POLICY_NOSYNC && view.sems_wait == nullptr)
    rc = CUSYNC_ERROR_NOT_INITIALIZED;
  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  const uint32_t cap = d.max_ctas > 0 ? static_cast<uint32_t>(d.max_ctas) : static_cast<uint32_t>(sms);
  pl->num_ctas = static_cast<uint32_t>(p.num_tiles) < cap ? static_cast<uint32_t>(p.num_tiles) : cap;
  // The slab kernel serves the 64 -> 64 channel layer when a tile's padded rows still fit the 128-row MMA and
  // the consumer side waits once per tile (no input policy, or Conv2DTileSync over a one-column producer grid).
  pl->conv_slab = rc == CUSYNC_SUCCESS && d.c == 64 && d.k == 64 && rows * (d.w + 2) <= kBlockM &&
                  d.w + 2 <= 256 &&
                  (view.in_policy.kind == CUSYNC_POLICY_NOSYNC ||
                   (view.in_policy.kind == CUSYNC_POLICY_CONV2DTILESYNC && view.prod_grid.x == 1)) &&
                  std::getenv("CUSYNC_CONV_GENERAL") == nullptr;
  if (rc == CUSYNC_SUCCESS) {
    bool ok = (pl->conv_slab ? make_map_nhwc(&pl->tmA, d.x, d.n, d.h, d.w, d.c, static_cast<uint32_t>(rows + 2),
                                             static_cast<uint32_t>(d.w + 2))
                             : make_map_nhwc(&pl->tmA, d.x, d.n, d.h, d.w, d.c, static_cast<uint32_t>(rows))) &&
              make_map(&pl->tmB, d.filter, d.k, 9ull * d.c, 9ull * d.c, kBlockK, 64);
    pl->tmB2 = pl->tmB; pl->tmD = pl->tmB; pl->tmWS = pl->tmB;      // unused by the convolution path
    if (!ok) rc = CUSYNC_ERROR_CUDA;
  }
  if (rc == CUSYNC_SUCCESS &&
      (pl->conv_slab
           ? cudaFuncSetAttribute(reinterpret_cast<const void*>(cusync_conv3x3_slab_kernel),
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSlabSmemBytes))
           : cudaFuncSetAttribute(reinterpret_cast<const void*>(pl->kernel.fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(pl->kernel.smem))) != cudaSuccess) {
    (void)cudaGetLastError();
    rc = CUSYNC_ERROR_CUDA;
  }
  if (rc != CUSYNC_SUCCESS) {
    if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
    delete pl;
    return rc;
  }
  *out = pl;
  return CUSYNC_SUCCESS;
}

int cusync_conv2d_plan_destroy(cusync_conv2d_plan_t* pl) { return cusync_gemm_plan_destroy(pl); }
int cusync_conv2d_run(cusync_conv2d_plan_t* pl, cusync_stream_t stream) { return cusync_gemm_run(pl, stream); }
uint32_t cusync_conv2d_plan_num_ctas(const cusync_conv2d_plan_t* pl) { return pl ? pl->num_ctas : 0; }

}  // extern "C"
