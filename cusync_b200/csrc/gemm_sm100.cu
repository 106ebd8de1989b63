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

#include "sm100_device.cuh"
#include "gemm_kernel_1cta.cuh"
#include "conv3x3_slab_kernel.cuh"
#include "gemm_kernel_pair.cuh"

namespace {

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
      case 192: *out = entry<192, false>(); return true;
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
// From three row tiles on: with two (M <= 256) the one-CTA kernel's 128-row tiles give twice the work units,
// which measured 9 % faster on the GPT-3 MLP shard at M = 256.
bool pair_by_default(int m, int tile_n, bool dual) {
  // (the dual GEMM on CTA pairs computes 128-column output tiles: its 256-column MMA is [A B | A B2])
  return tile_n == (dual ? kPairBN / 2 : kPairBN) && m > 2 * kBlockM;
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
    if (dual) {
      if (d.b_layout == CUSYNC_B_ROW_MAJOR_NK) okp = okp && make_map_chunked(&pl->tmB2, d.b2, d.n, d.k, d.ldb, kPairBN / 2, kPairBlockK / 64);
      else                                     okp = okp && make_map_chunked(&pl->tmB2, d.b2, d.k, d.n, d.ldb, kPairBlockK, kPairBN / 2 / 64);
    }
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

// The library kernels evaluate a stage's policies with THEIR tile shape: tile_m rows (128, or the pixels of a
// convolution tile) by tile_n columns, K walked in 64-element blocks.  A policy built for another shape would
// index semaphores the stage does not have (a producer posting past the end of its array) or cover fewer rows
// than a block loads (a consumer reading rows nobody has waited for).  Checked once, on the host.
int check_stage_policies(const cusync_stage_view_t& v, uint32_t tile_m, uint32_t tile_n, uint32_t k_extent, bool conv) {
  const cusync_policy_t& out = v.out_policy;
  if (out.kind != CUSYNC_POLICY_NOSYNC && out.kind != CUSYNC_POLICY_CUSTOM) {
    const uint64_t num_sems = static_cast<uint64_t>(v.grid.x) * v.grid.y * v.grid.z;
    for (uint32_t y = 0; y < v.grid.y; y++)
      for (uint32_t x = 0; x < v.grid.x; x++)
        if (cusync::eval::tileIndex(out, y * tile_m, x * tile_n, v.grid.x, v.grid.y) >= num_sems)
          return CUSYNC_ERROR_INVALID_ARGUMENT;
  }
  const cusync_policy_t& in = v.in_policy;
  if (in.kind != CUSYNC_POLICY_NOSYNC && in.kind != CUSYNC_POLICY_CUSTOM) {
    // a block waits on the semaphore of its first row: the producer's row tiles must be whole multiples of it
    if (conv ? in.tile_m != tile_m : in.tile_m % tile_m != 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
    const bool walks_k = in.kind == CUSYNC_POLICY_TILESYNC || in.kind == CUSYNC_POLICY_STRIDEDTILESYNC ||
                         in.kind == CUSYNC_POLICY_CONV2DTILESYNC;
    // (a convolution's K walk is channel chunks of 64 outermost: producer tiles are whole chunks wide)
    if (walks_k && in.tile_n % kBlockK != 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
    const uint64_t prod_sems = static_cast<uint64_t>(v.prod_grid.x) * v.prod_grid.y * v.prod_grid.z;
    for (uint32_t y = 0; y < v.grid.y; y++)
      for (uint32_t k = 0; k < k_extent; k += kBlockK)
        if (cusync::eval::tileIndex(in, y * tile_m, k, v.prod_grid.x, v.prod_grid.y) >= prod_sems)
          return CUSYNC_ERROR_INVALID_ARGUMENT;
  }
  return CUSYNC_SUCCESS;
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

// The opt-in to more than 48 KB of dynamic shared memory is a property of (kernel, device): set once, not per call.
int noalloc_allow_large_smem(const KernelEntry& k) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  constexpr int kKernels = 8;
  static KernelFn done_fn[kNoAllocMaxDevices][kKernels] = {};
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  for (int i = 0; i < kKernels; i++) {
    if (done_fn[dev][i] == k.fn) return CUSYNC_SUCCESS;
    if (done_fn[dev][i] == nullptr) {
      if (cudaFuncSetAttribute(reinterpret_cast<const void*>(k.fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(k.smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return CUSYNC_ERROR_CUDA;
      }
      done_fn[dev][i] = k.fn;
      return CUSYNC_SUCCESS;
    }
  }
  return CUSYNC_ERROR_CUDA;   // more kernel instantiations than select_kernel offers: cannot happen
}

}  // namespace

// The timeout record of the allocation-free entry point lives in its static array (no stage owns it): copies
// it to the host.  Synchronous with respect to the device's work; allocates nothing.
extern "C" int cusync_gemm_noalloc_read_status(cusync_status_t* out) {
  if (out == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  NoAllocScratch* scratch = nullptr;
  const int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (cudaMemcpy(out, &scratch->words[8], sizeof(cusync_status_t), cudaMemcpyDeviceToHost) != cudaSuccess) {
    (void)cudaGetLastError();
    return CUSYNC_ERROR_CUDA;
  }
  return CUSYNC_SUCCESS;
}

extern "C" int cusync_gemm_run_noalloc(const cusync_gemm_desc_t* desc, cusync_stream_t stream) {
  if (desc == nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const cusync_gemm_desc_t& d = *desc;
  if (d.stage != nullptr || d.b_stage != nullptr) return CUSYNC_ERROR_INVALID_ARGUMENT;   // stages own allocated memory
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
  // Only the one-CTA-per-tile kernel without K slices runs here: the other forms need a workspace or a
  // schedule of their own, which the plan-based path allocates.  Asking for them is refused, not ignored.
  if (d.split_k > 1 || d.cta_pair == 2 || d.tail_split > 1) return CUSYNC_ERROR_UNSUPPORTED;

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
  rc = noalloc_allow_large_smem(pl.kernel);
  if (rc != CUSYNC_SUCCESS) return rc;

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
  const bool pair_ok = pl->tile_n == (dual ? kPairBN / 2 : kPairBN) && d.k % 64 == 0 &&
                       (d.b_layout == CUSYNC_B_ROW_MAJOR_NK || d.n % 64 == 0);
  if (d.cta_pair == 2 && !pair_ok) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  pl->pair = d.cta_pair == 2 || (d.cta_pair == 0 && pair_ok && pair_by_default(d.m, pl->tile_n, dual));
  if (pl->pair) pl->kernel = KernelEntry{nullptr, PairCfg::kSmemBytes};
  // A produced B operand is waited for by the CTA-pair kernel's loader only, one wait per unit or ring stage.
  if (d.b_stage != nullptr && (!pl->pair || d.split_k > 1 || d.tail_split > 1 || d.b_sem_value == 0)) {
    delete pl;
    return CUSYNC_ERROR_UNSUPPORTED;
  }

  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  if (d.split_k < 0 || d.split_k > 64 || (dual && d.split_k > 1)) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  if (d.tail_split < 0 || d.tail_split > 16) { delete pl; return CUSYNC_ERROR_INVALID_ARGUMENT; }
  // (the K-sliced paths sum plain accumulators: no finaliser for the dual epilogue's two halves)
  if (dual && d.tail_split > 1) { delete pl; return CUSYNC_ERROR_UNSUPPORTED; }
  pl->split_k = d.split_k > 0 ? d.split_k : d.b_stage ? 1 : auto_split_k(d.m, d.n, d.k, pl->tile_n, dual, pl->pair, sms);

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
  {
    const int prc = check_stage_policies(view, kBlockM, static_cast<uint32_t>(pl->tile_n), static_cast<uint32_t>(d.k), false);
    if (prc != CUSYNC_SUCCESS) {
      if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
      delete pl;
      return prc;
    }
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

namespace {
int gemm_launch(cusync_gemm_plan_t* pl, cusync_stream_t stream, bool dependent);
}

int cusync_gemm_run(cusync_gemm_plan_t* pl, cusync_stream_t stream) { return gemm_launch(pl, stream, false); }

int cusync_gemm_run_dependent(cusync_gemm_plan_t* pl, cusync_stream_t stream) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  // Only a consumer may start before the kernel ahead of it has finished: its semaphore waits order the reads.
  cusync_stage_view_t v;
  cusync_stage_get_view(pl->stage, &v);
  if (v.in_policy.kind == CUSYNC_POLICY_NOSYNC && pl->desc.b_stage == nullptr) return CUSYNC_ERROR_NOT_CONSUMER;
  return gemm_launch(pl, stream, true);
}

namespace {
int gemm_launch(cusync_gemm_plan_t* pl, cusync_stream_t stream, bool dependent) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  GemmParams p = pl->params;
  cusync_stage_get_view(pl->stage, &p.stage);   // picks up the current iter
  p.is_producer = p.stage.out_policy.kind != CUSYNC_POLICY_NOSYNC;
  p.is_consumer = p.stage.in_policy.kind != CUSYNC_POLICY_NOSYNC;
  if (p.is_producer) cusync_stage_note_launch(pl->stage, pl->num_ctas);
  if (pl->desc.b_stage != nullptr) {
    cusync_stage_view_t bv;
    cusync_stage_get_view(pl->desc.b_stage, &bv);
    if (bv.sems_post == nullptr) return CUSYNC_ERROR_NOT_PRODUCER;
    // every index the kernel can form must be one of the producer's semaphores
    const uint64_t blocks = (static_cast<uint64_t>(p.b_kmajor ? p.n : p.k) + kBlockM - 1) / kBlockM;
    const uint64_t last = pl->desc.b_sem_first + (blocks - 1) * pl->desc.b_sem_stride;
    if (last >= static_cast<uint64_t>(bv.grid.x) * bv.grid.y * bv.grid.z) return CUSYNC_ERROR_INVALID_ARGUMENT;
    p.b_sems = bv.sems_post;
    p.b_sem_first = pl->desc.b_sem_first; p.b_sem_stride = pl->desc.b_sem_stride; p.b_sem_value = pl->desc.b_sem_value;
  }
  const cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dependent) {
    cudaError_t e;
    if (pl->conv_slab)
      e = launchDependent(cusync_conv3x3_slab_kernel, dim3(pl->num_ctas), dim3(kThreads), kSlabSmemBytes, st,
                          pl->tmA, pl->tmB, p);
    else if (pl->pair)
      e = launchDependent(cusync_gemm_pair_kernel, dim3(pl->num_ctas), dim3(kThreads), pl->kernel.smem, st,
                          pl->tmA, pl->tmB, pl->tmD, pl->tmWS, pl->tmB2, p);
    else
      e = launchDependent(pl->kernel.fn, dim3(pl->num_ctas), dim3(kThreads), pl->kernel.smem, st,
                          pl->tmA, pl->tmB, pl->tmB2, pl->tmD, pl->tmWS, p);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
    return CUSYNC_SUCCESS;
  }
  if (pl->conv_slab)
    cusync_conv3x3_slab_kernel<<<pl->num_ctas, kThreads, kSlabSmemBytes, st>>>(pl->tmA, pl->tmB, p);
  else if (pl->pair)
    cusync_gemm_pair_kernel<<<pl->num_ctas, kThreads, pl->kernel.smem, st>>>(
        pl->tmA, pl->tmB, pl->tmD, pl->tmWS, pl->tmB2, p);
  else
    pl->kernel.fn<<<pl->num_ctas, kThreads, pl->kernel.smem, st>>>(pl->tmA, pl->tmB, pl->tmB2, pl->tmD, pl->tmWS, p);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}
}  // namespace

// Two dependent GEMMs in one persistent grid (both on the CTA-pair kernel).
int cusync_gemm_chain_supported(const cusync_gemm_plan_t* first, const cusync_gemm_plan_t* second) {
  return first && second && first->pair && second->pair && !first->conv_slab && !second->conv_slab ? 1 : 0;
}

// Loads the chain kernel and opts it in to its shared-memory size, once.  Called when a chain is set up (the
// MLP driver's create) and again, as a no-op, by every run: the first run must not be the one that loads the
// kernel, since a load can wait for kernels that are already running (an all-reduce kernel beside the chain).
int cusync_gemm_chain_prepare(void) {
  static bool attr_set = false;
  if (attr_set) return CUSYNC_SUCCESS;
  if (cudaFuncSetAttribute(reinterpret_cast<const void*>(cusync_gemm_pair_chain_kernel),
                           cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(PairCfg::kSmemBytes)) != cudaSuccess) {
    (void)cudaGetLastError();
    return CUSYNC_ERROR_CUDA;
  }
  attr_set = true;
  return CUSYNC_SUCCESS;
}

int cusync_gemm_run_chain(cusync_gemm_plan_t* first, cusync_gemm_plan_t* second, cusync_stream_t stream) {
  if (!first || !second) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!cusync_gemm_chain_supported(first, second)) return CUSYNC_ERROR_UNSUPPORTED;
  if (cusync_gemm_chain_prepare() != CUSYNC_SUCCESS) return CUSYNC_ERROR_CUDA;
  GemmParams p0 = first->params, p1 = second->params;
  cusync_stage_get_view(first->stage, &p0.stage);
  cusync_stage_get_view(second->stage, &p1.stage);
  p0.is_producer = p0.stage.out_policy.kind != CUSYNC_POLICY_NOSYNC;
  p0.is_consumer = p0.stage.in_policy.kind != CUSYNC_POLICY_NOSYNC;
  p1.is_producer = p1.stage.out_policy.kind != CUSYNC_POLICY_NOSYNC;
  p1.is_consumer = p1.stage.in_policy.kind != CUSYNC_POLICY_NOSYNC;
  // The grid: as many pairs as either plan may use, and no more than there are work units.
  uint32_t ctas = first->num_ctas > second->num_ctas ? first->num_ctas : second->num_ctas;
  const uint32_t units = static_cast<uint32_t>(p0.num_pairs) + static_cast<uint32_t>(p1.num_pairs);
  if (ctas > 2 * units) ctas = 2 * units;
  if (p0.is_producer) cusync_stage_note_launch(first->stage, ctas);
  if (p1.is_producer) cusync_stage_note_launch(second->stage, ctas);
  cusync_gemm_pair_chain_kernel<<<ctas, kThreads, PairCfg::kSmemBytes, reinterpret_cast<cudaStream_t>(stream)>>>(
      first->tmA, first->tmB, first->tmD, first->tmWS, second->tmA, second->tmB, second->tmD, second->tmWS,
      first->tmB2, second->tmB2, p0, p1);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}

// ---------------------------------------------------------------------------
// 3x3 convolution (implicit GEMM on the same kernel)
// ---------------------------------------------------------------------------
int cusync_conv2d_tile_rows(int32_t w) {
  if (w <= 0 || w > kBlockM) return 0;
  return kBlockM / w;     // whole image rows per 128-pixel M tile
}

int cusync_conv2d_tile_rows_hw(int32_t h, int32_t w) {
  // the most whole image rows whose pixels fit the 128-row MMA AND that divide the image height, so that no tile
  // straddles two images (14 x 14: 7 rows = 98 pixels; 7 x 7: the whole image, 49 pixels)
  int rows = cusync_conv2d_tile_rows(w);
  if (rows == 0 || h <= 0) return 0;
  if (rows > h) rows = h;
  while (h % rows) rows--;
  return rows;
}

int cusync_conv2d_default_tile_n(int32_t n, int32_t h, int32_t w, int32_t c, int32_t k) {
  (void)c;
  const int rows = cusync_conv2d_tile_rows_hw(h, w);
  if (rows <= 0 || n <= 0 || k <= 0 || k % 64) return 0;
  if (k == 64) return 64;
  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  const long long tiles_m = static_cast<long long>(n) * (h / rows);
  // Rounds of tiles on the device times the time of one tile: a K block costs the issuing thread about the same
  // whatever the tile's width up to 128 columns and a quarter more at 256 (then the tensor pipe is the longer
  // pole), and wider tiles re-read the input pixels less often.
  const int widths[3] = {256, 128, 64};
  const double unit_time[3] = {1.25, 1.05, 1.0};
  int best = 64;
  double best_cost = 1e30;
  for (int i = 0; i < 3; i++) {
    if (k % widths[i]) continue;
    const long long units = tiles_m * (k / widths[i]);
    const double cost = static_cast<double>((units + sms - 1) / sms) * unit_time[i];
    if (cost < best_cost - 1e-9) { best_cost = cost; best = widths[i]; }
  }
  return best;
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
  const int rows = cusync_conv2d_tile_rows_hw(d.h, d.w);
  if (d.c % 64 || d.k % 64 || rows == 0) return CUSYNC_ERROR_UNSUPPORTED;
  if (!aligned16(d.x) || !aligned16(d.filter) || !aligned16(d.y)) return CUSYNC_ERROR_UNSUPPORTED;

  cusync_gemm_plan* pl = new (std::nothrow) cusync_gemm_plan();
  if (!pl) return CUSYNC_ERROR_CUDA;
  std::memset(pl, 0, sizeof(*pl));
  pl->tile_n = cusync_conv2d_default_tile_n(d.n, d.h, d.w, d.c, d.k);
  pl->split_k = 1;
  switch (pl->tile_n) {
    case 256: pl->kernel = KernelEntry{cusync_gemm_kernel<256, false, true>, Cfg<256, false>::kSmemBytes}; break;
    case 128: pl->kernel = KernelEntry{cusync_gemm_kernel<128, false, true>, Cfg<128, false>::kSmemBytes}; break;
    default:  pl->tile_n = 64;
              pl->kernel = KernelEntry{cusync_gemm_kernel<64, false, true>, Cfg<64, false>::kSmemBytes}; break;
  }
  GemmParams& p = pl->params;
  p.m = d.n * d.h * d.w; p.n = d.k; p.k = 9 * d.c;
  p.d = d.y; p.ldd = d.k;
  p.tiles_n = d.k / pl->tile_n;
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
  if (rc == CUSYNC_SUCCESS)
    rc = check_stage_policies(view, static_cast<uint32_t>(rows * d.w), static_cast<uint32_t>(pl->tile_n),
                              static_cast<uint32_t>(9 * d.c), true);
  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  const uint32_t cap = d.max_ctas > 0 ? static_cast<uint32_t>(d.max_ctas) : static_cast<uint32_t>(sms);
  pl->num_ctas = static_cast<uint32_t>(p.num_tiles) < cap ? static_cast<uint32_t>(p.num_tiles) : cap;
  // The slab kernel serves the 64 -> 64 channel layer when a tile's padded rows still fit the 128-row MMA and
  // the consumer side waits once per tile (no input policy, or Conv2DTileSync over a one-column producer grid).
  const bool slab_ok = d.c == 64 && d.k == 64 && rows * (d.w + 2) <= kBlockM && d.w + 2 <= 256 &&
                       (view.in_policy.kind == CUSYNC_POLICY_NOSYNC ||
                        (view.in_policy.kind == CUSYNC_POLICY_CONV2DTILESYNC && view.prod_grid.x == 1));
  if (rc == CUSYNC_SUCCESS && (d.kernel < 0 || d.kernel > 2)) rc = CUSYNC_ERROR_INVALID_ARGUMENT;
  if (rc == CUSYNC_SUCCESS && d.kernel == 2 && !slab_ok) rc = CUSYNC_ERROR_UNSUPPORTED;
  pl->conv_slab = rc == CUSYNC_SUCCESS && slab_ok && d.kernel != 1;
  if (rc == CUSYNC_SUCCESS) {
    bool ok = (pl->conv_slab ? make_map_nhwc(&pl->tmA, d.x, d.n, d.h, d.w, d.c, static_cast<uint32_t>(rows + 2),
                                             static_cast<uint32_t>(d.w + 2))
                             : make_map_nhwc(&pl->tmA, d.x, d.n, d.h, d.w, d.c, static_cast<uint32_t>(rows))) &&
              make_map(&pl->tmB, d.filter, d.k, 9ull * d.c, 9ull * d.c, kBlockK, static_cast<uint32_t>(pl->tile_n));
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
int cusync_conv2d_run_dependent(cusync_conv2d_plan_t* pl, cusync_stream_t stream) {
  return cusync_gemm_run_dependent(pl, stream);
}
uint32_t cusync_conv2d_plan_num_ctas(const cusync_conv2d_plan_t* pl) { return pl ? pl->num_ctas : 0; }

}  // extern "C"

