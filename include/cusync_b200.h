/*
 * cusync_b200 -- C ABI of the B200-native CuSync library (libcusync_b200.so).
 *
 * Plain C: opaque handles, POD descriptors, int status codes, caller-owned
 * device memory, explicit streams.  The C++ template API in <cusync/cusync.h>
 * (CuStage, CuSync, the sync policies, tile orders) is a thin layer over these
 * entry points, and so is any foreign-language binding.
 *
 * Every entry point cites the interface of microsoft/cusync it replaces
 * (paths relative to that project's root).
 */
#ifndef CUSYNC_B200_H
#define CUSYNC_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32)
  #define CUSYNC_API
#else
  #define CUSYNC_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* cusync_stream_t;   /* a cudaStream_t */

typedef struct cusync_dim3 { uint32_t x, y, z; } cusync_dim3_t;

/* Status codes.  The first six keep the reference's enumerator order
 * (src/include/cusync/cusync.h:46-53): success is 5, not 0. */
enum {
  CUSYNC_ERROR_NOT_PRODUCER = 0,
  CUSYNC_ERROR_NOT_CONSUMER = 1,
  CUSYNC_ERROR_NOT_INITIALIZED = 2,
  CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX = 3,
  CUSYNC_ERROR_CUDA = 4,
  CUSYNC_SUCCESS = 5,
  /* additions */
  CUSYNC_ERROR_TIMEOUT = 6,            /* a bounded device-side wait gave up */
  CUSYNC_ERROR_INVALID_ARGUMENT = 7,
  CUSYNC_ERROR_UNSUPPORTED = 8,        /* shape/alignment outside what the kernels implement */
  CUSYNC_ERROR_EXCEEDS_STATIC_SCRATCH = 9  /* cusync_gemm_run_noalloc: more output tiles than its fixed scratch holds */
};

/* Optimizations bit set (src/include/cusync/cusync.h:69-75). */
enum {
  CUSYNC_OPT_NONE = 0,
  CUSYNC_OPT_NO_ATOMIC_ADD = 1,
  CUSYNC_OPT_AVOID_WAIT_KERNEL = 2,
  CUSYNC_OPT_AVOID_CUSTOM_ORDER = 4,
  CUSYNC_OPT_REORDER_TILE_LOADS = 8,
  CUSYNC_OPT_STREAM_WAIT = 16      /* addition: invokeWaitKernel becomes a stream memory operation
                                      (cuStreamWaitValue32 on the "blocks started" word) instead of a kernel launch:
                                      same condition, no launch, no SM, but no timeout record either */
};

/* Tile orders (src/include/cusync/tile-orders.h:50-76). */
enum { CUSYNC_ORDER_IDENTITY = 0, CUSYNC_ORDER_TRANSPOSE_XY = 1, CUSYNC_ORDER_GROUPED_ROWS = 2 };
/* Addition for L2 locality on large-L2 parts: blocks are taken in groups of `rows` consecutive grid rows
 * (M tiles); inside a group the row index runs fastest, then the column (N tile).  Blocks that run at the
 * same time then share few weight (B) tiles and a bounded set of activation (A) row panels.  As a stage's
 * schedule order only; a policy's `order` field stays IDENTITY or TRANSPOSE_XY. */
#define CUSYNC_ORDER_GROUPED(rows) (CUSYNC_ORDER_GROUPED_ROWS | ((rows) << 8))

/* Sync policies as data.  NOSYNC/ROWSYNC/TILESYNC/CONV2DTILESYNC:
 * src/include/cusync/policies.h:18-210.  STRIDEDTILESYNC: StridedSync,
 * src/ml-bench/transformer/mlp.cu:76-101.  CONSECUTIVETILESYNC:
 * ConsecutiveSync, src/ml-bench/transformer/attention.cu:51-70. */
enum {
  CUSYNC_POLICY_NOSYNC = 0,
  CUSYNC_POLICY_ROWSYNC = 1,
  CUSYNC_POLICY_TILESYNC = 2,
  CUSYNC_POLICY_STRIDEDTILESYNC = 3,
  CUSYNC_POLICY_CONV2DTILESYNC = 4,
  CUSYNC_POLICY_CONSECUTIVETILESYNC = 5,
  CUSYNC_POLICY_CUSTOM = 6   /* user-written policy class; evaluated only by code compiled against <cusync/cusync.h> */
};

typedef struct cusync_policy {
  int32_t  kind;        /* CUSYNC_POLICY_* */
  int32_t  order;       /* CUSYNC_ORDER_* used to linearise the semaphore index */
  uint32_t tile_m;      /* TileM template argument of the reference policy */
  uint32_t tile_n;      /* TileN template argument */
  uint32_t wait_value;  /* waitValue_ (ROW / TILE / CONV2D) */
  uint32_t post_value;  /* postValue_ (ROW / TILE / CONV2D) */
  uint32_t p0;          /* STRIDED: GridN, CONV2D: R*S, CONSECUTIVE: H */
  uint32_t p1;          /* STRIDED: stride */
} cusync_policy_t;

/* Record a bounded wait leaves behind when it gives up. */
typedef struct cusync_status {
  uint32_t code;        /* 0 = nothing recorded, else CUSYNC_ERROR_TIMEOUT */
  uint32_t where;       /* 1 semaphore wait, 2 pipeline barrier, 3 wait kernel */
  uint32_t tile_x, tile_y, tile_z;
  uint32_t sem_index;
  uint32_t seen;
  uint32_t expected;
} cusync_status_t;

/* What a kernel needs of a stage, passed by value in its parameters -- the
 * role the by-value CuStage copy plays in the reference
 * (gemm/device/cusyncgemm.h:352 `params_.custage`). */
typedef struct cusync_stage_view {
  cusync_dim3_t   grid;         /* tiles of this stage: (N tiles, M tiles, split-K) */
  cusync_dim3_t   prod_grid;    /* the producer's grid, set by cusync_stage_link */
  cusync_dim3_t   tile_size;
  uint32_t        iter;         /* run counter, starts at 1 */
  int32_t         opts;
  int32_t         order;
  int32_t         reserved;
  cusync_policy_t in_policy;
  cusync_policy_t out_policy;
  cusync_dim3_t*  tile_order;   /* [numTiles] schedule buffer */
  uint32_t*       tile_counter; /* ticket counter for tile_order */
  uint32_t*       started;      /* [3]: [0] = iter stored by block 0 (reference protocol),
                                   [1] = blocks started so far, all runs (persistent kernels),
                                   [2] = blocks finished so far, all runs: a producer block adds 1 after its last post */
  uint32_t*       sems_post;    /* semaphores this stage posts to (producer) */
  uint32_t*       sems_wait;    /* semaphores this stage waits on (consumer) */
  uint32_t*       status;       /* device copy of cusync_status_t */
  uint64_t        timeout_ns;   /* bound of every device-side spin */
  /* Consumer: the producer's "blocks finished" word and the count it reaches when the producer kernel of THIS run
   * has finished altogether (cusync_stage_note_launch of the producer writes it into its linked consumers).  A
   * consumer block that finds the count reached need not look at the semaphores of its tiles any more: everything
   * it could wait for is there.  Null when the producer's launch of this run was not noted before the consumer's
   * view was taken (the consumer then checks every tile, as the reference does).  No counterpart. */
  const uint32_t* prod_finished;
  uint32_t        prod_finish_target;
  uint32_t        reserved2;
} cusync_stage_view_t;

typedef struct cusync_stage cusync_stage_t;

/* ---- stages ------------------------------------------------------------- */

/* CuStage::CuStage(grid, tileSize, inputPolicy, outputPolicy) incl.
 * buildScheduleBuffer (cusync.h:125-157,176-198).  Allocates the schedule
 * buffer, the ticket counter, and for a producer the semaphore array (one per
 * tile, zeroed) and the started words.  Returns
 * CUSYNC_ERROR_INVALID_LINEAR_BLOCK_INDEX when the order is not a bijection
 * (the reference computes this error and drops it, cusync.h:184). */
CUSYNC_API int cusync_stage_create(cusync_stage_t** out, cusync_dim3_t grid, cusync_dim3_t tile_size,
                        int order, const cusync_policy_t* in_policy,
                        const cusync_policy_t* out_policy, int opts);

/* The reference never frees a stage's device memory (no destructor). */
CUSYNC_API int cusync_stage_destroy(cusync_stage_t* stage);

/* CuSync::setProducerConsumerPair (cusync.h:287-299). */
CUSYNC_API int cusync_stage_link(cusync_stage_t* producer, cusync_stage_t* consumer);

/* CuStage::incrementIter (cusync.h:212).  The handle is the single owner of
 * `iter`; views taken afterwards carry the new value. */
CUSYNC_API int cusync_stage_increment_iter(cusync_stage_t* stage);

/* Sets the run counter outright.  The C++ CuStage keeps a counter in every
 * copy (as the reference does) and mirrors it here, so that incrementing the
 * host object and the by-value copy inside a kernel handle (mlp.cu:709-712)
 * does not count twice. */
CUSYNC_API int cusync_stage_set_iter(cusync_stage_t* stage, uint32_t iter);

/* Replaces the schedule buffer (user-defined tile orders of the C++ API). */
CUSYNC_API int cusync_stage_write_tile_order(cusync_stage_t* stage, const cusync_dim3_t* order, uint32_t count);

/* No counterpart: zero the semaphores, ticket and started words and set
 * iter = 1, so a stage can be reused after an error. */
CUSYNC_API int cusync_stage_reset(cusync_stage_t* stage, cusync_stream_t stream);

/* The by-value copy a kernel takes (cusyncgemm.h:352). */
CUSYNC_API int cusync_stage_get_view(const cusync_stage_t* stage, cusync_stage_view_t* out);

/* Bound, in nanoseconds, of every device-side spin of kernels using this
 * stage (the reference spins forever, cusync_device_defs.h:41-43). */
CUSYNC_API int cusync_stage_set_timeout_ns(cusync_stage_t* stage, uint64_t ns);

/* CuStage::invokeWaitKernel (cusync.h:203-209): enqueue on `stream` a
 * one-thread kernel that returns once this producer's kernel has started. */
CUSYNC_API int cusync_stage_invoke_wait_kernel(cusync_stage_t* producer, cusync_stream_t stream);

/* Tells the stage that a persistent kernel of `num_blocks` blocks was
 * launched for the current run; the next wait kernel then waits until all of
 * them are resident instead of only block 0. */
CUSYNC_API int cusync_stage_note_launch(cusync_stage_t* stage, uint32_t num_blocks);

/* cusync::invokeWaitKernel(uint32_t*, uint32_t, cudaStream_t)
 * (src/include/cusync/wait-kernel.h:10, src/cusync.cu:11-25).  `status` may
 * be NULL; `timeout_ns` 0 selects the default bound. */
CUSYNC_API int cusync_wait_kernel(uint32_t* semaphore, uint32_t given_value, cusync_stream_t stream,
                       uint32_t* status, uint64_t timeout_ns);

/* The same for a contiguous range of semaphores: the kernel ends when each of `count` semaphores has reached
 * `given_value`.  No counterpart in the reference; it is what lets a stream of another library (an NCCL
 * all-reduce of some rows of the output) start behind the tiles it depends on instead of behind the kernel. */
CUSYNC_API int cusync_wait_kernel_range(uint32_t* semaphores, uint32_t count, uint32_t given_value,
                                        cusync_stream_t stream, uint32_t* status, uint64_t timeout_ns);

/* The same wait without a kernel (the driver's stream memory operations, cuStreamWaitValue32 with GEQ): `stream`
 * holds until each of `count` semaphores has reached `value`.  A kernel needs room on an SM, and while the
 * persistent GEMM blocks are resident there is none, so a wait kernel enqueued behind them starts only when
 * they retire; this form does not depend on that.  Unbounded, no timeout record: wait only for values that
 * work ALREADY SUBMITTED will write (streams can share a hardware queue, and a wait at its head keeps everything
 * submitted later to that queue from being issued).  More than one semaphore goes to the stream as one batched
 * operation (cuStreamBatchMemOp, up to 64 per batch) where the driver offers it.  No counterpart. */
CUSYNC_API int cusync_stream_wait_values(uint32_t* semaphores, uint32_t count, uint32_t value, cusync_stream_t stream);
/* The posting counterpart (cuStreamWriteValue32): `stream` stores `value` into each of `count` semaphores once
 * everything enqueued on it before has completed - the way something that is not a kernel of this library (a
 * host-to-device copy, another library's kernel) acts as a producer stage.  A store, not an add: one poster per
 * semaphore, values that only grow (the NoAtomicAdd protocol, policies of mlp.cu:9-14).  No counterpart. */
CUSYNC_API int cusync_stream_write_values(uint32_t* semaphores, uint32_t count, uint32_t value, cusync_stream_t stream);

/* Test access, the role of the reference's friend class CuSyncTest
 * (tests/cusync-test.h:8-44): copy the schedule buffer / the producer's
 * semaphores / the timeout record to the host (synchronous). */
CUSYNC_API int cusync_stage_read_tile_order(const cusync_stage_t* stage, cusync_dim3_t* out, uint32_t count);
CUSYNC_API int cusync_stage_read_semaphores(const cusync_stage_t* stage, uint32_t* out, uint32_t count);
CUSYNC_API int cusync_stage_read_status(const cusync_stage_t* stage, cusync_status_t* out);
CUSYNC_API uint32_t cusync_stage_num_tiles(const cusync_stage_t* stage);
CUSYNC_API uint32_t cusync_stage_iter(const cusync_stage_t* stage);

/* ---- GEMM --------------------------------------------------------------- */

enum { CUSYNC_EPILOGUE_NONE = 0, CUSYNC_EPILOGUE_GELU_ERF = 1, CUSYNC_EPILOGUE_RELU = 2,
       CUSYNC_EPILOGUE_SILU_MUL_DUAL = 3 };
enum { CUSYNC_B_ROW_MAJOR_KN = 0, CUSYNC_B_ROW_MAJOR_NK = 1 };

/* D[m,n] = epilogue(A[m,k] * B[k,n]); fp16 operands, fp32 accumulate, fp16
 * out.  Replaces cutlass::gemm::device::CuSyncGemm<...>::Arguments
 * (gemm/device/cusyncgemm.h:293-350): custage, problem_size, ref_A, ref_B,
 * ref_D.  alpha = 1 and beta = 0 as in every reference driver
 * (src/ml-bench/transformer/mlp.cu:239-240); split-K is 1. */
typedef struct cusync_gemm_desc {
  int32_t m, n, k;
  const void* a; int64_t lda;      /* row-major [m,k] */
  const void* b; int64_t ldb;      /* row-major [k,n] (b_layout 0) or [n,k] (b_layout 1) */
  const void* b2;                  /* second B of CUSYNC_EPILOGUE_SILU_MUL_DUAL, same layout/ldb */
  void* d; int64_t ldd;            /* row-major [m,n] */
  int32_t b_layout;
  int32_t epilogue;
  int32_t tile_n;                  /* 0 = choose; else 64, 128, 192 or 256.  Tile M is 128. */
  int32_t max_ctas;                /* 0 = one per SM */
  int32_t split_k;                 /* K slices per output tile (the stage grid's z): 0 = choose, 1 = none.  Slices add
                                      their parts into an fp32 workspace owned by the plan; the last one to arrive applies
                                      the epilogue, stores and posts (serial split-K of gemm/kernel/cusyncgemm.h:374-392,
                                      without its ordering of the slices).  Not with CUSYNC_EPILOGUE_SILU_MUL_DUAL. */
  int32_t cta_pair;                /* 0 = choose; 1 = one CTA per 128 x tile_n tile; 2 = CTA pairs (tcgen05
                                      cta_group::2): two CTAs share a 256 x 256 tile, each loading half of B
                                      (tile_n 256), or, for CUSYNC_EPILOGUE_SILU_MUL_DUAL, a 256 x 128 output tile whose
                                      MMA is [A B | A B2], one CTA loading B and the other B2 (tile_n 128).
                                      Semaphores stay per 128-row tile. */
  int32_t tail_split;              /* CTA-pair kernel without uniform split-K: K slices for the tiles of the last,
                                      partial wave, so that the tail occupies every SM pair (the remedy the reference
                                      gets from Stream-K, src/ml-bench/transformer/mlp.cu:137-207).  0 = choose
                                      (none for a single launch: it measured slower; the MLP driver's table uses it
                                      inside the one-grid layer), 1 = none, 2..16 = forced.  The stage grid is
                                      unchanged (z = 1); a split tile posts once, from the pair that adds its last
                                      slice.  Not with CUSYNC_EPILOGUE_SILU_MUL_DUAL (CUSYNC_ERROR_UNSUPPORTED). */
  cusync_stage_t* stage;           /* NULL = no tile synchronisation (stream-ordered use) */
  /* A B operand that is itself the output of an earlier stage of the chain (the K^T and V operands of the
   * attention GEMMs S = Q K^T and O = S V, src/ml-bench/transformer/attention.cu:272-276, whose policies wait for
   * the A operand only).  b_stage is that producer stage (NULL = B holds weights, never waited for); rows
   * [128 r, 128 r + 128) of the B matrix as given (n rows of a [n,k] B, k rows of a [k,n] B) are complete when the
   * producer's semaphore b_sem_first + r * b_sem_stride has reached b_sem_value times the run counter.  CTA-pair
   * kernel only (else CUSYNC_ERROR_UNSUPPORTED); not with K slices. */
  cusync_stage_t* b_stage;
  uint32_t b_sem_first, b_sem_stride, b_sem_value;
} cusync_gemm_desc_t;

typedef struct cusync_gemm_plan cusync_gemm_plan_t;

/* Tile shape the library would pick for a GEMM (tile M is always 128); lets
 * the caller size the CuStage grid the way
 * CuSyncGemmHorizontalThreadblockSwizzle::get_tiled_shape does
 * (gemm/threadblock/cusync_threadblock_swizzle.h:12-54). */
CUSYNC_API int cusync_gemm_default_tile_n(int32_t m, int32_t n, int32_t k, int32_t epilogue);
/* K slices the library would pick (get_tiled_shape's third component); tile_n 0 and cta_pair 0 = its own choice. */
CUSYNC_API int cusync_gemm_default_split_k(int32_t m, int32_t n, int32_t k, int32_t epilogue, int32_t tile_n,
                                           int32_t cta_pair);

/* can_implement + get_workspace_size + initialize
 * (gemm/device/cusyncgemm.h:364-456). */
CUSYNC_API int cusync_gemm_plan_create(cusync_gemm_plan_t** out, const cusync_gemm_desc_t* desc);
CUSYNC_API int cusync_gemm_plan_destroy(cusync_gemm_plan_t* plan);
/* update / updateA / updateC / updateD (gemm/device/cusyncgemm.h:459-494). */
CUSYNC_API int cusync_gemm_plan_update(cusync_gemm_plan_t* plan, const void* a, const void* b,
                            const void* b2, void* d);
/* run(bool overlap, int*, cudaStream_t) (gemm/device/cusyncgemm.h:525-563). */
CUSYNC_API int cusync_gemm_run(cusync_gemm_plan_t* plan, cusync_stream_t stream);
/* The same launch as a programmatic dependent of the kernel ahead of it in `stream` (launch attribute
 * "programmatic stream serialization"): the GEMM becomes resident as soon as EVERY block of that kernel is resident
 * or done, not when it has finished, and is ordered against its producer's writes by its semaphore waits alone.
 * This is what the reference obtains with a second stream and CuStage::invokeWaitKernel (cusync.h:277-283,
 * waitKernel in cusync_device_defs.h:78-83) - the consumer must not take the SMs before the producer's blocks
 * have them - done by the launch hardware: one stream, no polling kernel, no events, and the consumer's launch
 * latency and prologue run under the producer.  The plan must be a consumer (an input policy, or b_stage), else
 * CUSYNC_ERROR_NOT_CONSUMER; the kernel ahead must be one of this library's GEMM, convolution or attention
 * kernels (they release their dependents as soon as they run; behind any other kernel the launch is stream-ordered). */
CUSYNC_API int cusync_gemm_run_dependent(cusync_gemm_plan_t* plan, cusync_stream_t stream);
/* Two dependent GEMMs launched as ONE persistent grid: the blocks draw the work units of `first`, then those of
 * `second`, from one ticket counter, so a block that finds no unit of the first GEMM left goes straight on to
 * units of the second (whose waits on the first's semaphores are the usual ones) instead of idling until a second
 * launch can become resident.  Stages, policies, semaphore counts and results are those of two cusync_gemm_run
 * calls; no wait kernel is needed.  The second plan's stage should be the consumer of the first's (or wait for
 * nothing).  Both plans must run the CTA-pair kernel (cusync_gemm_chain_supported), else
 * CUSYNC_ERROR_UNSUPPORTED.  The reference always launches one kernel per GEMM
 * (src/ml-bench/transformer/mlp.cu:691-712); this is what its overlap of the producer's last wave turns into
 * when every kernel is persistent and holds a whole SM per block. */
CUSYNC_API int cusync_gemm_run_chain(cusync_gemm_plan_t* first, cusync_gemm_plan_t* second, cusync_stream_t stream);
CUSYNC_API int cusync_gemm_chain_supported(const cusync_gemm_plan_t* first, const cusync_gemm_plan_t* second);
/* Loads the one-grid kernel ahead of its first run (a first launch that has to load its kernel can stall behind
 * kernels already running on the device).  Optional; cusync_gemm_run_chain does it otherwise. */
CUSYNC_API int cusync_gemm_chain_prepare(void);
/* K slices the plan uses for the tiles of its last partial wave (1 = none). */
CUSYNC_API int cusync_gemm_plan_tail_split(const cusync_gemm_plan_t* plan);
/* Allocation-free GEMM.  It has no counterpart in the reference.
 *
 * For callers that must not allocate device memory at the point of the call: a plug-in inside a
 * serving runtime that owns the whole device through its own arena and forbids cudaMalloc, a
 * latency-critical loop where cudaMalloc / cudaFree would serialise against every stream of the
 * device, a process already at its memory limit.  cusync_gemm_plan_create allocates a stage
 * (schedule buffer, ticket counter, status words) with cudaMalloc; this entry point runs the same
 * kernel, without tile synchronisation (desc->stage must be NULL), on scratch that lives in a fixed
 * array inside the library image.  It calls no cudaMalloc, cudaFree or other allocating routine;
 * inputs and the output are still the caller's buffers.
 *
 * Limit: at most 8192 output tiles per call (ceil(m / 128) * ceil(n / tile_n)); a larger problem is
 * refused with CUSYNC_ERROR_EXCEEDS_STATIC_SCRATCH and nothing is launched.  The array costs about
 * 97 KB of device memory on every GPU that loads the library, for the life of the process.
 *
 * The first call on each device looks up the array's device address (with that device current) and
 * caches it; make that first call outside any stream capture.  All calls on a device share the one
 * array, which keeps the last call's contents: each call re-arms it on `stream` before its kernel,
 * so calls issued to one stream are safe back to back, while calls that can overlap on the GPU
 * (different streams, no dependency) race on it and must be serialised by the caller.
 *
 * It runs the one-CTA-per-tile kernel without K slices: desc->split_k > 1, desc->cta_pair == 2 and
 * desc->tail_split > 1 are refused with CUSYNC_ERROR_UNSUPPORTED (those forms need a workspace or a schedule
 * that only the plan-based path allocates); 0 and 1 are accepted. */
CUSYNC_API int cusync_gemm_run_noalloc(const cusync_gemm_desc_t* desc, cusync_stream_t stream);
/* The timeout record of the most recent cusync_gemm_run_noalloc on the current device (it lives in the same
 * fixed array, so no stage handle gives access to it): code 0 when every bounded wait inside the kernel
 * completed.  A synchronous device-to-host copy of 32 bytes; allocates nothing.  No counterpart in the reference. */
CUSYNC_API int cusync_gemm_noalloc_read_status(cusync_status_t* out);

/* Optional per-tile timeline, the only profiling hook beyond CUDA events: with a device buffer of
 * 8 * capacity_tiles 64-bit words set, every tile writes, at index 8 * ticket (CTA-pair kernel:
 * 8 * (2 * ticket + rank)),
 * {globaltimer at the ticket draw, at the end of its MMAs, after its stores and post,
 *  (SM id << 32) | block index, SM cycles the MMA thread waited for operands, SM cycles the loader
 *  waited for a free ring slot, SM cycles of the tile in the MMA thread, of which waiting for a free
 *  accumulator}.  (The 64 -> 64 channel convolution kernel packs into the sixth word the loader's cycles for the
 *  tile instead, 12 bits each from bit 0: dependencies, schedule slot, free slab, TMA issue.)
 *  NULL switches it off (the default).  No counterpart in the reference. */
CUSYNC_API int cusync_gemm_plan_set_trace(cusync_gemm_plan_t* plan, void* device_buffer, uint32_t capacity_tiles);
/* Blocks the launch uses (persistent grid). */
CUSYNC_API uint32_t cusync_gemm_plan_num_ctas(const cusync_gemm_plan_t* plan);

/* ---- 3x3 convolution ---------------------------------------------------- */

/* y[n,h,w,k] = epilogue(conv(x[n,h,w,c], filter[k,r,s,c])), NHWC / KRSC fp16, fp32 accumulate: the forward
 * convolution of cutlass::conv::device::CuSyncImplicitGemmConvolution
 * (conv/device/cusyncimplicit_gemm_convolution.h:51-319) as the reference's resnet.cu / vgg.cu drive it.
 * Implicit GEMM [n*h*w, 9c] x [9c, k]: the K walk is channel-chunk outermost, filter tap innermost, as
 * Conv2DTileSync assumes (policies.h:160-210).  An M tile is cusync_conv2d_tile_rows_hw(h, w) whole image rows
 * (w <= 128), an N tile cusync_conv2d_default_tile_n(...) output channels; the stage grid is
 * (k / tile_n, n * h / rows, 1).  A consumer
 * convolution also waits for the producer tiles holding the image rows just above and below its own.
 * Supported: r = s = 3, stride 1, pad 1, c and k multiples of 64. */
typedef struct cusync_conv2d_desc {
  int32_t n, h, w, c, k;
  int32_t r, s, stride, pad;
  const void* x; const void* filter; void* y;
  int32_t epilogue;                /* CUSYNC_EPILOGUE_NONE or CUSYNC_EPILOGUE_RELU */
  int32_t max_ctas;
  int32_t kernel;                  /* 0 = choose; 1 = the general implicit-GEMM kernel; 2 = the slab kernel (c = k = 64,
                                      resident filter, one input slab per tile), CUSYNC_ERROR_UNSUPPORTED where it
                                      does not apply */
  cusync_stage_t* stage;           /* NULL = no tile synchronisation */
} cusync_conv2d_desc_t;

typedef struct cusync_gemm_plan cusync_conv2d_plan_t;

CUSYNC_API int cusync_conv2d_tile_rows(int32_t w);          /* floor(128 / w): the most image rows a tile can hold */
/* Image rows per M tile for an h x w image: the largest divisor of h that is at most floor(128 / w), so that
 * tiles never straddle two images (56 x 56: 2; 28 x 28: 4; 14 x 14: 7; 7 x 7: 7, the layer sizes of
 * src/ml-bench/volta_conv2d/eval_resnet.py:12-17).  0 when w > 128. */
CUSYNC_API int cusync_conv2d_tile_rows_hw(int32_t h, int32_t w);
/* Output channels per N tile the library picks for a layer: 64, 128 or 256 (a divisor of k), by the rounds of
 * tiles the layer makes on the device; 64 for k = 64.  The stage grid is (k / tile_n, n * h / rows, 1) and the
 * policies of a chain take TileN = tile_n (the reference fixes its tile shape at compile time,
 * src/ml-bench/volta_conv2d/resnet.cu:95-105, and tunes it per layer in eval_resnet.py:18-60). */
CUSYNC_API int cusync_conv2d_default_tile_n(int32_t n, int32_t h, int32_t w, int32_t c, int32_t k);
/* can_implement + initialize (conv/device/cusyncimplicit_gemm_convolution.h:100-265). */
CUSYNC_API int cusync_conv2d_plan_create(cusync_conv2d_plan_t** out, const cusync_conv2d_desc_t* desc);
CUSYNC_API int cusync_conv2d_plan_destroy(cusync_conv2d_plan_t* plan);
/* run(stream) (conv/device/cusyncimplicit_gemm_convolution.h:283-297). */
CUSYNC_API int cusync_conv2d_run(cusync_conv2d_plan_t* plan, cusync_stream_t stream);
/* As cusync_gemm_run_dependent: the convolution starts once every block of the kernel ahead of it is resident. */
CUSYNC_API int cusync_conv2d_run_dependent(cusync_conv2d_plan_t* plan, cusync_stream_t stream);
CUSYNC_API uint32_t cusync_conv2d_plan_num_ctas(const cusync_conv2d_plan_t* plan);

/* A chain of 3x3 convolutions with equal channel counts, the workload of
 * src/ml-bench/volta_conv2d/resnet.cu (two convolutions) and vgg.cu (up to four):
 * activations[0] -> conv(filters[0]) -> activations[1] -> ... -> activations[num_convs], NHWC fp16 on the device,
 * caller-owned; ReLU after every convolution when `relu` is set.  Stage i posts TileSync<rows * w, tile_n> and stage
 * i + 1 waits with Conv2DTileSync<3, 3, rows * w, tile_n> (resnet.cu:107-116). */
typedef struct cusync_conv_chain_desc {
  int32_t num_convs;               /* 2..8 */
  int32_t n, h, w, channels;
  int32_t relu;
  int32_t max_ctas;                /* blocks per convolution; 0 = choose: one per SM, or one per two SMs for each
                                      synchronised convolution of a chain of three or more 64-channel convolutions
                                      (two adjacent stages resident together) */
  const void* const* filters;      /* [num_convs] pointers to [channels, 3, 3, channels] */
  void* const* activations;        /* [num_convs + 1] pointers to [n, h, w, channels] */
} cusync_conv_chain_desc_t;

typedef struct cusync_conv_chain cusync_conv_chain_t;

/* Stage construction + setProducerConsumerPair + every convolution's initialisation (resnet.cu:659-700). */
CUSYNC_API int cusync_conv_chain_create(cusync_conv_chain_t** out, const cusync_conv_chain_desc_t* desc);
CUSYNC_API int cusync_conv_chain_destroy(cusync_conv_chain_t* chain);
/* runBaseline, one iteration: the convolutions back to back on one stream, no tile synchronisation
 * (resnet.cu:461-520). */
CUSYNC_API int cusync_conv_chain_run_stream_ordered(cusync_conv_chain_t* chain, cusync_stream_t stream);
/* runCuSync, one iteration: convolution i on streams[i], each dependent one behind a wait kernel unless all
 * stages fit on the device at once, then incrementIter on every stage (resnet.cu:560-590).  streams: [num_convs]. */
CUSYNC_API int cusync_conv_chain_run_cusync(cusync_conv_chain_t* chain, const cusync_stream_t* streams);
/* The same iteration on ONE stream: every dependent convolution is launched with cusync_conv2d_run_dependent, so
 * it becomes resident once all blocks of the convolution ahead of it are, with no wait kernel, stream or event
 * between them.  Same stages, semaphore counts and results as run_cusync. */
CUSYNC_API int cusync_conv_chain_run_dependent(cusync_conv_chain_t* chain, cusync_stream_t stream);
/* The same work in a form that can be recorded once and replayed (a CUDA graph captured on streams[0]; no
 * counterpart in the reference): resets every stage (semaphores zero, iteration 1) on streams[0], makes the other
 * streams wait for the resets, then launches as run_cusync does, without incrementIter.  The caller joins
 * streams[1..] back into streams[0] before ending a capture.  These kernels run for tens of microseconds, less
 * than the host needs to submit three launches, so replaying one graph is what keeps the GPU fed. */
CUSYNC_API int cusync_conv_chain_run_cusync_replayable(cusync_conv_chain_t* chain, const cusync_stream_t* streams);
/* Stage handle of convolution `which`, for inspection. */
CUSYNC_API cusync_stage_t* cusync_conv_chain_stage(cusync_conv_chain_t* chain, int which);
/* 1 when run_cusync launches wait kernels, 0 when every stage fits on the device at once (AvoidWaitKernel). */
CUSYNC_API int cusync_conv_chain_uses_wait_kernels(const cusync_conv_chain_t* chain);

/* ---- decode attention (a middle stage) ---------------------------------- */

/* One query token per batch row attends, per head, over `seq` cached keys/values plus its own new key/value;
 * scores scaled by 1/sqrt(head_dim), softmax in fp32, fp16 out.  It stands where the reference's attention
 * chain has its two un-normalised GEMMs S = Q K^T and O = S V (src/ml-bench/transformer/attention.cu:105-118,
 * 706-833): a stage that both waits (on the Q, K and V thirds of the QKV projection's row panel, ConsecutiveSync
 * attention.cu:51-70) and posts (RowSync on its output's row panel, published when every row and head of the
 * panel is written; use wait value 1 and post value 1).
 * qkv[batch, 3 * heads * 128] = Q | K | V (row pitch ld_qkv), caches [batch, seq, heads, 128], out[batch, heads * 128].
 * The stage grid is (heads, batch, kv_splits).  head_dim must be 128. */
typedef struct cusync_attn_desc {
  int32_t batch, seq, heads, head_dim;
  const void* qkv; int64_t ld_qkv;
  const void* k_cache; const void* v_cache;
  void* out; int64_t ld_out;
  int32_t kv_splits;               /* blocks per (row, head) over the key range: 0 = choose */
  cusync_stage_t* stage;           /* NULL = no tile synchronisation */
} cusync_attn_desc_t;

typedef struct cusync_attn_plan cusync_attn_plan_t;

CUSYNC_API int cusync_attn_default_splits(int32_t batch, int32_t seq, int32_t heads);
CUSYNC_API int cusync_attn_plan_create(cusync_attn_plan_t** out, const cusync_attn_desc_t* desc);
CUSYNC_API int cusync_attn_plan_destroy(cusync_attn_plan_t* plan);
CUSYNC_API int cusync_attn_plan_splits(const cusync_attn_plan_t* plan);
CUSYNC_API int cusync_attn_run(cusync_attn_plan_t* plan, cusync_stream_t stream);
/* As cusync_gemm_run_dependent: the attention kernel starts once every block of the kernel ahead of it is resident. */
CUSYNC_API int cusync_attn_run_dependent(cusync_attn_plan_t* plan, cusync_stream_t stream);

/* The whole attention block of one tensor-parallel shard, the workload of src/ml-bench/transformer/attention.cu:
 * qkv = x * w_qkv; attn_out = attention(qkv, caches); y = attn_out * w_o.  x[batch, hidden], w_qkv[hidden, 3 * heads
 * * 128], w_o[heads * 128, out_features], row-major fp16 on the device, caller-owned, as are the intermediates
 * qkv[batch, 3 * heads * 128] and attn_out[batch, heads * 128].  model_hidden is the H of ConsecutiveSync<H, ...>
 * (attention.cu:105-110): the un-sharded hidden size. */
typedef struct cusync_attn_block_desc {
  int32_t batch, seq, hidden, heads, out_features, model_hidden;
  int32_t kv_splits;               /* 0 = choose */
  const void* x; const void* w_qkv; const void* k_cache; const void* v_cache; const void* w_o;
  void* qkv; void* attn_out; void* y;
} cusync_attn_block_desc_t;

typedef struct cusync_attn_block cusync_attn_block_t;

/* Stage construction, both setProducerConsumerPair calls and the three kernels' initialisation
 * (attention.cu:706-790), for the synchronised chain and for the same kernels without synchronisation. */
CUSYNC_API int cusync_attn_block_create(cusync_attn_block_t** out, const cusync_attn_block_desc_t* desc);
CUSYNC_API int cusync_attn_block_destroy(cusync_attn_block_t* block);
/* The three kernels back to back on one stream (the reference's baseline loop). */
CUSYNC_API int cusync_attn_block_run_stream_ordered(cusync_attn_block_t* block, cusync_stream_t stream);
/* runAttentionCuSync, one iteration (attention.cu:792-833): stage i on streams[i], a wait kernel before each
 * dependent stage, incrementIter on all three afterwards.  streams: [3]. */
CUSYNC_API int cusync_attn_block_run_cusync(cusync_attn_block_t* block, const cusync_stream_t* streams);
/* The same on ONE stream, each dependent stage launched as a programmatic dependent of the stage ahead of it
 * (cusync_gemm_run_dependent, cusync_attn_run_dependent). */
CUSYNC_API int cusync_attn_block_run_dependent(cusync_attn_block_t* block, cusync_stream_t stream);
/* Stage handles (0 = QKV projection, 1 = attention, 2 = output projection) for inspection. */
CUSYNC_API cusync_stage_t* cusync_attn_block_stage(cusync_attn_block_t* block, int which);
/* Configuration in use: out[0..4] = tile_n of the two GEMMs, their K slices, key-range splits of the attention. */
CUSYNC_API int cusync_attn_block_config(const cusync_attn_block_t* block, int32_t* out5);

/* The same block in the prompt phase, as the reference runs it (attention.cu:272-276 with seqlen = 0 and a
 * batch of 512 to 2048 tokens; numbers in results/attention-results-gpt-3-cuda-12.2): four dependent GEMMs,
 *   XQKV = X Wqkv;  S = Q K^T;  O = S V;  Y = O Wo
 * with Q, K, V the three thirds of XQKV's columns and no softmax or heads (attention.cu:445-509), each on its own
 * stream behind a wait kernel (:792-811).  Stage typing: ConsecutiveSync out of the first GEMM, RowSync between the
 * others (the STRIDEDSYNC configuration, :105-118).  The reference's policies wait for A operands only; here
 * S = Q K^T also waits for the K rows of the column tile it computes and O = S V for the V rows of each K block
 * (cusync_gemm_desc_t.b_stage).  x[batch, hidden], w_qkv[hidden, 3 * heads * 128], w_o[heads * 128, out_features];
 * intermediates qkv[batch, 3 * heads * 128], s[batch, batch], o[batch, heads * 128]; all row-major fp16 on the
 * device, caller-owned.  batch > 256 and a multiple of 64; model_hidden = 8 * heads * 128.  Without a softmax the
 * values grow with every GEMM: inputs must be scaled so that O stays inside fp16 (the reference skips its own
 * check of this chain for that reason, attention.cu:512-515). */
typedef struct cusync_attn_prompt_desc {
  int32_t batch, hidden, heads, out_features, model_hidden;
  const void* x; const void* w_qkv; const void* w_o;
  void* qkv; void* s; void* o; void* y;
} cusync_attn_prompt_desc_t;

typedef struct cusync_attn_prompt cusync_attn_prompt_t;

CUSYNC_API int cusync_attn_prompt_create(cusync_attn_prompt_t** out, const cusync_attn_prompt_desc_t* desc);
CUSYNC_API int cusync_attn_prompt_destroy(cusync_attn_prompt_t* block);
/* The four GEMMs back to back on one stream (runAttentionBaseline, attention.cu:557-704). */
CUSYNC_API int cusync_attn_prompt_run_stream_ordered(cusync_attn_prompt_t* block, cusync_stream_t stream);
/* runAttentionCuSync, one iteration (attention.cu:706-833).  streams: [4]. */
CUSYNC_API int cusync_attn_prompt_run_cusync(cusync_attn_prompt_t* block, const cusync_stream_t* streams);
/* The same on ONE stream, GEMMs 2 to 4 launched with cusync_gemm_run_dependent. */
CUSYNC_API int cusync_attn_prompt_run_dependent(cusync_attn_prompt_t* block, cusync_stream_t stream);
/* Stage handles (0 = XQKV, 1 = S, 2 = O, 3 = Y) for inspection. */
CUSYNC_API cusync_stage_t* cusync_attn_prompt_stage(cusync_attn_prompt_t* block, int which);

/* ---- MLP driver ---------------------------------------------------------- */

enum { CUSYNC_MLP_GPT3 = 0, CUSYNC_MLP_LLAMA = 1 };

/* One tensor-parallel MLP shard, the workload of
 * src/ml-bench/transformer/mlp.cu (MLPParameters :209-330):
 *   GPT-3 : H = GELU(X * W1);            Y = H * W2
 *   LLaMA : H = SiLU(X * W1) (.) (X * V); Y = H * W2   (the fused form of mlp-lib.cu:123-134)
 * X[batch, hidden], W1 and V [hidden, ffn], W2 [ffn, hidden], H[batch, ffn],
 * Y[batch, hidden]; all row-major fp16 on the device, caller-owned. */
typedef struct cusync_mlp_desc {
  int32_t model;                 /* CUSYNC_MLP_* */
  int32_t batch, hidden, ffn;
  int32_t policy;                /* CUSYNC_POLICY_ROWSYNC or CUSYNC_POLICY_TILESYNC between the two GEMMs; 0 = choose
                                    (cusync_mlp_choose_config) */
  int32_t opts;                  /* CUSYNC_OPT_* applied to both stages */
  int32_t tile_n1, tile_n2;      /* 0 = choose */
  int32_t split_k1, split_k2;    /* 0 = choose (mlp.cu's --split-k1 / --split-k2) */
  int32_t max_ctas;              /* 0 = one per SM */
  int32_t cta_pair;              /* as cusync_gemm_desc_t.cta_pair, for both GEMMs */
  int32_t group_rows2;           /* the consumer's tile order: 0 = choose (cusync_mlp_choose_config), 1 = plain,
                                    n > 1 = CUSYNC_ORDER_GROUPED(n) */
  int32_t tail_split_sync1, tail_split_sync2;    /* cusync_gemm_desc_t.tail_split of the two synchronised GEMMs ... */
  int32_t tail_split_plain1, tail_split_plain2;  /* ... and of the two stream-ordered ones: 0 = choose, 1 = none */
  int32_t group_rows1;           /* the producer's tile order, like group_rows2 */
  int32_t x_rows;                /* 1: X arrives in row blocks while the layer runs (e.g. host-to-device copies on
                                    another stream): the first GEMM of run_cusync waits, per 128-row tile, on a RowSync
                                    semaphore that the caller posts with cusync_mlp_post_x_rows once per run */
  int32_t single_grid;           /* run_cusync launches both GEMMs as one persistent grid (cusync_gemm_run_chain) on the
                                    producer stream and lets the consumer stream wait for it: 0 = choose
                                    (cusync_mlp_choose_config, and only where both GEMMs run the CTA-pair kernel), 1 = never (one launch per GEMM and a wait
                                    kernel, as mlp.cu:691-712), 2 = required (else cusync_mlp_create fails) */
  int32_t post_rows;             /* 1: the second GEMM of run_cusync is a producer too: it posts RowSync semaphores, one
                                    per 128-row tile of Y, counting its column tiles, so that whatever consumes Y (the
                                    all-reduce of a tensor-parallel layer) can start row block by row block
                                    (cusync_mlp_wait_rows) */
  const void* x; const void* w1; const void* v; const void* w2;
  void* h; void* y;
} cusync_mlp_desc_t;

typedef struct cusync_mlp cusync_mlp_t;

/* MLPParameters + stage construction + setProducerConsumerPair + both
 * GEMM initialisations (mlp.cu:1026-1062, 653-684). */
CUSYNC_API int cusync_mlp_create(cusync_mlp_t** out, const cusync_mlp_desc_t* desc);
CUSYNC_API int cusync_mlp_destroy(cusync_mlp_t* mlp);
/* runBaselineGPT3 / runBaselineLLaMA, one iteration: the same two kernels,
 * no tile synchronisation, back to back on one stream (mlp.cu:411-491). */
CUSYNC_API int cusync_mlp_run_stream_ordered(cusync_mlp_t* mlp, cusync_stream_t stream);
/* runCuSyncGPT3 / runCuSyncLLaMA, one iteration: producer GEMM on
 * producer_stream, wait kernel + consumer GEMM on consumer_stream, then
 * incrementIter on both stages (mlp.cu:691-712). */
CUSYNC_API int cusync_mlp_run_cusync(cusync_mlp_t* mlp, cusync_stream_t producer_stream,
                                     cusync_stream_t consumer_stream);
/* The same two synchronised launches on ONE stream, the consumer GEMM as a programmatic dependent of the producer
 * (cusync_gemm_run_dependent) in place of the second stream and the wait kernel.  Never the one-grid form; same
 * stages, semaphore counts and results as run_cusync. */
CUSYNC_API int cusync_mlp_run_dependent(cusync_mlp_t* mlp, cusync_stream_t stream);
/* One of the two un-synchronised kernels alone (1 = first GEMM, 2 = second), for per-kernel timing
 * (the reference's baseline prints both, mlp.cu:463-488). */
CUSYNC_API int cusync_mlp_run_single(cusync_mlp_t* mlp, int which, cusync_stream_t stream);
/* New X / Y buffers for later runs (update, gemm/device/cusyncgemm.h:459-494). */
CUSYNC_API int cusync_mlp_update_io(cusync_mlp_t* mlp, const void* x, void* y);
/* Stage handles (0 = producer, 1 = consumer) for inspection. */
CUSYNC_API cusync_stage_t* cusync_mlp_stage(cusync_mlp_t* mlp, int which);
/* Timeline buffers for the two synchronised GEMMs (see cusync_gemm_plan_set_trace). */
CUSYNC_API int cusync_mlp_set_trace(cusync_mlp_t* mlp, void* trace1, uint32_t capacity1, void* trace2, uint32_t capacity2);
/* Configuration in use: out[0..5] = tile_n1, tile_n2, ctas1, ctas2, split_k1, split_k2. */
CUSYNC_API int cusync_mlp_config(const cusync_mlp_t* mlp, int32_t* out6);
/* With desc.x_rows: enqueues on `stream` the post (a stream memory operation, no kernel) for the 128-row tiles
 * [first_tile, first_tile + num_tiles) of X; what was enqueued on `stream` before (the copy that brings those
 * rows) is complete when the first GEMM sees the post.  Call it once per row tile and run_cusync: the j-th post of
 * a tile is the one the j-th run_cusync waits for, whether it is enqueued before that run's launch or after it
 * (launching first lets the GEMMs be resident when the first rows land; their waits are bounded, so rows that
 * never come end in a timeout record, not a hang).  The copy itself must not need an SM (a host-to-device
 * cudaMemcpyAsync does not; a copy kernel might wait for the GEMM's blocks to retire). */
CUSYNC_API int cusync_mlp_post_x_rows(cusync_mlp_t* mlp, uint32_t first_tile, uint32_t num_tiles, cusync_stream_t stream);
/* With desc.post_rows: makes `stream` wait (a stream memory operation, no kernel) for the 128-row tiles
 * [first_tile, first_tile + num_tiles) of Y as written by the most recent run_cusync (call it after that
 * run_cusync).  Work enqueued on `stream` afterwards sees those rows complete. */
CUSYNC_API int cusync_mlp_wait_rows(cusync_mlp_t* mlp, uint32_t first_tile, uint32_t num_tiles, cusync_stream_t stream);
/* What the library picks for a layer when the descriptor leaves it open: the role of the reference's tuning
 * table src/ml-bench/transformer/tile_sizes_db.py as applied by eval_mlp.py:141-210 (tile shapes, split-K and the
 * optimisation switches per model and batch).  A pure host function: needs no device. */
typedef struct cusync_mlp_choice {
  int32_t policy;                /* CUSYNC_POLICY_ROWSYNC or CUSYNC_POLICY_TILESYNC */
  int32_t single_grid;           /* 1 = one launch per GEMM and a wait, 2 = one persistent grid */
  int32_t stream_wait;           /* 1 = the wait before the second launch is a stream memory operation */
  int32_t group_rows1, group_rows2;
  int32_t tile_n1, tile_n2, split_k1, split_k2;
  int32_t tail_split1;           /* K slices for the tiles of the first GEMM's last partial round in the one-grid form
                                    (0 = none); cusync_mlp_create applies it where the caller left single_grid and
                                    tail_split_sync1 open and the tail's units fit one round of the SM pairs */
} cusync_mlp_choice_t;
CUSYNC_API int cusync_mlp_choose_config(int32_t model, int32_t batch, int32_t hidden, int32_t ffn, cusync_mlp_choice_t* out);
/* 1 when run_cusync launches both GEMMs as one persistent grid. */
CUSYNC_API int cusync_mlp_uses_single_grid(const cusync_mlp_t* mlp);
/* Tail splits in use: out[0..3] = synchronised GEMM 1, 2, stream-ordered GEMM 1, 2. */
CUSYNC_API int cusync_mlp_tail_splits(const cusync_mlp_t* mlp, int32_t* out4);

/* ---- all-reduce beside the producing GEMM (tensor-parallel layers) -------- */

/* Sum all-reduce, in place, of the fp16 matrix Y[rows, cols] that every rank of a tensor-parallel group holds a
 * partial copy of: the one exchange step of the sharded MLP / attention layer.  The reference times this
 * collective on its own and runs it after the layer (src/ml-bench/transformer/allreduce_times.py:11-35); here it
 * is a small persistent kernel that runs BESIDE the GEMM producing Y and takes the matrix by 128-row tile as the
 * GEMM's RowSync semaphores publish them (cusync_mlp_desc_t.post_rows), so only the last tiles' exchange is left
 * once the GEMM ends.  Rank r sums rows [r, r + 1) * tile_rows / world of every tile over all ranks (fp32
 * accumulation, one rounding to fp16) and writes the sums into every rank's copy: through the NVSwitch
 * (multimem.ld_reduce / multimem.st on multicast addresses) when such addresses are given, else with plain peer
 * loads (summed in rank order) and peer stores.  Every rank must run its plan equally often.
 *
 * Memory comes from the caller and must be peer-accessible (one process per GPU: symmetric / IPC-mapped
 * memory): buffers[w] / flags[w] are rank w's matrix and flag words AS MAPPED INTO THIS PROCESS
 * (buffers[rank] is the local one); flags need cusync_allreduce_flag_words() uint32 each, zeroed once before
 * the first run; multicast_* are the NVLS multicast addresses of the same two allocations, or both NULL.
 * Launch it BEFORE the GEMMs of the run (it must be resident while they run; give the GEMMs max_ctas =
 * SMs - num_ctas) on a stream of its own. */
typedef struct cusync_allreduce_desc {
  int32_t rank, world;             /* world <= 8 */
  int32_t rows, cols;              /* cols a multiple of 8 */
  int64_t ld;                      /* row pitch in elements, the same on every rank */
  int32_t tile_rows;               /* 0 = 128 */
  int32_t num_ctas;                /* 0 = choose (4); even: blocks are launched in pairs that fill whole TPCs */
  void* const* buffers;            /* [world] */
  uint32_t* const* flags;          /* [world] */
  void* multicast_buffer;
  uint32_t* multicast_flags;
  uint64_t timeout_ns;             /* 0 = default bound of every wait inside the kernel */
} cusync_allreduce_desc_t;

typedef struct cusync_allreduce_plan cusync_allreduce_plan_t;

CUSYNC_API uint32_t cusync_allreduce_flag_words(int32_t rows, int32_t tile_rows);
CUSYNC_API int cusync_allreduce_plan_create(cusync_allreduce_plan_t** out, const cusync_allreduce_desc_t* desc);
CUSYNC_API int cusync_allreduce_plan_destroy(cusync_allreduce_plan_t* plan);
/* One all-reduce.  row_semaphores: this rank's per-tile semaphores (one per tile_rows rows), a tile being complete
 * when its semaphore has reached `value`; NULL = the matrix is complete when the kernel starts (stream order). */
CUSYNC_API int cusync_allreduce_run(cusync_allreduce_plan_t* plan, const uint32_t* row_semaphores, uint32_t value,
                                    cusync_stream_t stream);
/* Timeout record: where = 1 the local producer never published a tile, 2 another rank did not, 3 the final
 * handshake.  After a timeout the flag words have to be zeroed on every rank and the plans recreated. */
CUSYNC_API int cusync_allreduce_read_status(const cusync_allreduce_plan_t* plan, cusync_status_t* out);
CUSYNC_API uint32_t cusync_allreduce_plan_num_ctas(const cusync_allreduce_plan_t* plan);

/* One layer of a tensor-parallel MLP shard with its all-reduce overlapped: the reducer goes to reduce_stream
 * first, then run_cusync's GEMMs (created with post_rows), and consumer_stream ends up waiting for both.  The
 * sharded driver of mlp.cu (:243-251 shapes) plus the collective the reference leaves to its caller. */
CUSYNC_API int cusync_mlp_run_cusync_allreduce(cusync_mlp_t* mlp, cusync_allreduce_plan_t* reducer,
                                               cusync_stream_t producer_stream, cusync_stream_t consumer_stream,
                                               cusync_stream_t reduce_stream);

/* ---- tensor-parallel layer (one process per GPU) ------------------------- */

/* The sharded layer with its collective below the C ABI: rank r of `world` holds the r-th column slice of W1 (and
 * V) and the r-th row slice of W2 (the shard shapes of src/ml-bench/transformer/mlp.cu:243-251), X is replicated,
 * and the layer ends with the sum all-reduce of Y over the ranks, the collective the reference times on its own
 * (allreduce_times.py:11-35).  cusync_tp_layer_run runs one layer of a cusync_mlp_t either
 *   - with `reducer`: the all-reduce kernel of this library beside the second GEMM
 *     (cusync_mlp_run_cusync_allreduce; the shard was created with post_rows and Y is the reducer's matrix), or
 *   - without: cusync_mlp_run_cusync, then ncclAllReduce(sum, fp16, in place) of y[0 .. y_count) on
 *     consumer_stream over `comm` (nothing when the communicator has one rank).
 * The NCCL communicator is created here: rank 0 calls cusync_tp_unique_id and hands the 128 bytes to every rank by
 * whatever channel the application has (a file, a socket, another library's broadcast); then every rank calls
 * cusync_tp_comm_create with its device current.  NCCL is taken from the process's libnccl.so.2 at run time:
 * CUSYNC_ERROR_UNSUPPORTED where there is none. */
typedef struct cusync_tp_comm cusync_tp_comm_t;
CUSYNC_API int cusync_tp_unique_id(void* out128);
CUSYNC_API int cusync_tp_comm_create(cusync_tp_comm_t** out, int32_t world, int32_t rank, const void* unique_id128);
CUSYNC_API int cusync_tp_comm_destroy(cusync_tp_comm_t* comm);
/* ncclAllReduce(sum) of `count` fp16 values in place on `stream`. */
CUSYNC_API int cusync_tp_all_reduce(cusync_tp_comm_t* comm, void* buffer, uint64_t count, cusync_stream_t stream);
CUSYNC_API int cusync_tp_layer_run(cusync_mlp_t* mlp, cusync_tp_comm_t* comm, cusync_allreduce_plan_t* reducer, void* y,
                                   uint64_t y_count, cusync_stream_t producer_stream, cusync_stream_t consumer_stream,
                                   cusync_stream_t reduce_stream);

/* Library / device information. */
CUSYNC_API const char* cusync_b200_version(void);
CUSYNC_API int cusync_b200_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CUSYNC_B200_H */
