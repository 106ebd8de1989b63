/*
 * CPU oracle for the CuSync hot path.  TEST INFRASTRUCTURE ONLY: nothing the
 * product ships may link, load or call this file.  It restates, in plain C,
 *   (1) the integer side of microsoft/cusync -- tile orders, sync policies,
 *       the schedule buffer and the semaphore counts a producer/consumer pair
 *       must reach -- and
 *   (2) the arithmetic the reference's check path pins its kernels to:
 *       fp16 operands, fp32 accumulation in k order, fp16 rounding of every
 *       intermediate that lives in global memory.
 * Each function cites the reference file:line it follows.
 *
 * Parity pinning: the integer side is pinned to the reference's own policy and
 * tile-order code (compiled for the host from the reference headers, see
 * oracle/Makefile target `_ref`) and to the known answers of the reference's
 * tests (tests/simple-test.cu:83-96, src/examples/twoMatMuls/matrixMul.cu:235-272).
 * The arithmetic side is pinned to NVIDIA CUTLASS's host reference kernels, the
 * code the reference's drivers check their GPU kernels against
 * (cutlass::reference::host::Conv2dFprop, src/ml-bench/volta_conv2d/resnet.cu:706-720;
 * the CUTLASS host GEMM; the GELU / SiLu / ReLu functors of its epilogues):
 * oracle/cutlass_host_ref.cpp wraps them and tests/test_oracle_cutlass_pin.py
 * compares bit patterns (GEMM, GELU, ReLU, convolution: bit-exact; SiLU*mul:
 * within one half-precision ulp).  The softmax of the decode-attention stage
 * has no counterpart in the reference (its attention.cu has no softmax):
 * parity unpinned for that one function; it is checked against float64 numpy.
 */
#ifndef CUSYNC_ORACLE_H
#define CUSYNC_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct { uint32_t x, y, z; } orc_dim3;

/* Tile orders (src/include/cusync/tile-orders.h:50-76). */
enum { ORC_ORDER_IDENTITY = 0, ORC_ORDER_TRANSPOSE_XY = 1 };

/* Policy kinds.  ROW/TILE/CONV2D: src/include/cusync/policies.h:37-210.
 * STRIDED: StridedSync, src/ml-bench/transformer/mlp.cu:76-101.
 * CONSECUTIVE: ConsecutiveSync, src/ml-bench/transformer/attention.cu:51-70. */
enum {
  ORC_NOSYNC = 0, ORC_ROWSYNC = 1, ORC_TILESYNC = 2, ORC_STRIDEDSYNC = 3,
  ORC_CONV2DTILESYNC = 4, ORC_CONSECUTIVESYNC = 5
};

typedef struct {
  int32_t  kind;
  int32_t  order;       /* tile order used by tileIndex (ignored by ROW) */
  uint32_t tile_m;      /* TileM template argument */
  uint32_t tile_n;      /* TileN template argument */
  uint32_t wait_value;  /* waitValue_ member (ROW/TILE/CONV2D) */
  uint32_t post_value;  /* postValue_ member (ROW/TILE/CONV2D) */
  uint32_t p0;          /* STRIDED: GridN;  CONV2D: R*S;  CONSECUTIVE: H */
  uint32_t p1;          /* STRIDED: stride */
} orc_policy;

enum { ORC_OPT_NO_ATOMIC_ADD = 1 };  /* Optimizations::NoAtomicAdd, cusync.h:69-75 */

/* ---- integer side -------------------------------------------------------- */
uint32_t orc_block_index(int order, orc_dim3 grid, orc_dim3 block);
orc_dim3 orc_tile_to_block(int order, orc_dim3 tile);
uint32_t orc_order_tile_index(int order, orc_dim3 tile, orc_dim3 grid);

uint32_t orc_policy_wait_value(const orc_policy* p, orc_dim3 tile, orc_dim3 grid);
uint32_t orc_policy_post_value(const orc_policy* p, orc_dim3 tile, orc_dim3 grid);
uint32_t orc_policy_tile_index(const orc_policy* p, orc_dim3 tile, orc_dim3 grid);
int      orc_policy_is_sync(const orc_policy* p, orc_dim3 tile, orc_dim3 grid);

/* Schedule buffer (cusync.h:125-157).  out[numTiles].  Returns 0 when the
 * order is a bijection onto [0,numTiles), 1 otherwise
 * (CuSyncErrorInvalidLinearBlockIndex). */
int orc_build_tile_order(int order, orc_dim3 grid, orc_dim3* out);

/* Semaphore array of a GEMM-shaped producer after `iters` runs: every tile of
 * grid (x = N tile, y = M tile, z = split-K slice) posts
 * {y*tile_m, x*tile_n, z} once per run, only from the last split-K slice
 * (gemm/kernel/cusyncgemm.h:374-398).  sems[num_sems] must be zeroed by the
 * caller.  Returns the number of posts that fell outside [0,num_sems). */
int orc_producer_semaphores(const orc_policy* out_policy, orc_dim3 grid,
                            uint32_t tile_m, uint32_t tile_n, int opts,
                            uint32_t iters, uint32_t* sems, uint32_t num_sems);

/* Waits of one GEMM-shaped consumer tile whose A operand starts at row
 * `row_off`: K is walked in steps of block_k; the first step is the
 * "prologue" wait (tile.z = 1), later steps carry z = 0
 * (gemm/threadblock/cusyncmma_multistage.h:986-994,1032-1039,1076-1084).
 * Writes (index, expected = iter*waitValue) pairs for the steps where isSync
 * holds; returns how many. */
uint32_t orc_consumer_tile_waits(const orc_policy* in_policy, orc_dim3 prod_grid,
                                 uint32_t row_off, uint32_t k_extent,
                                 uint32_t block_k, uint32_t iter,
                                 uint32_t* idx_out, uint32_t* expect_out,
                                 uint32_t cap);

/* ---- arithmetic side ------------------------------------------------------ */
enum { ORC_EPI_NONE = 0, ORC_EPI_GELU_ERF = 1, ORC_EPI_RELU = 2 };

float    orc_half_to_float(uint16_t h);
uint16_t orc_float_to_half(float f);   /* round to nearest even */

/* C[M,N] = epi(A[M,K] * B[K,N]); all row-major fp16, fp32 accumulate in k
 * order, fp32 epilogue, one rounding to fp16
 * (src/ml-bench/transformer/common.h:89-102; GELU = 0.5x(1+erf(x/sqrt2)), the
 * form CUTLASS LinearCombinationGELU selects at mlp.cu:146). */
void orc_gemm_f16(int M, int N, int K, const uint16_t* A, int lda,
                  const uint16_t* B, int ldb, uint16_t* C, int ldc, int epilogue);

/* G[M,N] = SiLU(A*B1) (.) (A*B2), SiLU(x) = x/(1+exp(-x))
 * (src/ml-bench/transformer/mlp-lib.cu:123-134). */
void orc_gemm_dual_silu_mul_f16(int M, int N, int K, const uint16_t* A, int lda,
                                const uint16_t* B1, const uint16_t* B2, int ldb,
                                uint16_t* G, int ldg);

/* fp32 GEMM of the twoMatMuls example (matrixMul.cu:41-121). */
void orc_gemm_f32(int M, int N, int K, const float* A, const float* B, float* C);

/* NHWC 3x3 stride-1 pad-1 forward convolution, filter KRSC, fp32 accumulate
 * in (r,s,c) order, optional ReLU, fp16 out
 * (cutlass::reference::host::Conv2dFprop as called at
 * src/ml-bench/volta_conv2d/resnet.cu:708-720). */
void orc_conv2d_3x3_nhwc_f16(int N, int H, int W, int C, int K,
                             const uint16_t* x, const uint16_t* w, uint16_t* y,
                             int relu);

/* Decode attention for one tensor-parallel shard: q[B,heads,d] against cached
 * k,v[B,S,heads,d]; scores scaled by 1/sqrt(d), fp32 softmax, fp16 out.
 * The reference's chain has no softmax (attention.cu:445-509); this follows
 * the standard definition. */
void orc_attention_decode_f16(int B, int S, int heads, int d, const uint16_t* q,
                              int ldq, const uint16_t* k, const uint16_t* v,
                              uint16_t* o, int ldo);

/* Largest |got-ref|/max(|ref|, floor) with floor = floor_frac * max|ref|.
 * Elements below the floor are thereby compared absolutely, which makes the
 * small-magnitude escape of common.h:104-137 explicit. */
double orc_max_rel_err_f16(size_t n, const uint16_t* got, const uint16_t* ref,
                           double floor_frac);

/* Number of OpenMP threads the arithmetic functions will use. */
int orc_num_threads(void);
/* Threads the OpenMP loops use from now on (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
