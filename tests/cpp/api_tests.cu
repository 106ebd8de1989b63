// Tests of the C++ template API (<cusync/cusync.h>, <cusync/gemm.h>), compiled
// with nvcc into a shared library whose extern "C" entry points pytest calls.
// They restate the reference's own tests for this build:
//   api_simple_test    tests/simple-test.cu:14-138 (the four gtest cases)
//   api_two_matmuls    src/examples/twoMatMuls/matrixMul.cu (known answers 2.56 / 6.5536)
// and add what the reference lacks: a GEMM chain through the Gemm handle, a
// user-written policy and tile order, and a bounded-wait timeout.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include <cusync/cusync.h>
#include <cusync/conv.h>
#include <cusync/gemm.h>

#define API extern "C" __attribute__((visibility("default")))

namespace cusync {
// The friend class the CuStage template names, as in tests/cusync-test.h:8-44:
// records inside the consumer kernel whether each semaphore holds exactly
// expectedWaitValue * iter when its wait returns.
class CuSyncTest {
 public:
  char* semValid;
  explicit CuSyncTest(int n) {
    CUDA_CHECK(cudaMalloc(&semValid, n));
    CUDA_CHECK(cudaMemset(semValid, 1, n));
  }
  template <typename Stage>
  __device__ void setSemValue(unsigned idx, dim3 tile, Stage& stage) {
    if (!stage.isConsumer()) return;
    if (threadIdx.x == 0) {
      bool eq = stage.expectedWaitValue(tile) * stage.iter == stage.waitSemValue(tile);
      if (!eq) semValid[idx] = 0;
    }
  }
  bool allSemsCorrect(int n) {
    std::vector<char> h(n);
    CUDA_CHECK(cudaMemcpy(h.data(), semValid, n, cudaMemcpyDeviceToHost));
    for (char c : h) if (!c) return false;
    return true;
  }
  void destroy() { cudaFree(semValid); }
};
}  // namespace cusync

using namespace cusync;

// ---------------------------------------------------------------------------
// simple-test: two dependent copy kernels
// ---------------------------------------------------------------------------
template <typename Stage>
__global__ void copyKernel(CuSyncTest test, Stage stage, int idx, const unsigned* in, unsigned* out) {
  __shared__ int tileSh[3];
  dim3 tile = stage.tile((dim3*)&tileSh[0]);
  stage.wait(tile);
  unsigned i = threadIdx.x + tile.x * blockDim.x;
  out[i] = in[i];
  stage.post(tile);
  if (idx >= 0) test.setSemValue(idx, tile, stage);
}

template <typename Sync, typename Prod, typename Cons>
static int runSimple(int iters, size_t size) {
  unsigned *a1, *a2, *a3;
  CUDA_CHECK(cudaMalloc(&a1, size * 4)); CUDA_CHECK(cudaMalloc(&a2, size * 4)); CUDA_CHECK(cudaMalloc(&a3, size * 4));
  std::vector<unsigned> host(size);
  for (size_t i = 0; i < size; i++) host[i] = (unsigned)i;
  CUDA_CHECK(cudaMemcpy(a1, host.data(), size * 4, cudaMemcpyHostToDevice));
  cudaStream_t ps, cs;
  CUDA_CHECK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
  CUDA_CHECK(cudaStreamCreateWithFlags(&ps, cudaStreamNonBlocking));
  dim3 threads(128, 1, 1), grid((unsigned)(size / 128), 1, 1);
  Sync sync;
  Prod prod(grid, threads, NoSync(), sync);
  Cons cons(grid, threads, sync, NoSync());
  int result = 0;
  if (CuSync::setProducerConsumerPair(prod, cons) != CuSyncSuccess) result |= 8;
  CuSyncTest test(1);
  for (int it = 0; it < iters; it++) {
    // poison the outputs so a consumer that ran ahead of its producer is caught
    CUDA_CHECK(cudaMemset(a2, 0xff, size * 4)); CUDA_CHECK(cudaMemset(a3, 0xff, size * 4));
    CUDA_CHECK(cudaDeviceSynchronize());
    copyKernel<Prod><<<grid, threads, 0, ps>>>(test, prod, -1, a1, a2);
    prod.invokeWaitKernel(cs);
    copyKernel<Cons><<<grid, threads, 0, cs>>>(test, cons, 0, a2, a3);
    CUDA_CHECK(cudaDeviceSynchronize());
    prod.incrementIter(); cons.incrementIter();
  }
  CUDA_CHECK(cudaMemcpy(host.data(), a2, size * 4, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < size; i++) if (host[i] != i) { result |= 1; break; }
  CUDA_CHECK(cudaMemcpy(host.data(), a3, size * 4, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < size; i++) if (host[i] != i) { result |= 2; break; }
  if (!test.allSemsCorrect(1)) result |= 4;
  if (prod.status().code != 0 || cons.status().code != 0) result |= 16;
  // every semaphore == iters (TileSync<.,1,1> posts 1 per run)
  std::vector<uint32_t> sems(grid.x);
  cusync_stage_read_semaphores(prod.handle(), sems.data(), grid.x);
  for (uint32_t s : sems) if (s != (uint32_t)iters) { result |= 32; break; }
  test.destroy(); prod.destroy(); cons.destroy();
  cudaFree(a1); cudaFree(a2); cudaFree(a3);
  cudaStreamDestroy(ps); cudaStreamDestroy(cs);
  return result;   // 0 = pass
}

// variant: 0 NoOpts, 1 NoAtomicAdd, 2 AvoidCustomOrder (tests/simple-test.cu:107-138)
API int api_simple_test(int variant, int iters, int log2_size) {
  using Sync = TileSync<IdentityOrder, 1, 1>;
  using Cons = CuStage<IdentityOrder, Sync, NoSync>;
  size_t size = (size_t)1 << log2_size;
  switch (variant) {
    case 0: return runSimple<Sync, CuStage<IdentityOrder, NoSync, Sync>, Cons>(iters, size);
    case 1: return runSimple<Sync, CuStage<IdentityOrder, NoSync, Sync, NoAtomicAdd>, Cons>(iters, size);
    case 2: return runSimple<Sync, CuStage<IdentityOrder, NoSync, Sync, AvoidCustomOrder>, Cons>(iters, size);
    default: return -1;
  }
}

// ---------------------------------------------------------------------------
// twoMatMuls: fp32 SIMT tiled matmul chain with a wait per K tile
// ---------------------------------------------------------------------------
constexpr int kTile = 32;
using MMSync = TileSync<IdentityOrder, kTile, kTile>;
using MMProd = CuStage<IdentityOrder, NoSync, MMSync>;
using MMCons = CuStage<IdentityOrder, MMSync, NoSync>;

template <typename Stage>
__global__ void simtMatmul(Stage stage, float* C, const float* A, const float* B, int n) {
  __shared__ int tileSh[3];
  __shared__ float As[kTile][kTile], Bs[kTile][kTile];
  dim3 t = stage.tile((dim3*)&tileSh[0]);
  const int col0 = t.x * kTile, row0 = t.y * kTile;
  float acc = 0.f;
  for (int k0 = 0; k0 < n; k0 += kTile) {
    // A's tile (rows row0.., columns k0..) is the producer's tile (x = k0/32, y = row0/32)
    dim3 w((unsigned)k0, (unsigned)row0, 1);
    stage.wait(w);
    As[threadIdx.y][threadIdx.x] = A[(row0 + threadIdx.y) * n + k0 + threadIdx.x];
    Bs[threadIdx.y][threadIdx.x] = B[(k0 + threadIdx.y) * n + col0 + threadIdx.x];
    __syncthreads();
    for (int k = 0; k < kTile; k++) acc += As[threadIdx.y][k] * Bs[k][threadIdx.x];
    __syncthreads();
  }
  C[(row0 + threadIdx.y) * n + col0 + threadIdx.x] = acc;
  stage.post(dim3((unsigned)col0, (unsigned)row0, 0));
}

// A = a_val, B = D = b_val (n x n): C = A*B, E = C*D.  Outputs C and E to host.
API int api_two_matmuls(int n, float a_val, float b_val, float* hostC, float* hostE, int iters) {
  size_t bytes = (size_t)n * n * 4;
  std::vector<float> ha((size_t)n * n, a_val), hb((size_t)n * n, b_val);
  float *A, *B, *C, *D, *E;
  CUDA_CHECK(cudaMalloc(&A, bytes)); CUDA_CHECK(cudaMalloc(&B, bytes)); CUDA_CHECK(cudaMalloc(&C, bytes));
  CUDA_CHECK(cudaMalloc(&D, bytes)); CUDA_CHECK(cudaMalloc(&E, bytes));
  CUDA_CHECK(cudaMemcpy(A, ha.data(), bytes, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(B, hb.data(), bytes, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(D, hb.data(), bytes, cudaMemcpyHostToDevice));
  dim3 threads(kTile, kTile), grid(n / kTile, n / kTile, 1);
  MMSync sync;
  MMProd prod(grid, threads, NoSync(), sync);
  MMCons cons(grid, threads, sync, NoSync());
  int rc = 0;
  if (CuSync::setProducerConsumerPair(prod, cons) != CuSyncSuccess) rc |= 1;
  cudaStream_t ps, cs;
  CUDA_CHECK(cudaStreamCreateWithFlags(&ps, cudaStreamNonBlocking));
  CUDA_CHECK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
  for (int it = 0; it < iters; it++) {
    CUDA_CHECK(cudaMemset(C, 0xff, bytes)); CUDA_CHECK(cudaMemset(E, 0xff, bytes));
    CUDA_CHECK(cudaDeviceSynchronize());
    simtMatmul<MMProd><<<grid, threads, 0, ps>>>(prod, C, A, B, n);
    prod.invokeWaitKernel(cs);
    simtMatmul<MMCons><<<grid, threads, 0, cs>>>(cons, E, C, D, n);
    CUDA_CHECK(cudaDeviceSynchronize());
    prod.incrementIter(); cons.incrementIter();
  }
  CUDA_CHECK(cudaMemcpy(hostC, C, bytes, cudaMemcpyDeviceToHost));
  CUDA_CHECK(cudaMemcpy(hostE, E, bytes, cudaMemcpyDeviceToHost));
  if (prod.status().code || cons.status().code) rc |= 2;
  prod.destroy(); cons.destroy();
  cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(D); cudaFree(E);
  cudaStreamDestroy(ps); cudaStreamDestroy(cs);
  return rc;
}

// ---------------------------------------------------------------------------
// GEMM chain through cusync::b200::Gemm, the reference's call pattern
// (ml-bench/transformer/mlp.cu:653-712).  policy: 0 RowSync, 1 TileSync.
// Host fp16 in, host fp16 out (C = A*B, E = C*D).  sems_out[numTiles of GEMM1].
// ---------------------------------------------------------------------------
template <typename Sync, typename Prod, typename Cons>
static int runChain(Sync sync, int M, int N, int K, const void* hA, const void* hB, const void* hD, void* hC,
                    void* hE, int iters, uint32_t* sems_out) {
  using namespace cusync::b200;
  using Gemm1 = Gemm<Prod, EpilogueNone, 128>;
  using Gemm2 = Gemm<Cons, EpilogueNone, 128>;
  half *A, *B, *C, *D, *E;
  CUDA_CHECK(cudaMalloc(&A, (size_t)M * K * 2)); CUDA_CHECK(cudaMalloc(&B, (size_t)K * N * 2));
  CUDA_CHECK(cudaMalloc(&C, (size_t)M * N * 2)); CUDA_CHECK(cudaMalloc(&D, (size_t)N * N * 2));
  CUDA_CHECK(cudaMalloc(&E, (size_t)M * N * 2));
  CUDA_CHECK(cudaMemcpy(A, hA, (size_t)M * K * 2, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(B, hB, (size_t)K * N * 2, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(D, hD, (size_t)N * N * 2, cudaMemcpyHostToDevice));
  GemmCoord p1(M, N, K), p2(M, N, N);
  dim3 grid1 = gemmGridShape(p1, 128), grid2 = gemmGridShape(p2, 128);
  Prod prod(grid1, {1, 1, 1}, NoSync(), sync);
  Cons cons(grid2, {1, 1, 1}, sync, NoSync());
  int rc = 0;
  if (CuSync::setProducerConsumerPair(prod, cons) != CuSyncSuccess) rc |= 1;
  typename Gemm1::Arguments a1{prod, p1, {A, K}, {B, N}, {C, N}, {C, N}, {1.f, 0.f}, 1};
  typename Gemm2::Arguments a2{cons, p2, {C, N}, {D, N}, {E, N}, {E, N}, {1.f, 0.f}, 1};
  Gemm1 g1; Gemm2 g2;
  if (g1.can_implement(a1) != Status::kSuccess || g1.initialize(a1) != Status::kSuccess) rc |= 2;
  if (g2.can_implement(a2) != Status::kSuccess || g2.initialize(a2) != Status::kSuccess) rc |= 4;
  cudaStream_t ps, cs;
  int lo, hi;
  CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  CUDA_CHECK(cudaStreamCreateWithPriority(&ps, cudaStreamNonBlocking, hi));
  CUDA_CHECK(cudaStreamCreateWithPriority(&cs, cudaStreamNonBlocking, lo));
  for (int it = 0; it < iters && rc == 0; it++) {
    CUDA_CHECK(cudaMemset(C, 0xff, (size_t)M * N * 2)); CUDA_CHECK(cudaMemset(E, 0xff, (size_t)M * N * 2));
    CUDA_CHECK(cudaDeviceSynchronize());
    if (it % 2 == 0) {
      if (g1.run(true, NULL, ps) != Status::kSuccess) rc |= 8;
      prod.invokeWaitKernel(cs);
      if (g2.run(true, NULL, cs) != Status::kSuccess) rc |= 16;
    } else {
      // every other run on one stream, the consumer a programmatic dependent launch in place of the wait kernel
      if (g1.run(true, NULL, ps) != Status::kSuccess) rc |= 8;
      if (g2.runDependent(ps) != Status::kSuccess) rc |= 16;
    }
    CUDA_CHECK(cudaDeviceSynchronize());
    prod.incrementIter(); cons.incrementIter();
    g1.params_.custage.incrementIter(); g2.params_.custage.incrementIter();
  }
  CUDA_CHECK(cudaMemcpy(hC, C, (size_t)M * N * 2, cudaMemcpyDeviceToHost));
  CUDA_CHECK(cudaMemcpy(hE, E, (size_t)M * N * 2, cudaMemcpyDeviceToHost));
  if (sems_out) cusync_stage_read_semaphores(prod.handle(), sems_out, grid1.x * grid1.y);
  if (prod.status().code || cons.status().code) rc |= 32;
  g1.destroy(); g2.destroy(); prod.destroy(); cons.destroy();
  cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(D); cudaFree(E);
  cudaStreamDestroy(ps); cudaStreamDestroy(cs);
  return rc;
}

API int api_gemm_chain(int policy, int M, int N, int K, const void* hA, const void* hB, const void* hD, void* hC,
                       void* hE, int iters, uint32_t* sems_out) {
  if (policy == 0) {
    using Sync = RowSync<128>;
    Sync sync((N + 127) / 128);
    return runChain<Sync, CuStage<TransposeXYOrder, NoSync, Sync>, CuStage<TransposeXYOrder, Sync, NoSync>>(
        sync, M, N, K, hA, hB, hD, hC, hE, iters, sems_out);
  }
  using Sync = TileSync<TransposeXYOrder, 128, 128>;
  return runChain<Sync, CuStage<TransposeXYOrder, NoSync, Sync, NoAtomicAdd>, CuStage<TransposeXYOrder, Sync, NoSync>>(
      Sync(), M, N, K, hA, hB, hD, hC, hE, iters, sems_out);
}

// ---------------------------------------------------------------------------
// Chain of two 3x3 convolutions through cusync::b200::Conv2dFprop, the reference's call pattern
// (ml-bench/volta_conv2d/resnet.cu:107-116, 659-700): TileSync out of the first, Conv2DTileSync into the second,
// ReLU after each.  Host NHWC / KRSC fp16 in, host fp16 out.  sems_out[N * H / rows].
// ---------------------------------------------------------------------------
API int api_conv_chain(int N, int H, int W, const void* hX, const void* hF1, const void* hF2, void* hY1, void* hY2,
                       int iters, uint32_t* sems_out) {
  using namespace cusync::b200;
  constexpr int C = 64, TileM = 112;            // 56-wide images: two rows per tile
  if (W != 56) return 64;
  using Sync1 = TileSync<TransposeXYOrder, TileM, 64>;
  using Sync2 = Conv2DTileSync<TransposeXYOrder, 3, 3, TileM, 64>;
  using Prod = CuStage<TransposeXYOrder, NoSync, Sync1>;
  using Cons = CuStage<TransposeXYOrder, Sync2, NoSync>;
  using Conv1 = Conv2dFprop<Prod, EpilogueRelu>;
  using Conv2 = Conv2dFprop<Cons, EpilogueRelu>;
  const size_t act = (size_t)N * H * W * C * 2, filt = (size_t)C * 9 * C * 2;
  half *X, *F1, *F2, *Y1, *Y2;
  CUDA_CHECK(cudaMalloc(&X, act)); CUDA_CHECK(cudaMalloc(&Y1, act)); CUDA_CHECK(cudaMalloc(&Y2, act));
  CUDA_CHECK(cudaMalloc(&F1, filt)); CUDA_CHECK(cudaMalloc(&F2, filt));
  CUDA_CHECK(cudaMemcpy(X, hX, act, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(F1, hF1, filt, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemcpy(F2, hF2, filt, cudaMemcpyHostToDevice));
  Conv2dProblemSize problem(N, H, W, C, C);
  int rc = 0;
  if (conv2dTileM(problem) != TileM) rc |= 1;
  dim3 grid = conv2dGridShape(problem);
  Prod prod(grid, {1, 1, 1}, NoSync(), Sync1());
  Cons cons(grid, {1, 1, 1}, Sync2(), NoSync());
  if (CuSync::setProducerConsumerPair(prod, cons) != CuSyncSuccess) rc |= 1;
  typename Conv1::Arguments a1{prod, problem, X, F1, Y1, Y1, {1.f, 0.f}};
  typename Conv2::Arguments a2{cons, problem, Y1, F2, Y2, Y2, {1.f, 0.f}};
  Conv1 c1; Conv2 c2;
  if (c1.can_implement(a1) != Status::kSuccess || c1.initialize(a1) != Status::kSuccess) rc |= 2;
  if (c2.can_implement(a2) != Status::kSuccess || c2.initialize(a2) != Status::kSuccess) rc |= 4;
  cudaStream_t ps, cs;
  int lo, hi;
  CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  CUDA_CHECK(cudaStreamCreateWithPriority(&ps, cudaStreamNonBlocking, hi));
  CUDA_CHECK(cudaStreamCreateWithPriority(&cs, cudaStreamNonBlocking, lo));
  for (int it = 0; it < iters && rc == 0; it++) {
    CUDA_CHECK(cudaMemset(Y1, 0xff, act)); CUDA_CHECK(cudaMemset(Y2, 0xff, act));   // NaN poison
    CUDA_CHECK(cudaDeviceSynchronize());
    if (it % 2 == 0) {
      if (c1(ps) != Status::kSuccess) rc |= 8;
      prod.invokeWaitKernel(cs);
      if (c2(cs) != Status::kSuccess) rc |= 16;
    } else {
      if (c1(ps) != Status::kSuccess) rc |= 8;
      if (c2.runDependent(ps) != Status::kSuccess) rc |= 16;
    }
    CUDA_CHECK(cudaDeviceSynchronize());
    prod.incrementIter(); cons.incrementIter();
    c1.params_.custage.incrementIter(); c2.params_.custage.incrementIter();
  }
  CUDA_CHECK(cudaMemcpy(hY1, Y1, act, cudaMemcpyDeviceToHost));
  CUDA_CHECK(cudaMemcpy(hY2, Y2, act, cudaMemcpyDeviceToHost));
  if (sems_out) cusync_stage_read_semaphores(prod.handle(), sems_out, grid.x * grid.y);
  if (prod.status().code || cons.status().code) rc |= 32;
  c1.destroy(); c2.destroy(); prod.destroy(); cons.destroy();
  cudaFree(X); cudaFree(F1); cudaFree(F2); cudaFree(Y1); cudaFree(Y2);
  cudaStreamDestroy(ps); cudaStreamDestroy(cs);
  return rc;
}

// ---------------------------------------------------------------------------
// User-written policy and tile order (the concept of policies.h:8-13 and
// tile-orders.h:5-16): pairs of adjacent blocks share a semaphore; blocks take
// tiles in reverse order.
// ---------------------------------------------------------------------------
struct PairSync {
  __device__ __host__ PairSync() {}
  __device__ uint32_t waitValue(const dim3&, const dim3&) { return 2; }
  __device__ uint32_t postValue(const dim3&, const dim3&) { return 1; }
  __device__ uint32_t tileIndex(const dim3& tile, const dim3&) { return tile.x / 2; }
  __device__ bool isSync(const dim3&, const dim3&) { return true; }
};
struct ReverseOrder : public GenericTileOrder<ReverseOrder> {
  __device__ __host__ uint32_t blockIndex(const dim3& grid, const dim3& block) { return grid.x - 1 - block.x; }
  __device__ __host__ dim3 tileToBlock(const dim3& tile) { return tile; }
};

API int api_custom_policy_and_order(int blocks, uint32_t* order_out_x, uint32_t* sems_out) {
  using Prod = CuStage<ReverseOrder, NoSync, PairSync>;
  using Cons = CuStage<ReverseOrder, PairSync, NoSync>;
  size_t size = (size_t)blocks * 128;
  unsigned *a1, *a2, *a3;
  CUDA_CHECK(cudaMalloc(&a1, size * 4)); CUDA_CHECK(cudaMalloc(&a2, size * 4)); CUDA_CHECK(cudaMalloc(&a3, size * 4));
  std::vector<unsigned> host(size);
  for (size_t i = 0; i < size; i++) host[i] = (unsigned)(i * 7 + 1);
  CUDA_CHECK(cudaMemcpy(a1, host.data(), size * 4, cudaMemcpyHostToDevice));
  CUDA_CHECK(cudaMemset(a2, 0xff, size * 4)); CUDA_CHECK(cudaMemset(a3, 0xff, size * 4));
  dim3 threads(128), grid(blocks);
  Prod prod(grid, threads, NoSync(), PairSync());
  Cons cons(grid, threads, PairSync(), NoSync());
  int rc = 0;
  if (prod.createStatus() != CuSyncSuccess) rc |= 1;
  if (CuSync::setProducerConsumerPair(prod, cons) != CuSyncSuccess) rc |= 2;
  cudaStream_t ps, cs;
  CUDA_CHECK(cudaStreamCreateWithFlags(&ps, cudaStreamNonBlocking));
  CUDA_CHECK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
  CuSyncTest test(1);
  copyKernel<Prod><<<grid, threads, 0, ps>>>(test, prod, -1, a1, a2);
  prod.invokeWaitKernel(cs);
  copyKernel<Cons><<<grid, threads, 0, cs>>>(test, cons, -1, a2, a3);
  CUDA_CHECK(cudaDeviceSynchronize());
  std::vector<unsigned> got(size);
  CUDA_CHECK(cudaMemcpy(got.data(), a3, size * 4, cudaMemcpyDeviceToHost));
  if (memcmp(got.data(), host.data(), size * 4) != 0) rc |= 4;
  std::vector<cusync_dim3_t> order(blocks);
  cusync_stage_read_tile_order(prod.handle(), order.data(), blocks);
  for (int i = 0; i < blocks; i++) order_out_x[i] = order[i].x;
  cusync_stage_read_semaphores(prod.handle(), sems_out, blocks);
  if (prod.status().code || cons.status().code) rc |= 8;
  test.destroy(); prod.destroy(); cons.destroy();
  cudaFree(a1); cudaFree(a2); cudaFree(a3); cudaStreamDestroy(ps); cudaStreamDestroy(cs);
  return rc;
}

// A tile order that maps two blocks to one slot must be reported.
struct BrokenOrder : public GenericTileOrder<BrokenOrder> {
  __device__ __host__ uint32_t blockIndex(const dim3&, const dim3& block) { return block.x / 2; }
  __device__ __host__ dim3 tileToBlock(const dim3& tile) { return tile; }
};
API int api_broken_order_status() {
  CuStage<BrokenOrder, NoSync, TileSync<IdentityOrder, 1, 1>> s(dim3(8), dim3(1), NoSync(), TileSync<IdentityOrder, 1, 1>());
  int rc = s.createStatus();
  s.destroy();
  return rc;
}

// ---------------------------------------------------------------------------
// Bounded wait: a consumer whose producer never runs must come back with a
// timeout record instead of hanging.  Four small blocks, 20 ms bound.
// ---------------------------------------------------------------------------
API int api_wait_times_out(cusync_status_t* status_out, float* elapsed_ms) {
  using Sync = TileSync<IdentityOrder, 1, 1>;
  using Prod = CuStage<IdentityOrder, NoSync, Sync>;
  using Cons = CuStage<IdentityOrder, Sync, NoSync>;
  dim3 threads(128), grid(4);
  Prod prod(grid, threads, NoSync(), Sync());
  Cons cons(grid, threads, Sync(), NoSync());
  CuSync::setProducerConsumerPair(prod, cons);
  cons.setTimeoutNs(20ull * 1000 * 1000);
  unsigned *a, *b;
  CUDA_CHECK(cudaMalloc(&a, 4 * 128 * 4)); CUDA_CHECK(cudaMalloc(&b, 4 * 128 * 4));
  CUDA_CHECK(cudaMemset(a, 0, 4 * 128 * 4));
  CuSyncTest test(1);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0);
  copyKernel<Cons><<<grid, threads>>>(test, cons, -1, a, b);   // the producer kernel is never launched
  cudaEventRecord(e1);
  cudaError_t err = cudaDeviceSynchronize();
  cudaEventElapsedTime(elapsed_ms, e0, e1);
  *status_out = cons.status();
  int rc = err == cudaSuccess ? 0 : 1;
  // the stage is reusable after reset
  if (cons.reset() != CuSyncSuccess) rc |= 2;
  CUDA_CHECK(cudaDeviceSynchronize());
  if (cons.status().code != 0) rc |= 4;
  test.destroy(); prod.destroy(); cons.destroy(); cudaFree(a); cudaFree(b);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  return rc;
}

// Host-only checks that need no device work.
API int api_error_codes() {
  int rc = 0;
  if ((int)CuSyncSuccess != 5 || (int)CuSyncErrorNotProducer != 0 || (int)CuSyncErrorCUDAError != 4) rc |= 1;
  if ((int)NoAtomicAdd != 1 || (int)AvoidWaitKernel != 2 || (int)AvoidCustomOrder != 4 || (int)ReorderTileLoads != 8) rc |= 2;
  return rc;
}
