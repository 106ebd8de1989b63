// Runs the REFERENCE's own CuStage / wait / post / tile code on the GPU and
// prints what it produced, one JSON object per case.  TEST INFRASTRUCTURE ONLY.
// Nothing of the reference is copied here: its headers and src/cusync.cu are
// compiled where they lie (see oracle/Makefile, target `_ref`), and this file
// only drives them.  Every grid is small enough (<= 512 blocks of 32 threads
// for producer and consumer together) that all blocks are resident at once,
// so the reference's unbounded spin loops cannot starve a producer block.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cusync/cusync.h>

namespace cusync {
// The reference befriends a class of this name (cusync.h:120); defining it
// here gives read access to the private device pointers.
class CuSyncTest {
public:
  template <class Stage> static dim3* tileOrder(Stage& s) { return s.tileOrder; }
  template <class Stage> static uint32_t* semsToPost(Stage& s) { return (uint32_t*)s.tileStatusWrite_; }
  template <class Stage> static int iter(Stage& s) { return s.iter; }
};
}
using namespace cusync;

struct WaitRecord { uint32_t idx, expect, seen; };

// Stage kernel: block = one tile.
// gemmShaped = 0: the copy-kernel protocol of tests/simple-test.cu:14-27 -- wait(tile); post(tile) with the
//   tile exactly as tile() returned it.
// gemmShaped = 1: producer posts {m*TM, n*TN, 0}; consumer walks K in steps of BK and waits the way the
//   reference main loop does (z = 1 on the first step, 0 afterwards).
template <class Stage>
__global__ void stageKernel(Stage stage, int gemmShaped, uint32_t tm, uint32_t tn, uint32_t kExtent, uint32_t bk,
                            uint32_t* ticketTile, WaitRecord* waits, uint32_t waitsPerTile) {
  __shared__ int tileSh[3];
  dim3 t = stage.tile((dim3*)&tileSh[0]);
  uint32_t linear = blockIdx.x + blockIdx.y * gridDim.x + blockIdx.z * gridDim.x * gridDim.y;
  if (threadIdx.x == 0 && ticketTile) {
    ticketTile[3 * linear + 0] = t.x; ticketTile[3 * linear + 1] = t.y; ticketTile[3 * linear + 2] = t.z;
  }
  uint32_t tileLinear = t.x + t.y * gridDim.x;
  if (!gemmShaped) {
    if (stage.isConsumer()) {
      stage.wait(t);
      if (threadIdx.x == 0 && waits) {
        WaitRecord r;
        r.idx = stage.waitTileIndex(t); r.expect = stage.expectedWaitValue(t); r.seen = stage.waitSemValue(t);
        waits[tileLinear * waitsPerTile] = r;
      }
    }
    if (stage.isProducer()) stage.post(t);
    return;
  }
  if (stage.isConsumer()) {
    uint32_t n = 0;
    for (uint32_t k = 0; k < kExtent; k += bk) {
      dim3 w = {t.y * tm, k, k == 0 ? 1u : 0u};
      stage.wait(w);
      if (threadIdx.x == 0 && waits && n < waitsPerTile) {
        // what the wait resolved to, recorded after it returned
        WaitRecord r;
        r.idx = stage.waitTileIndex(w); r.expect = stage.expectedWaitValue(w); r.seen = stage.waitSemValue(w);
        waits[tileLinear * waitsPerTile + n] = r;
      }
      n++;
    }
  }
  if (stage.isProducer()) stage.post({t.y * tm, t.x * tn, 0});
}

template <class Prod, class Cons, class Policy>
static void runCase(const char* name, int gemmShaped, dim3 gridP, dim3 gridC, uint32_t tm, uint32_t tn,
                    uint32_t bk, Policy policy, int iters) {
  Prod prod(gridP, {1, 1, 1}, NoSync(), policy);
  Cons cons(gridC, {1, 1, 1}, policy, NoSync());
  CuSync::setProducerConsumerPair(prod, cons);
  cudaStream_t ps, cs;
  CUDA_CHECK(cudaStreamCreateWithFlags(&ps, cudaStreamNonBlocking));
  CUDA_CHECK(cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking));
  uint32_t nP = gridP.x * gridP.y * gridP.z, nC = gridC.x * gridC.y * gridC.z;
  uint32_t kExtent = gridP.x * tn, waitsPerTile = gemmShaped ? (kExtent + bk - 1) / bk : 1;
  WaitRecord* dWaits; uint32_t* dTicket;
  CUDA_CHECK(cudaMalloc(&dWaits, sizeof(WaitRecord) * nC * waitsPerTile));
  CUDA_CHECK(cudaMalloc(&dTicket, sizeof(uint32_t) * 3 * nP));
  std::vector<WaitRecord> hWaits(nC * waitsPerTile);
  std::vector<uint32_t> hSems(nP), hTicket(3 * nP);
  std::vector<dim3> hOrder(nP);
  for (int it = 1; it <= iters; it++) {
    CUDA_CHECK(cudaMemset(dWaits, 0xff, sizeof(WaitRecord) * nC * waitsPerTile));
    stageKernel<Prod><<<gridP, 32, 0, ps>>>(prod, gemmShaped, tm, tn, kExtent, bk, dTicket, nullptr, 0);
    prod.invokeWaitKernel(cs);
    stageKernel<Cons><<<gridC, 32, 0, cs>>>(cons, gemmShaped, tm, tn, kExtent, bk, nullptr, dWaits, waitsPerTile);
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(hSems.data(), CuSyncTest::semsToPost(prod), 4 * nP, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(hWaits.data(), dWaits, sizeof(WaitRecord) * hWaits.size(), cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(hOrder.data(), CuSyncTest::tileOrder(prod), sizeof(dim3) * nP, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(hTicket.data(), dTicket, 4 * 3 * nP, cudaMemcpyDeviceToHost));
    printf("{\"case\":\"%s\",\"gemm_shaped\":%d,\"iter\":%d,\"grid_p\":[%u,%u,%u],\"grid_c\":[%u,%u,%u],\"tm\":%u,\"tn\":%u,\"bk\":%u,",
           name, gemmShaped, it, gridP.x, gridP.y, gridP.z, gridC.x, gridC.y, gridC.z, tm, tn, bk);
    printf("\"tile_order\":[");
    for (uint32_t i = 0; i < nP; i++) printf("%s[%u,%u,%u]", i ? "," : "", hOrder[i].x, hOrder[i].y, hOrder[i].z);
    printf("],\"sems\":[");
    for (uint32_t i = 0; i < nP; i++) printf("%s%u", i ? "," : "", hSems[i]);
    // consumer waits as a sorted-by-tile list of [idx, expect*iter reached?]; 0xffffffff = no sync at that step
    printf("],\"waits\":[");
    bool first = true;
    for (uint32_t t = 0; t < nC; t++)
      for (uint32_t w = 0; w < waitsPerTile; w++) {
        WaitRecord r = hWaits[t * waitsPerTile + w];
        printf("%s[%u,%u,%u,%u,%u]", first ? "" : ",", t, w, r.idx, r.expect, r.seen);
        first = false;
      }
    printf("]}\n");
    fflush(stdout);
    prod.incrementIter();
    cons.incrementIter();
  }
  CUDA_CHECK(cudaFree(dWaits)); CUDA_CHECK(cudaFree(dTicket));
}

int main() {
  {  // tests/simple-test.cu:107-113 shape, shrunk: 1-D grid, one semaphore per block
    using Sync = TileSync<IdentityOrder, 1, 1>;
    runCase<CuStage<IdentityOrder, NoSync, Sync>, CuStage<IdentityOrder, Sync, NoSync>, Sync>(
        "tilesync_identity_1_1", 0, {64, 1, 1}, {64, 1, 1}, 1, 1, 64, Sync(), 2);
    runCase<CuStage<IdentityOrder, NoSync, Sync, NoAtomicAdd>, CuStage<IdentityOrder, Sync, NoSync>, Sync>(
        "tilesync_identity_1_1_noatomic", 0, {64, 1, 1}, {64, 1, 1}, 1, 1, 64, Sync(), 2);
    runCase<CuStage<IdentityOrder, NoSync, Sync, AvoidCustomOrder>, CuStage<IdentityOrder, Sync, NoSync>, Sync>(
        "tilesync_identity_1_1_nocustomorder", 0, {64, 1, 1}, {64, 1, 1}, 1, 1, 64, Sync(), 1);
  }
  {  // mlp.cu:103-118 stage typing, GEMM grid (tilesN, tilesM, 1)
    using Sync = RowSync<128>;
    runCase<CuStage<TransposeXYOrder, NoSync, Sync>, CuStage<TransposeXYOrder, Sync, NoSync>, Sync>(
        "rowsync_128", 1, {8, 2, 1}, {8, 2, 1}, 128, 128, 64, Sync(8), 3);
    runCase<CuStage<TransposeXYOrder, NoSync, Sync>, CuStage<TransposeXYOrder, Sync, NoSync>, Sync>(
        "rowsync_128_wide", 1, {6, 4, 1}, {12, 4, 1}, 128, 256, 64, Sync(6), 2);
  }
  {
    using Sync = TileSync<TransposeXYOrder, 128, 128>;
    runCase<CuStage<TransposeXYOrder, NoSync, Sync>, CuStage<TransposeXYOrder, Sync, NoSync>, Sync>(
        "tilesync_transpose_128_128", 1, {8, 2, 1}, {8, 2, 1}, 128, 128, 64, Sync(), 3);
    runCase<CuStage<TransposeXYOrder, NoSync, Sync, NoAtomicAdd>, CuStage<TransposeXYOrder, Sync, NoSync>, Sync>(
        "tilesync_transpose_128_128_noatomic", 1, {8, 2, 1}, {8, 2, 1}, 128, 128, 64, Sync(), 2);
  }
  {
    using Sync = TileSync<TransposeXYOrder, 128, 256>;
    runCase<CuStage<TransposeXYOrder, NoSync, Sync>, CuStage<TransposeXYOrder, Sync, NoSync>, Sync>(
        "tilesync_transpose_128_256", 1, {6, 4, 1}, {12, 4, 1}, 128, 256, 64, Sync(), 2);
  }
  return 0;
}
