// Chain of 3x3 convolutions wired through CuSync stages, plus the stream-ordered baseline built from the same
// kernels: the flow of the reference driver src/ml-bench/volta_conv2d/resnet.cu (stage typing :107-116, the
// baseline loop that runs the convolutions back to back on one stream, and the CuSync loop that puts each
// convolution on its own stream behind a wait kernel and increments the stages' iterations afterwards).
// Host-only code over the library's own C ABI.  Doing the launches here keeps a whole chain at a handful of
// microseconds of host time, which matters for these short kernels.
#include <cuda_runtime.h>

#include <cstring>
#include <new>

#include "common.cuh"

namespace { constexpr int kMaxConvs = 8; }

struct cusync_conv_chain {
  cusync_conv_chain_desc_t desc;
  int num;
  cusync_stage_t* stages[kMaxConvs];
  cusync_conv2d_plan_t* sync[kMaxConvs];    // convolution i with its stage
  cusync_conv2d_plan_t* plain[kMaxConvs];   // the same kernel without tile synchronisation
  int sync_ctas;                            // blocks per synchronised convolution
  bool wait_kernels;                        // false: every stage fits on the device at once
  cudaEvent_t fork;                         // orders the resets of a replayable run before every stage
  RunOrder order;                           // run r + 1 starts after run r has finished (activations are reused)
};

namespace {

void destroy_all(cusync_conv_chain* c) {
  for (int i = 0; i < c->num; i++) {
    if (c->sync[i]) cusync_conv2d_plan_destroy(c->sync[i]);
    if (c->plain[i]) cusync_conv2d_plan_destroy(c->plain[i]);
    if (c->stages[i]) cusync_stage_destroy(c->stages[i]);
  }
  if (c->fork) cudaEventDestroy(c->fork);
  c->order.destroy();
  delete c;
}

}  // namespace

extern "C" {

int cusync_conv_chain_create(cusync_conv_chain_t** out, const cusync_conv_chain_desc_t* desc) {
  if (!out || !desc) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_conv_chain_desc_t& d = *desc;
  if (d.num_convs < 2 || d.num_convs > kMaxConvs || !d.filters || !d.activations) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.n <= 0 || d.h <= 0 || d.w <= 0 || d.channels <= 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  for (int i = 0; i < d.num_convs; i++)
    if (!d.filters[i] || !d.activations[i] || !d.activations[i + 1]) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const int rows = cusync_conv2d_tile_rows_hw(d.h, d.w);
  if (rows == 0 || d.channels % 64) return CUSYNC_ERROR_UNSUPPORTED;

  cusync_conv_chain* c = new (std::nothrow) cusync_conv_chain();
  if (!c) return CUSYNC_ERROR_CUDA;
  std::memset(c, 0, sizeof(*c));
  c->desc = d;
  c->num = d.num_convs;

  // Every convolution has the same tile grid: (K / tile_n, N * H / rows, 1); tiles are rows * W pixels by tile_n
  // channels (64 for the 64-channel layer, 64 to 256 otherwise).
  const int tile_n = cusync_conv2d_default_tile_n(d.n, d.h, d.w, d.channels, d.channels);
  if (tile_n <= 0) return CUSYNC_ERROR_UNSUPPORTED;
  const cusync_dim3_t grid = {static_cast<uint32_t>(d.channels / tile_n), static_cast<uint32_t>(d.n * (d.h / rows)), 1};
  const cusync_dim3_t ts = {1, 1, 1};
  const uint32_t tile_m = static_cast<uint32_t>(rows * d.w);
  cusync_policy_t none, post, wait;
  std::memset(&none, 0, sizeof(none));
  none.tile_m = none.tile_n = 1;
  std::memset(&post, 0, sizeof(post));
  post.kind = CUSYNC_POLICY_TILESYNC; post.order = CUSYNC_ORDER_TRANSPOSE_XY;
  post.tile_m = tile_m; post.tile_n = static_cast<uint32_t>(tile_n); post.wait_value = 1; post.post_value = 1;
  wait = post;
  wait.kind = CUSYNC_POLICY_CONV2DTILESYNC; wait.p0 = 9;          // R * S (resnet.cu:113-116)

  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  // Left to choose, every synchronised convolution gets the whole device, except in chains of three or more
  // 64-channel convolutions (the slab kernel), where each gets half of it: two adjacent stages are then resident
  // together and run as a pipeline over the semaphores, and a stage's tiles spread over more rounds (224 tiles are
  // 3.03 rounds of 74 blocks but 1.51, run as 2, of 148).  Measured with all streams meeting before every step,
  // eight 56 x 56 x 64 images, four convolutions: 41 us with half the device per stage, 45.5 us with all of it,
  // 49 us with a quarter each, against 44.4 us stream-ordered; two images 32 / 33-39 / 35-40 against 39 us.  Chains
  // of the general kernel (128 channels and more) and chains of two convolutions measured best on the whole device.
  // Where the blocks of all stages fit on the device at once no wait is needed before a launch (the reference's
  // AvoidWaitKernel case, cusync.h:61-62); otherwise the next stage becomes resident as the previous one's blocks
  // retire.
  const uint32_t tiles = grid.x * grid.y;
  const bool slab = d.channels == 64;
  const uint32_t cap = d.max_ctas > 0 ? static_cast<uint32_t>(d.max_ctas)
                                      : (slab && d.num_convs >= 3 ? static_cast<uint32_t>(sms > 1 ? sms / 2 : 1)
                                                                  : static_cast<uint32_t>(sms));
  const uint32_t blocks = tiles < cap ? tiles : cap;
  c->sync_ctas = static_cast<int>(cap);
  c->wait_kernels = static_cast<uint64_t>(blocks) * d.num_convs > static_cast<uint64_t>(sms);
  // (where a wait is needed it is a stream memory operation, not a kernel launch: these kernels are short)
  const int opts = c->wait_kernels ? CUSYNC_OPT_STREAM_WAIT : CUSYNC_OPT_AVOID_WAIT_KERNEL;

  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++)
    rc = cusync_stage_create(&c->stages[i], grid, ts, CUSYNC_ORDER_TRANSPOSE_XY, i == 0 ? &none : &wait,
                             i + 1 == c->num ? &none : &post, opts);
  for (int i = 0; i + 1 < c->num && rc == CUSYNC_SUCCESS; i++) rc = cusync_stage_link(c->stages[i], c->stages[i + 1]);
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++) {
    cusync_conv2d_desc_t cd;
    std::memset(&cd, 0, sizeof(cd));
    cd.n = d.n; cd.h = d.h; cd.w = d.w; cd.c = d.channels; cd.k = d.channels;
    cd.r = 3; cd.s = 3; cd.stride = 1; cd.pad = 1;
    cd.x = d.activations[i]; cd.filter = d.filters[i]; cd.y = d.activations[i + 1];
    cd.epilogue = d.relu ? CUSYNC_EPILOGUE_RELU : CUSYNC_EPILOGUE_NONE;
    cd.max_ctas = c->sync_ctas;
    cd.stage = c->stages[i];
    rc = cusync_conv2d_plan_create(&c->sync[i], &cd);
    cd.max_ctas = d.max_ctas;        // the stream-ordered convolutions each take the whole device
    cd.stage = nullptr;
    if (rc == CUSYNC_SUCCESS) rc = cusync_conv2d_plan_create(&c->plain[i], &cd);
  }
  if (rc == CUSYNC_SUCCESS && cudaEventCreateWithFlags(&c->fork, cudaEventDisableTiming) != cudaSuccess) {
    (void)cudaGetLastError();
    c->fork = nullptr;
    rc = CUSYNC_ERROR_CUDA;
  }
  if (rc == CUSYNC_SUCCESS && !c->order.create()) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  if (rc != CUSYNC_SUCCESS) { destroy_all(c); return rc; }
  *out = c;
  return CUSYNC_SUCCESS;
}

int cusync_conv_chain_destroy(cusync_conv_chain_t* c) {
  if (!c) return CUSYNC_ERROR_NOT_INITIALIZED;
  destroy_all(c);
  return CUSYNC_SUCCESS;
}

int cusync_conv_chain_run_stream_ordered(cusync_conv_chain_t* c, cusync_stream_t stream) {
  if (!c) return CUSYNC_ERROR_NOT_INITIALIZED;
  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++) rc = cusync_conv2d_run(c->plain[i], stream);
  return rc;
}

int cusync_conv_chain_run_cusync(cusync_conv_chain_t* c, const cusync_stream_t* streams) {
  if (!c || !streams) return CUSYNC_ERROR_NOT_INITIALIZED;
  int rc = CUSYNC_SUCCESS;
  // Every stream waits for the previous run, not only the first: without wait kernels a dependent convolution
  // would otherwise start while the previous run (which may have gone to other streams: run_dependent) still
  // draws tiles from the same stage.
  for (int i = 0; i < c->num; i++)
    if (i == 0 || streams[i] != streams[0])
      if (!c->order.begin(streams[i])) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++) {
    // a dependent convolution is launched only once every block of its producer is resident
    if (i > 0 && c->wait_kernels) rc = cusync_stage_invoke_wait_kernel(c->stages[i - 1], streams[i]);
    if (rc == CUSYNC_SUCCESS) rc = cusync_conv2d_run(c->sync[i], streams[i]);
  }
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!c->order.end(streams[c->num - 1])) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < c->num; i++) cusync_stage_increment_iter(c->stages[i]);
  return rc;
}

int cusync_conv_chain_run_dependent(cusync_conv_chain_t* c, cusync_stream_t stream) {
  if (!c) return CUSYNC_ERROR_NOT_INITIALIZED;
  // One stream: convolution i + 1 is launched as a programmatic dependent of convolution i, so it becomes
  // resident once every block of convolution i is, and waits for its tiles through the semaphores.
  int rc = CUSYNC_SUCCESS;
  if (!c->order.begin(stream)) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++)
    rc = i == 0 ? cusync_conv2d_run(c->sync[i], stream) : cusync_conv2d_run_dependent(c->sync[i], stream);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!c->order.end(stream)) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < c->num; i++) cusync_stage_increment_iter(c->stages[i]);
  return rc;
}

int cusync_conv_chain_run_cusync_replayable(cusync_conv_chain_t* c, const cusync_stream_t* streams) {
  if (!c || !streams) return CUSYNC_ERROR_NOT_INITIALIZED;
  // Every run starts from freshly zeroed semaphores at iteration 1, so the recorded work does not depend on
  // how often it ran before.  The resets go to streams[0]; the other streams wait for them through an event
  // (in a stream capture this is the fork).
  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++) rc = cusync_stage_reset(c->stages[i], streams[0]);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (cudaEventRecord(c->fork, reinterpret_cast<cudaStream_t>(streams[0])) != cudaSuccess) return CUSYNC_ERROR_CUDA;
  for (int i = 1; i < c->num; i++)
    if (cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(streams[i]), c->fork, 0) != cudaSuccess) return CUSYNC_ERROR_CUDA;
  for (int i = 0; i < c->num && rc == CUSYNC_SUCCESS; i++) {
    if (i > 0 && c->wait_kernels) rc = cusync_stage_invoke_wait_kernel(c->stages[i - 1], streams[i]);
    if (rc == CUSYNC_SUCCESS) rc = cusync_conv2d_run(c->sync[i], streams[i]);
  }
  return rc;
}

cusync_stage_t* cusync_conv_chain_stage(cusync_conv_chain_t* c, int which) {
  if (!c || which < 0 || which >= c->num) return nullptr;
  return c->stages[which];
}

int cusync_conv_chain_uses_wait_kernels(const cusync_conv_chain_t* c) { return c && c->wait_kernels ? 1 : 0; }

}  // extern "C"
