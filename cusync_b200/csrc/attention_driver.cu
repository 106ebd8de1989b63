// The attention block of one tensor-parallel shard as a three-stage CuSync chain, plus the same three kernels
// in stream order: QKV projection (producer, ConsecutiveSync out) -> decode attention (waits and posts) ->
// output projection (RowSync in).  Stage typing and the run loop follow the reference driver
// src/ml-bench/transformer/attention.cu (XQKVCuStage ... XW12CuStage :105-118; runAttentionCuSync :706-833: each
// stage on its own stream, a wait kernel before every dependent stage, incrementIter at the end).  Unlike the
// reference's chain, the middle stage is a real attention with heads and an fp32 softmax over a K/V cache.
// Host-only code over the library's own C ABI.
#include <cstring>
#include <new>

#include "common.cuh"

struct cusync_attn_block {
  cusync_attn_block_desc_t desc;
  cusync_stage_t* stages[3];          // synchronised chain
  cusync_stage_t* plain_stages[3];    // NoSync stages of the stream-ordered arm (same grids and orders)
  cusync_gemm_plan_t* qkv[2];         // [0] synchronised, [1] stream-ordered
  cusync_attn_plan_t* attn[2];
  cusync_gemm_plan_t* proj[2];
  int tile_n1, tile_n3, split1, split3, kv_splits;
  RunOrder order;                     // run r + 1 starts after run r has finished (qkv and attn_out are reused)
};

namespace {

void destroy_all(cusync_attn_block* b) {
  for (int i = 0; i < 2; i++) {
    if (b->qkv[i]) cusync_gemm_plan_destroy(b->qkv[i]);
    if (b->attn[i]) cusync_attn_plan_destroy(b->attn[i]);
    if (b->proj[i]) cusync_gemm_plan_destroy(b->proj[i]);
  }
  for (int i = 0; i < 3; i++) {
    if (b->stages[i]) cusync_stage_destroy(b->stages[i]);
    if (b->plain_stages[i]) cusync_stage_destroy(b->plain_stages[i]);
  }
  b->order.destroy();
  delete b;
}

}  // namespace

extern "C" {

int cusync_attn_block_create(cusync_attn_block_t** out, const cusync_attn_block_desc_t* desc) {
  if (!out || !desc) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_attn_block_desc_t& d = *desc;
  if (d.batch <= 0 || d.seq < 0 || d.hidden <= 0 || d.heads <= 0 || d.out_features <= 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (!d.x || !d.w_qkv || !d.w_o || !d.qkv || !d.attn_out || !d.y || (d.seq > 0 && (!d.k_cache || !d.v_cache)))
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  const int hd = d.heads * 128;

  cusync_attn_block* b = new (std::nothrow) cusync_attn_block();
  if (!b) return CUSYNC_ERROR_CUDA;
  std::memset(b, 0, sizeof(*b));
  b->desc = d;
  b->tile_n1 = cusync_gemm_default_tile_n(d.batch, 3 * hd, d.hidden, CUSYNC_EPILOGUE_NONE);
  b->split1 = cusync_gemm_default_split_k(d.batch, 3 * hd, d.hidden, CUSYNC_EPILOGUE_NONE, b->tile_n1, 0);
  b->tile_n3 = cusync_gemm_default_tile_n(d.batch, d.out_features, hd, CUSYNC_EPILOGUE_NONE);
  b->split3 = cusync_gemm_default_split_k(d.batch, d.out_features, hd, CUSYNC_EPILOGUE_NONE, b->tile_n3, 0);
  b->kv_splits = d.kv_splits > 0 ? d.kv_splits : cusync_attn_default_splits(d.batch, d.seq, d.heads);

  const uint32_t tiles_m = static_cast<uint32_t>((d.batch + 127) / 128);
  const cusync_dim3_t grids[3] = {
      {static_cast<uint32_t>((3 * hd + b->tile_n1 - 1) / b->tile_n1), tiles_m, static_cast<uint32_t>(b->split1)},
      {static_cast<uint32_t>(d.heads), static_cast<uint32_t>(d.batch), static_cast<uint32_t>(b->kv_splits)},
      {static_cast<uint32_t>((d.out_features + b->tile_n3 - 1) / b->tile_n3), tiles_m, static_cast<uint32_t>(b->split3)}};
  const int orders[3] = {CUSYNC_ORDER_TRANSPOSE_XY, CUSYNC_ORDER_IDENTITY, CUSYNC_ORDER_TRANSPOSE_XY};
  const cusync_dim3_t ts = {1, 1, 1};
  cusync_policy_t none, sync12, sync23;
  std::memset(&none, 0, sizeof(none));
  none.tile_m = none.tile_n = 1;
  // ConsecutiveSync<Order, H, 128, TileN> (attention.cu:51-70, 105-110): the N tiles of one third of the QKV row
  // panel share a semaphore; H is the model's hidden size.
  std::memset(&sync12, 0, sizeof(sync12));
  sync12.kind = CUSYNC_POLICY_CONSECUTIVETILESYNC; sync12.order = CUSYNC_ORDER_TRANSPOSE_XY;
  sync12.tile_m = 128; sync12.tile_n = static_cast<uint32_t>(b->tile_n1); sync12.p0 = static_cast<uint32_t>(d.model_hidden);
  // RowSync<128>(1, 1): the attention stage posts a row panel once, when all of it is written.
  std::memset(&sync23, 0, sizeof(sync23));
  sync23.kind = CUSYNC_POLICY_ROWSYNC; sync23.order = CUSYNC_ORDER_TRANSPOSE_XY;
  sync23.tile_m = 128; sync23.tile_n = 1; sync23.wait_value = 1; sync23.post_value = 1;
  const cusync_policy_t* in[3] = {&none, &sync12, &sync23};
  const cusync_policy_t* outp[3] = {&sync12, &sync23, &none};

  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < 3 && rc == CUSYNC_SUCCESS; i++) {
    // (the waits before the dependent stages are stream memory operations, not kernel launches)
    rc = cusync_stage_create(&b->stages[i], grids[i], ts, orders[i], in[i], outp[i], CUSYNC_OPT_STREAM_WAIT);
    if (rc == CUSYNC_SUCCESS)
      rc = cusync_stage_create(&b->plain_stages[i], grids[i], ts, orders[i], &none, &none, CUSYNC_OPT_NONE);
  }
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_link(b->stages[0], b->stages[1]);
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_link(b->stages[1], b->stages[2]);

  for (int arm = 0; arm < 2 && rc == CUSYNC_SUCCESS; arm++) {
    cusync_stage_t* const* st = arm == 0 ? b->stages : b->plain_stages;
    cusync_gemm_desc_t g;
    std::memset(&g, 0, sizeof(g));
    g.m = d.batch; g.n = 3 * hd; g.k = d.hidden;
    g.a = d.x; g.lda = d.hidden; g.b = d.w_qkv; g.ldb = 3 * hd; g.d = d.qkv; g.ldd = 3 * hd;
    g.b_layout = CUSYNC_B_ROW_MAJOR_KN; g.epilogue = CUSYNC_EPILOGUE_NONE;
    g.tile_n = b->tile_n1; g.split_k = b->split1; g.stage = st[0];
    rc = cusync_gemm_plan_create(&b->qkv[arm], &g);
    if (rc != CUSYNC_SUCCESS) break;
    cusync_attn_desc_t a;
    std::memset(&a, 0, sizeof(a));
    a.batch = d.batch; a.seq = d.seq; a.heads = d.heads; a.head_dim = 128;
    a.qkv = d.qkv; a.ld_qkv = 3 * hd; a.k_cache = d.k_cache; a.v_cache = d.v_cache;
    a.out = d.attn_out; a.ld_out = hd; a.kv_splits = b->kv_splits; a.stage = st[1];
    rc = cusync_attn_plan_create(&b->attn[arm], &a);
    if (rc != CUSYNC_SUCCESS) break;
    std::memset(&g, 0, sizeof(g));
    g.m = d.batch; g.n = d.out_features; g.k = hd;
    g.a = d.attn_out; g.lda = hd; g.b = d.w_o; g.ldb = d.out_features; g.d = d.y; g.ldd = d.out_features;
    g.b_layout = CUSYNC_B_ROW_MAJOR_KN; g.epilogue = CUSYNC_EPILOGUE_NONE;
    g.tile_n = b->tile_n3; g.split_k = b->split3; g.stage = st[2];
    rc = cusync_gemm_plan_create(&b->proj[arm], &g);
  }
  if (rc == CUSYNC_SUCCESS && !b->order.create()) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  if (rc != CUSYNC_SUCCESS) { destroy_all(b); return rc; }
  *out = b;
  return CUSYNC_SUCCESS;
}

int cusync_attn_block_destroy(cusync_attn_block_t* b) {
  if (!b) return CUSYNC_ERROR_NOT_INITIALIZED;
  destroy_all(b);
  return CUSYNC_SUCCESS;
}

int cusync_attn_block_run_stream_ordered(cusync_attn_block_t* b, cusync_stream_t stream) {
  if (!b) return CUSYNC_ERROR_NOT_INITIALIZED;
  int rc = cusync_gemm_run(b->qkv[1], stream);
  if (rc == CUSYNC_SUCCESS) rc = cusync_attn_run(b->attn[1], stream);
  if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run(b->proj[1], stream);
  return rc;
}

int cusync_attn_block_run_cusync(cusync_attn_block_t* b, const cusync_stream_t* streams) {
  if (!b || !streams) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!b->order.begin(streams[0])) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  int rc = cusync_gemm_run(b->qkv[0], streams[0]);
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_invoke_wait_kernel(b->stages[0], streams[1]);
  if (rc == CUSYNC_SUCCESS) rc = cusync_attn_run(b->attn[0], streams[1]);
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_invoke_wait_kernel(b->stages[1], streams[2]);
  if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run(b->proj[0], streams[2]);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!b->order.end(streams[2])) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < 3; i++) cusync_stage_increment_iter(b->stages[i]);
  return rc;
}

cusync_stage_t* cusync_attn_block_stage(cusync_attn_block_t* b, int which) {
  if (!b || which < 0 || which > 2) return nullptr;
  return b->stages[which];
}

int cusync_attn_block_config(const cusync_attn_block_t* b, int32_t* out5) {
  if (!b || !out5) return CUSYNC_ERROR_NOT_INITIALIZED;
  out5[0] = b->tile_n1; out5[1] = b->tile_n3; out5[2] = b->split1; out5[3] = b->split3; out5[4] = b->kv_splits;
  return CUSYNC_SUCCESS;
}

}  // extern "C"
