// The attention block of one tensor-parallel shard as a three-stage CuSync chain, plus the same three kernels
// in stream order: QKV projection (producer, ConsecutiveSync out) -> decode attention (waits and posts) ->
// output projection (RowSync in).  Stage typing and the run loop follow the reference driver
// src/ml-bench/transformer/attention.cu (XQKVCuStage ... XW12CuStage :105-118; runAttentionCuSync :706-833: each
// stage on its own stream, a wait kernel before every dependent stage, incrementIter at the end).  Unlike the
// reference's chain, the middle stage is a real attention with heads and an fp32 softmax over a K/V cache.
// Host-only code over the library's own C ABI.
#include <cuda_fp16.h>

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

int cusync_attn_block_run_dependent(cusync_attn_block_t* b, cusync_stream_t stream) {
  if (!b) return CUSYNC_ERROR_NOT_INITIALIZED;
  // One stream: each dependent stage is launched as a programmatic dependent of the stage ahead of it.
  if (!b->order.begin(stream)) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  int rc = cusync_gemm_run(b->qkv[0], stream);
  if (rc == CUSYNC_SUCCESS) rc = cusync_attn_run_dependent(b->attn[0], stream);
  if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run_dependent(b->proj[0], stream);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!b->order.end(stream)) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < 3; i++) cusync_stage_increment_iter(b->stages[i]);
  return rc;
}

// ---- prompt phase: the reference's four-GEMM chain ---------------------------------------------------------
// attention.cu:272-276 for seqlen = 0 and a batch of 512 to 2048 prompt tokens: XQKV = X Wqkv; S = Q K^T;
// O = S V; Y = O Wo, with Q, K, V the three thirds of XQKV's columns and no softmax (the reference has none,
// attention.cu:445-509).  Four stages on four streams, a wait kernel before each dependent one (:792-811).
// What the reference's policies leave open is closed here: S = Q K^T also reads K rows that OTHER row panels of
// the first GEMM produce, and O = S V reads all of V; both B operands are waited for through the first stage's
// ConsecutiveSync semaphores (cusync_gemm_desc_t.b_stage).
struct cusync_attn_prompt {
  cusync_attn_prompt_desc_t desc;
  cusync_stage_t* stages[4];
  cusync_stage_t* plain_stages[4];
  cusync_gemm_plan_t* gemm[2][4];     // [0] synchronised, [1] stream-ordered
  RunOrder order;
};

namespace {
void destroy_prompt(cusync_attn_prompt* b) {
  for (int arm = 0; arm < 2; arm++)
    for (int i = 0; i < 4; i++)
      if (b->gemm[arm][i]) cusync_gemm_plan_destroy(b->gemm[arm][i]);
  for (int i = 0; i < 4; i++) {
    if (b->stages[i]) cusync_stage_destroy(b->stages[i]);
    if (b->plain_stages[i]) cusync_stage_destroy(b->plain_stages[i]);
  }
  b->order.destroy();
  delete b;
}
}  // namespace

int cusync_attn_prompt_create(cusync_attn_prompt_t** out, const cusync_attn_prompt_desc_t* desc) {
  if (!out || !desc) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_attn_prompt_desc_t& d = *desc;
  if (d.batch <= 0 || d.hidden <= 0 || d.heads <= 0 || d.out_features <= 0 || d.model_hidden <= 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (!d.x || !d.w_qkv || !d.w_o || !d.qkv || !d.s || !d.o || !d.y) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const int hd = d.heads * 128;               // columns of each of Q, K, V in this shard
  constexpr int kTile = 256;
  // the CTA-pair kernels (256-column tiles) carry the chain: more than two row tiles, thirds in whole tiles,
  // and the ConsecutiveSync group (H / 8 / tile) equal to the tiles of one third
  if (d.batch <= 256 || d.batch % 64 || hd % kTile || d.model_hidden / 8 != hd) return CUSYNC_ERROR_UNSUPPORTED;

  cusync_attn_prompt* b = new (std::nothrow) cusync_attn_prompt();
  if (!b) return CUSYNC_ERROR_CUDA;
  std::memset(b, 0, sizeof(*b));
  b->desc = d;
  const uint32_t tiles_m = static_cast<uint32_t>((d.batch + 127) / 128);
  const uint32_t third_tiles = static_cast<uint32_t>(hd / kTile);
  const uint32_t s_tiles = static_cast<uint32_t>((d.batch + kTile - 1) / kTile);
  const cusync_dim3_t grids[4] = {{3 * third_tiles, tiles_m, 1}, {s_tiles, tiles_m, 1}, {third_tiles, tiles_m, 1},
                                  {static_cast<uint32_t>((d.out_features + kTile - 1) / kTile), tiles_m, 1}};
  const cusync_dim3_t ts = {1, 1, 1};
  cusync_policy_t none, thirds, rows_s, rows_o;
  std::memset(&none, 0, sizeof(none));
  none.tile_m = none.tile_n = 1;
  // ConsecutiveSync<TransposeXYOrder, H, 128, 256> (attention.cu:51-70, 105-110)
  std::memset(&thirds, 0, sizeof(thirds));
  thirds.kind = CUSYNC_POLICY_CONSECUTIVETILESYNC; thirds.order = CUSYNC_ORDER_TRANSPOSE_XY;
  thirds.tile_m = 128; thirds.tile_n = kTile; thirds.p0 = static_cast<uint32_t>(d.model_hidden);
  // RowSync<128>: a row panel of S / of O is complete when all of its column tiles are (Sync2 / Sync1, :113-117)
  std::memset(&rows_s, 0, sizeof(rows_s));
  rows_s.kind = CUSYNC_POLICY_ROWSYNC; rows_s.order = CUSYNC_ORDER_TRANSPOSE_XY;
  rows_s.tile_m = 128; rows_s.tile_n = kTile; rows_s.wait_value = s_tiles; rows_s.post_value = 1;
  rows_o = rows_s;
  rows_o.wait_value = third_tiles;
  const cusync_policy_t* in[4] = {&none, &thirds, &rows_s, &rows_o};
  const cusync_policy_t* outp[4] = {&thirds, &rows_s, &rows_o, &none};
  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < 4 && rc == CUSYNC_SUCCESS; i++) {
    rc = cusync_stage_create(&b->stages[i], grids[i], ts, CUSYNC_ORDER_TRANSPOSE_XY, in[i], outp[i], CUSYNC_OPT_NONE);
    if (rc == CUSYNC_SUCCESS)
      rc = cusync_stage_create(&b->plain_stages[i], grids[i], ts, CUSYNC_ORDER_TRANSPOSE_XY, &none, &none, CUSYNC_OPT_NONE);
  }
  for (int i = 0; i < 3 && rc == CUSYNC_SUCCESS; i++) rc = cusync_stage_link(b->stages[i], b->stages[i + 1]);

  // Semaphore of (row block r, third t) of the first stage: first + r * stride
  const uint32_t gx0 = grids[0].x, gy0 = grids[0].y;
  const uint32_t k_first = cusync::eval::tileIndex(thirds, 0, static_cast<uint32_t>(hd), gx0, gy0);
  const uint32_t v_first = cusync::eval::tileIndex(thirds, 0, static_cast<uint32_t>(2 * hd), gx0, gy0);
  const uint32_t stride = tiles_m > 1 ? cusync::eval::tileIndex(thirds, 128, static_cast<uint32_t>(hd), gx0, gy0) - k_first : 1;
  const __half* qkv = static_cast<const __half*>(d.qkv);

  for (int arm = 0; arm < 2 && rc == CUSYNC_SUCCESS; arm++) {
    cusync_stage_t* const* st = arm == 0 ? b->stages : b->plain_stages;
    cusync_gemm_desc_t g;
    // XQKV = X Wqkv
    std::memset(&g, 0, sizeof(g));
    g.m = d.batch; g.n = 3 * hd; g.k = d.hidden;
    g.a = d.x; g.lda = d.hidden; g.b = d.w_qkv; g.ldb = 3 * hd; g.d = d.qkv; g.ldd = 3 * hd;
    g.b_layout = CUSYNC_B_ROW_MAJOR_KN; g.tile_n = kTile; g.split_k = 1; g.cta_pair = 2; g.stage = st[0];
    rc = cusync_gemm_plan_create(&b->gemm[arm][0], &g);
    if (rc != CUSYNC_SUCCESS) break;
    // S = Q K^T: A = the Q third of XQKV, B = the K third read as an [n, k] matrix
    std::memset(&g, 0, sizeof(g));
    g.m = d.batch; g.n = d.batch; g.k = hd;
    g.a = qkv; g.lda = 3 * hd; g.b = qkv + hd; g.ldb = 3 * hd; g.d = d.s; g.ldd = d.batch;
    g.b_layout = CUSYNC_B_ROW_MAJOR_NK; g.tile_n = kTile; g.split_k = 1; g.cta_pair = 2; g.stage = st[1];
    if (arm == 0) { g.b_stage = b->stages[0]; g.b_sem_first = k_first; g.b_sem_stride = stride; g.b_sem_value = third_tiles; }
    rc = cusync_gemm_plan_create(&b->gemm[arm][1], &g);
    if (rc != CUSYNC_SUCCESS) break;
    // O = S V: B = the V third of XQKV, a [k, n] matrix whose k runs over the tokens
    std::memset(&g, 0, sizeof(g));
    g.m = d.batch; g.n = hd; g.k = d.batch;
    g.a = d.s; g.lda = d.batch; g.b = qkv + 2 * hd; g.ldb = 3 * hd; g.d = d.o; g.ldd = hd;
    g.b_layout = CUSYNC_B_ROW_MAJOR_KN; g.tile_n = kTile; g.split_k = 1; g.cta_pair = 2; g.stage = st[2];
    if (arm == 0) { g.b_stage = b->stages[0]; g.b_sem_first = v_first; g.b_sem_stride = stride; g.b_sem_value = third_tiles; }
    rc = cusync_gemm_plan_create(&b->gemm[arm][2], &g);
    if (rc != CUSYNC_SUCCESS) break;
    // Y = O Wo
    std::memset(&g, 0, sizeof(g));
    g.m = d.batch; g.n = d.out_features; g.k = hd;
    g.a = d.o; g.lda = hd; g.b = d.w_o; g.ldb = d.out_features; g.d = d.y; g.ldd = d.out_features;
    g.b_layout = CUSYNC_B_ROW_MAJOR_KN; g.tile_n = kTile; g.split_k = 1; g.cta_pair = 2; g.stage = st[3];
    rc = cusync_gemm_plan_create(&b->gemm[arm][3], &g);
  }
  if (rc == CUSYNC_SUCCESS && !b->order.create()) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  if (rc != CUSYNC_SUCCESS) { destroy_prompt(b); return rc; }
  *out = b;
  return CUSYNC_SUCCESS;
}

int cusync_attn_prompt_destroy(cusync_attn_prompt_t* b) {
  if (!b) return CUSYNC_ERROR_NOT_INITIALIZED;
  destroy_prompt(b);
  return CUSYNC_SUCCESS;
}

int cusync_attn_prompt_run_stream_ordered(cusync_attn_prompt_t* b, cusync_stream_t stream) {
  if (!b) return CUSYNC_ERROR_NOT_INITIALIZED;
  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < 4 && rc == CUSYNC_SUCCESS; i++) rc = cusync_gemm_run(b->gemm[1][i], stream);
  return rc;
}

int cusync_attn_prompt_run_cusync(cusync_attn_prompt_t* b, const cusync_stream_t* streams) {
  if (!b || !streams) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!b->order.begin(streams[0])) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < 4 && rc == CUSYNC_SUCCESS; i++) {
    if (i > 0) rc = cusync_stage_invoke_wait_kernel(b->stages[i - 1], streams[i]);
    if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run(b->gemm[0][i], streams[i]);
  }
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!b->order.end(streams[3])) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < 4; i++) cusync_stage_increment_iter(b->stages[i]);
  return rc;
}

int cusync_attn_prompt_run_dependent(cusync_attn_prompt_t* b, cusync_stream_t stream) {
  if (!b) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!b->order.begin(stream)) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  int rc = CUSYNC_SUCCESS;
  for (int i = 0; i < 4 && rc == CUSYNC_SUCCESS; i++)
    rc = i == 0 ? cusync_gemm_run(b->gemm[0][i], stream) : cusync_gemm_run_dependent(b->gemm[0][i], stream);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!b->order.end(stream)) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  for (int i = 0; i < 4; i++) cusync_stage_increment_iter(b->stages[i]);
  return rc;
}

cusync_stage_t* cusync_attn_prompt_stage(cusync_attn_prompt_t* b, int which) {
  if (!b || which < 0 || which > 3) return nullptr;
  return b->stages[which];
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
