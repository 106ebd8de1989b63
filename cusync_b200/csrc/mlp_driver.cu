// Tensor-parallel MLP shard driver: two dependent GEMMs wired through CuSync
// stages, plus the stream-ordered baseline built from the same kernels.
// Host-only code over the library's own C ABI; it follows the flow of the
// reference driver src/ml-bench/transformer/mlp.cu (stage typing :103-118,
// grid/sync set-up :1026-1062, runBaselineGPT3 :411-491, runCuSyncGPT3 :645-716).
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

struct cusync_mlp {
  cusync_mlp_desc_t desc;
  int tile_n1, tile_n2;
  int split_k1, split_k2;
  cusync_stage_t* input;        // x_rows: producer-only stage standing for whatever brings X, posted by the caller
  std::vector<uint32_t> x_posted;  // x_rows: per 128-row tile of X, the run its latest post was for
  cusync_stage_t* prod;
  cusync_stage_t* cons;
  cusync_gemm_plan_t* sync1;    // producer GEMM with its stage
  cusync_gemm_plan_t* sync2;    // consumer GEMM with its stage
  cusync_gemm_plan_t* plain1;   // same kernels without tile synchronisation
  cusync_gemm_plan_t* plain2;
  cusync_stage_t* plain_stage1; // NoSync stages carrying the two tile orders for the baseline
  cusync_stage_t* plain_stage2;
  RunOrder order;               // run r + 1 starts after run r has finished (H and Y are reused)
  bool single_grid;             // run_cusync launches both synchronised GEMMs as one persistent grid
  cudaEvent_t joined;           // single grid: lets the consumer stream wait for the launch on the producer stream
  cudaEvent_t reduced;          // overlapped all-reduce: lets the consumer stream wait for the reducer
};

namespace {

// What run_cusync does when the caller leaves the choice open, by model and batch range: the role of the
// reference's per-GPU tuning table (src/ml-bench/transformer/tile_sizes_db.py, applied by eval_mlp.py:141-210),
// which picks tile shapes, split-K and the AvoidWaitKernel / AvoidCustomOrder / ReorderTileLoads switches per
// batch.  Here tile shape and K slices follow from cusync_gemm_default_tile_n / _split_k; the table adds the
// policy, the launch form and the tile orders.  Rows come from interleaved A/B sweeps on B200 (every
// combination against the same stream-ordered layer): RowSync beats TileSync at every batch of both models;
// one persistent grid pays from about twelve row tiles on (+1.5 to +2 points at B = 2048, nothing at 1024, a
// loss at 512 where the first GEMM is a single round); walking the tiles in groups of rows pays from eight row
// tiles on.  Re-measured with the dual GEMM on CTA pairs and the lighter post path: one persistent grid is level
// with two launches at seven and eight row tiles and 2 to 4 % ahead from nine on (B = 1152 ... 1792); at seven and
// eight row tiles the first GEMM's 96 pair tiles are one round of 74 and a tail of 22, and cutting the tail's tiles
// into three K slices (66 units: one short round) brings the one-grid layer from 289-297 to 277-285 us at
// B = 960 and 1024 (with two launches the same split is a loss).  tail_split1 is applied only where the tail's
// units fit one round (see cusync_mlp_create).  LLaMA shard (the fused SwiGLU GEMM on CTA pairs): one grid is level
// with two launches up to eight row tiles and 4 to 6 % ahead from nine on (B = 1152 ... 3072: 150 / 170 / 186 /
// 242 / 373 us against 159 / 182 / 195 / 254 / 388 us at B = 1152 / 1280 / 1536 / 2048 / 3072).
struct ConfigRow { int model; int max_batch; int policy; int single_grid; int group_rows1; int group_rows2; int tail_split1; };
const ConfigRow kConfigTable[] = {
    {CUSYNC_MLP_GPT3, 512, CUSYNC_POLICY_ROWSYNC, 1, 1, 1, 0},
    {CUSYNC_MLP_GPT3, 768, CUSYNC_POLICY_ROWSYNC, 1, 4, 4, 0},
    {CUSYNC_MLP_GPT3, 1024, CUSYNC_POLICY_ROWSYNC, 2, 4, 4, 3},
    {CUSYNC_MLP_GPT3, 1536, CUSYNC_POLICY_ROWSYNC, 2, 4, 4, 0},
    {CUSYNC_MLP_GPT3, 0x7fffffff, CUSYNC_POLICY_ROWSYNC, 2, 4, 8, 0},
    {CUSYNC_MLP_LLAMA, 896, CUSYNC_POLICY_ROWSYNC, 1, 1, 1, 0},
    {CUSYNC_MLP_LLAMA, 1024, CUSYNC_POLICY_ROWSYNC, 1, 1, 4, 0},
    {CUSYNC_MLP_LLAMA, 0x7fffffff, CUSYNC_POLICY_ROWSYNC, 2, 1, 4, 0},
};

const ConfigRow* config_row(int model, int batch) {
  for (const ConfigRow& r : kConfigTable)
    if (r.model == model && batch <= r.max_batch) return &r;
  return nullptr;
}

void fill_gemm1(const cusync_mlp_desc_t& d, int tile_n, int split_k, int tail_split, cusync_stage_t* stage,
                cusync_gemm_desc_t* g) {
  std::memset(g, 0, sizeof(*g));
  g->m = d.batch; g->n = d.ffn; g->k = d.hidden;
  g->a = d.x; g->lda = d.hidden;
  g->b = d.w1; g->ldb = d.ffn;
  g->b2 = d.model == CUSYNC_MLP_LLAMA ? d.v : nullptr;
  g->d = d.h; g->ldd = d.ffn;
  g->b_layout = CUSYNC_B_ROW_MAJOR_KN;
  g->epilogue = d.model == CUSYNC_MLP_LLAMA ? CUSYNC_EPILOGUE_SILU_MUL_DUAL : CUSYNC_EPILOGUE_GELU_ERF;
  g->tile_n = tile_n; g->max_ctas = d.max_ctas; g->split_k = split_k; g->cta_pair = d.cta_pair; g->tail_split = tail_split;
  g->stage = stage;
}

void fill_gemm2(const cusync_mlp_desc_t& d, int tile_n, int split_k, int tail_split, cusync_stage_t* stage,
                cusync_gemm_desc_t* g) {
  std::memset(g, 0, sizeof(*g));
  g->m = d.batch; g->n = d.hidden; g->k = d.ffn;
  g->a = d.h; g->lda = d.ffn;
  g->b = d.w2; g->ldb = d.hidden;
  g->d = d.y; g->ldd = d.hidden;
  g->b_layout = CUSYNC_B_ROW_MAJOR_KN;
  g->epilogue = CUSYNC_EPILOGUE_NONE;
  g->tile_n = tile_n; g->max_ctas = d.max_ctas; g->split_k = split_k; g->cta_pair = d.cta_pair; g->tail_split = tail_split;
  g->stage = stage;
}

void destroy_all(cusync_mlp* m) {
  if (m->sync1) cusync_gemm_plan_destroy(m->sync1);
  if (m->sync2) cusync_gemm_plan_destroy(m->sync2);
  if (m->plain1) cusync_gemm_plan_destroy(m->plain1);
  if (m->plain2) cusync_gemm_plan_destroy(m->plain2);
  if (m->input) cusync_stage_destroy(m->input);
  if (m->prod) cusync_stage_destroy(m->prod);
  if (m->cons) cusync_stage_destroy(m->cons);
  if (m->plain_stage1) cusync_stage_destroy(m->plain_stage1);
  if (m->plain_stage2) cusync_stage_destroy(m->plain_stage2);
  m->order.destroy();
  if (m->joined) cudaEventDestroy(m->joined);
  if (m->reduced) cudaEventDestroy(m->reduced);
  delete m;
}

}  // namespace

extern "C" {

int cusync_mlp_create(cusync_mlp_t** out, const cusync_mlp_desc_t* desc) {
  if (!out || !desc) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_mlp_desc_t& d0 = *desc;
  if (d0.model != CUSYNC_MLP_GPT3 && d0.model != CUSYNC_MLP_LLAMA) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d0.batch <= 0 || d0.hidden <= 0 || d0.ffn <= 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (!d0.x || !d0.w1 || !d0.w2 || !d0.h || !d0.y || (d0.model == CUSYNC_MLP_LLAMA && !d0.v))
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d0.policy != 0 && d0.policy != CUSYNC_POLICY_ROWSYNC && d0.policy != CUSYNC_POLICY_TILESYNC)
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d0.single_grid < 0 || d0.single_grid > 2 || d0.group_rows1 < 0 || d0.group_rows2 < 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  cusync_mlp_choice_t choice;
  if (cusync_mlp_choose_config(d0.model, d0.batch, d0.hidden, d0.ffn, &choice) != CUSYNC_SUCCESS)
    return CUSYNC_ERROR_INVALID_ARGUMENT;

  cusync_mlp* m = new (std::nothrow) cusync_mlp();
  if (!m) return CUSYNC_ERROR_CUDA;
  std::memset(m, 0, sizeof(*m));
  m->desc = *desc;
  // whatever the caller left open (0) comes from the table
  cusync_mlp_desc_t& dd = m->desc;
  if (dd.policy == 0) dd.policy = choice.policy;
  if (dd.group_rows1 == 0) dd.group_rows1 = choice.group_rows1;
  // post_rows: whoever consumes Y (an all-reduce beside the GEMM, a copy) wants its rows to complete one after
  // the other, not a whole group at once at the end: pair-row groups unless the caller says otherwise
  if (dd.group_rows2 == 0) dd.group_rows2 = dd.post_rows ? 2 : choice.group_rows2;
  const int single_grid_wanted = dd.single_grid ? dd.single_grid : choice.single_grid;
  // The table's K slices for the first GEMM's last partial round go with the table's launch form: only where the
  // caller left both open, the form is one grid, and the tail's units fit one round of the SM pairs in use.
  if (d0.single_grid == 0 && d0.tail_split_sync1 == 0 && choice.single_grid == 2 && choice.tail_split1 > 1 &&
      choice.tile_n1 == 256 && dd.tile_n1 == 0 && dd.cta_pair != 1) {
    int sms = cusync_b200_sm_count();
    if (sms <= 0) sms = 148;
    const int ctas = dd.max_ctas > 0 && dd.max_ctas < sms ? dd.max_ctas : sms;
    const int pairs = ctas / 2;
    const int units = ((dd.batch + 255) / 256) * ((dd.ffn + 255) / 256);
    const int tail = pairs > 0 ? units % pairs : 0;
    if (units > pairs && tail > 0 && tail * choice.tail_split1 <= pairs) dd.tail_split_sync1 = choice.tail_split1;
  }
  const cusync_mlp_desc_t& d = m->desc;
  const int epi1 = d.model == CUSYNC_MLP_LLAMA ? CUSYNC_EPILOGUE_SILU_MUL_DUAL : CUSYNC_EPILOGUE_GELU_ERF;
  m->tile_n1 = d.tile_n1 ? d.tile_n1 : cusync_gemm_default_tile_n(d.batch, d.ffn, d.hidden, epi1);
  m->tile_n2 = d.tile_n2 ? d.tile_n2 : cusync_gemm_default_tile_n(d.batch, d.hidden, d.ffn, CUSYNC_EPILOGUE_NONE);

  m->split_k1 = d.split_k1 ? d.split_k1 : cusync_gemm_default_split_k(d.batch, d.ffn, d.hidden, epi1, m->tile_n1, d.cta_pair);
  m->split_k2 = d.split_k2 ? d.split_k2
                           : cusync_gemm_default_split_k(d.batch, d.hidden, d.ffn, CUSYNC_EPILOGUE_NONE, m->tile_n2, d.cta_pair);

  // Tile grids (N tiles, M tiles, K slices) and the sync policy between the GEMMs.
  const uint32_t tiles_m = static_cast<uint32_t>((d.batch + 127) / 128);
  cusync_dim3_t grid1 = {static_cast<uint32_t>((d.ffn + m->tile_n1 - 1) / m->tile_n1), tiles_m,
                         static_cast<uint32_t>(m->split_k1)};
  cusync_dim3_t grid2 = {static_cast<uint32_t>((d.hidden + m->tile_n2 - 1) / m->tile_n2), tiles_m,
                         static_cast<uint32_t>(m->split_k2)};
  cusync_policy_t sync;
  std::memset(&sync, 0, sizeof(sync));
  sync.kind = d.policy;
  sync.order = CUSYNC_ORDER_TRANSPOSE_XY;
  sync.tile_m = 128;
  sync.tile_n = static_cast<uint32_t>(m->tile_n1);
  if (d.policy == CUSYNC_POLICY_ROWSYNC) { sync.wait_value = grid1.x; sync.post_value = 1; }   // mlp.cu:1032-1034
  else                                   { sync.wait_value = 1; sync.post_value = 1; }
  cusync_policy_t none;
  std::memset(&none, 0, sizeof(none));
  none.tile_m = none.tile_n = 1;
  // NoAtomicAdd only where each semaphore has one poster (mlp.cu:9-14).
  int opts = d.opts;
  // Short chains (up to four row tiles) take the wait before the second GEMM as a stream memory operation
  // rather than a kernel launch: measured two points of gain at B <= 256 and nothing either way above.
  if (tiles_m <= 4) opts |= CUSYNC_OPT_STREAM_WAIT;
  if (d.policy == CUSYNC_POLICY_ROWSYNC) opts &= ~CUSYNC_OPT_NO_ATOMIC_ADD;
  cusync_dim3_t ts = {1, 1, 1};
  const int order1 = d.group_rows1 > 1 ? CUSYNC_ORDER_GROUPED(d.group_rows1) : CUSYNC_ORDER_TRANSPOSE_XY;
  // x_rows: the first GEMM is a consumer as well, of a stage with one tile per 128 rows of X that the caller posts
  cusync_policy_t rows_in = none;
  int rc = CUSYNC_SUCCESS;
  if (d.x_rows) {
    rows_in.kind = CUSYNC_POLICY_ROWSYNC; rows_in.order = CUSYNC_ORDER_TRANSPOSE_XY;
    rows_in.tile_m = 128; rows_in.tile_n = 1; rows_in.wait_value = 1; rows_in.post_value = 1;
    const cusync_dim3_t grid0 = {1, tiles_m, 1};
    rc = cusync_stage_create(&m->input, grid0, ts, CUSYNC_ORDER_TRANSPOSE_XY, &none, &rows_in, CUSYNC_OPT_NONE);
    if (rc == CUSYNC_SUCCESS) m->x_posted.assign(tiles_m, cusync_stage_iter(m->input) - 1u);
  }
  if (rc == CUSYNC_SUCCESS)
    rc = cusync_stage_create(&m->prod, grid1, ts, order1, &rows_in, &sync, opts & ~(d.x_rows ? CUSYNC_OPT_NO_ATOMIC_ADD : 0));
  if (rc == CUSYNC_SUCCESS && d.x_rows) rc = cusync_stage_link(m->input, m->prod);
  // Consumer tile order: left to choose, batches of at least 8 row tiles take their tiles in groups of 4 rows
  // (row fastest inside a group), which re-reads W2 once per group instead of once per row; measured 4 % faster
  // at B = 1024 and 2048, neutral below.
  const int group2 = d.group_rows2 > 1 ? d.group_rows2 : 0;
  const int order2 = group2 > 1 ? CUSYNC_ORDER_GROUPED(group2) : CUSYNC_ORDER_TRANSPOSE_XY;
  // post_rows: the consumer publishes Y by 128-row tile as well (RowSync counting its column tiles)
  cusync_policy_t rows_out = none;
  if (d.post_rows) {
    rows_out.kind = CUSYNC_POLICY_ROWSYNC; rows_out.order = CUSYNC_ORDER_TRANSPOSE_XY;
    rows_out.tile_m = 128; rows_out.tile_n = static_cast<uint32_t>(m->tile_n2);
    rows_out.wait_value = grid2.x; rows_out.post_value = 1;
  }
  if (rc == CUSYNC_SUCCESS)
    rc = cusync_stage_create(&m->cons, grid2, ts, order2, &sync, &rows_out, opts & ~CUSYNC_OPT_NO_ATOMIC_ADD);
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_link(m->prod, m->cons);

  cusync_gemm_desc_t g;
  if (rc == CUSYNC_SUCCESS) { fill_gemm1(d, m->tile_n1, m->split_k1, d.tail_split_sync1, m->prod, &g); rc = cusync_gemm_plan_create(&m->sync1, &g); }
  if (rc == CUSYNC_SUCCESS) { fill_gemm2(d, m->tile_n2, m->split_k2, d.tail_split_sync2, m->cons, &g); rc = cusync_gemm_plan_create(&m->sync2, &g); }
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_create(&m->plain_stage1, grid1, ts, order1, &none, &none, CUSYNC_OPT_NONE);
  if (rc == CUSYNC_SUCCESS) { fill_gemm1(d, m->tile_n1, m->split_k1, d.tail_split_plain1, m->plain_stage1, &g); rc = cusync_gemm_plan_create(&m->plain1, &g); }
  if (rc == CUSYNC_SUCCESS) rc = cusync_stage_create(&m->plain_stage2, grid2, ts, order2, &none, &none, CUSYNC_OPT_NONE);
  if (rc == CUSYNC_SUCCESS) { fill_gemm2(d, m->tile_n2, m->split_k2, d.tail_split_plain2, m->plain_stage2, &g); rc = cusync_gemm_plan_create(&m->plain2, &g); }
  if (rc == CUSYNC_SUCCESS && !m->order.create()) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  if (rc == CUSYNC_SUCCESS) {
    {
      const bool can = cusync_gemm_chain_supported(m->sync1, m->sync2) != 0;
      if (d.single_grid == 2 && !can) rc = CUSYNC_ERROR_UNSUPPORTED;      // asked for outright
      m->single_grid = can && single_grid_wanted == 2;
      if (m->single_grid && cusync_gemm_chain_prepare() != CUSYNC_SUCCESS) rc = CUSYNC_ERROR_CUDA;
      if (rc == CUSYNC_SUCCESS && m->single_grid &&
          cudaEventCreateWithFlags(&m->joined, cudaEventDisableTiming) != cudaSuccess) {
        (void)cudaGetLastError();
        m->joined = nullptr;
        rc = CUSYNC_ERROR_CUDA;
      }
    }
  }
  if (rc != CUSYNC_SUCCESS) { destroy_all(m); return rc; }
  *out = m;
  return CUSYNC_SUCCESS;
}

int cusync_mlp_destroy(cusync_mlp_t* m) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  destroy_all(m);
  return CUSYNC_SUCCESS;
}

int cusync_mlp_run_stream_ordered(cusync_mlp_t* m, cusync_stream_t stream) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  int rc = cusync_gemm_run(m->plain1, stream);
  if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run(m->plain2, stream);
  return rc;
}

int cusync_mlp_run_single(cusync_mlp_t* m, int which, cusync_stream_t stream) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (which != 1 && which != 2) return CUSYNC_ERROR_INVALID_ARGUMENT;
  return cusync_gemm_run(which == 1 ? m->plain1 : m->plain2, stream);
}

namespace {
int run_cusync_impl(cusync_mlp_t* m, cusync_allreduce_plan_t* reducer, cusync_stream_t producer_stream,
                    cusync_stream_t consumer_stream, cusync_stream_t reduce_stream);
}

int cusync_mlp_run_cusync(cusync_mlp_t* m, cusync_stream_t producer_stream, cusync_stream_t consumer_stream) {
  return run_cusync_impl(m, nullptr, producer_stream, consumer_stream, nullptr);
}

int cusync_mlp_run_cusync_allreduce(cusync_mlp_t* m, cusync_allreduce_plan_t* reducer, cusync_stream_t producer_stream,
                                    cusync_stream_t consumer_stream, cusync_stream_t reduce_stream) {
  if (!m || !reducer) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!m->desc.post_rows) return CUSYNC_ERROR_NOT_PRODUCER;      // the second GEMM has to publish its rows
  return run_cusync_impl(m, reducer, producer_stream, consumer_stream, reduce_stream);
}

namespace {
int run_cusync_impl(cusync_mlp_t* m, cusync_allreduce_plan_t* reducer, cusync_stream_t producer_stream,
                    cusync_stream_t consumer_stream, cusync_stream_t reduce_stream) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  // The next run's first GEMM overwrites H, which this run's second GEMM reads: runs are ordered one after the other.
  if (!m->order.begin(producer_stream)) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  int rc;
  if (reducer) {
    // The reducer goes out first, so that it is resident on its SMs before the persistent GEMM blocks take the
    // rest; it waits, tile by tile, for this run's RowSync posts of the second GEMM.
    // ... but not before the point the producer stream has reached: whatever the caller put there (the previous
    // layer, a copy) must not find some of the SMs taken by a kernel that only spins
    if (!m->reduced && cudaEventCreateWithFlags(&m->reduced, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      return CUSYNC_ERROR_CUDA;
    }
    if (cudaEventRecord(m->reduced, reinterpret_cast<cudaStream_t>(producer_stream)) != cudaSuccess ||
        cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(reduce_stream), m->reduced, 0) != cudaSuccess) {
      (void)cudaGetLastError();
      return CUSYNC_ERROR_CUDA;
    }
    cusync_stage_view_t v;
    cusync_stage_get_view(m->cons, &v);
    rc = cusync_allreduce_run(reducer, v.sems_post, v.iter * v.grid.x, reduce_stream);
    if (rc != CUSYNC_SUCCESS) return rc;
  }
  if (m->single_grid) {
    // One persistent grid for both GEMMs on the producer stream; the consumer stream, where callers expect the
    // layer's result, waits for it through an event.
    rc = cusync_gemm_run_chain(m->sync1, m->sync2, producer_stream);
    if (rc == CUSYNC_SUCCESS &&
        (cudaEventRecord(m->joined, reinterpret_cast<cudaStream_t>(producer_stream)) != cudaSuccess ||
         cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(consumer_stream), m->joined, 0) != cudaSuccess)) {
      (void)cudaGetLastError();
      rc = CUSYNC_ERROR_CUDA;
    }
  } else {
    rc = cusync_gemm_run(m->sync1, producer_stream);
    if (rc == CUSYNC_SUCCESS) rc = cusync_stage_invoke_wait_kernel(m->prod, consumer_stream);
    if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run(m->sync2, consumer_stream);
  }
  if (rc != CUSYNC_SUCCESS) return rc;      // nothing counted: the stages stay at this run's iteration
  if (reducer) {                            // the layer's result is complete once the reducer has finished
    if (cudaEventRecord(m->reduced, reinterpret_cast<cudaStream_t>(reduce_stream)) != cudaSuccess ||
        cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(consumer_stream), m->reduced, 0) != cudaSuccess) {
      (void)cudaGetLastError();
      rc = CUSYNC_ERROR_CUDA;
    }
  }
  if (!m->order.end(consumer_stream)) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  if (m->input) cusync_stage_increment_iter(m->input);
  cusync_stage_increment_iter(m->prod);
  cusync_stage_increment_iter(m->cons);
  return rc;
}
}  // namespace

int cusync_mlp_run_dependent(cusync_mlp_t* m, cusync_stream_t stream) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  // One stream: the second GEMM is a programmatic dependent of the first, resident as soon as every block of the
  // first is, and ordered against its writes by the semaphores.  No second stream, wait kernel or event.
  if (!m->order.begin(stream)) { (void)cudaGetLastError(); return CUSYNC_ERROR_CUDA; }
  int rc = cusync_gemm_run(m->sync1, stream);
  if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_run_dependent(m->sync2, stream);
  if (rc != CUSYNC_SUCCESS) return rc;
  if (!m->order.end(stream)) { (void)cudaGetLastError(); rc = CUSYNC_ERROR_CUDA; }
  if (m->input) cusync_stage_increment_iter(m->input);
  cusync_stage_increment_iter(m->prod);
  cusync_stage_increment_iter(m->cons);
  return rc;
}

int cusync_mlp_update_io(cusync_mlp_t* m, const void* x, void* y) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  int rc = CUSYNC_SUCCESS;
  if (x) {
    m->desc.x = x;
    rc = cusync_gemm_plan_update(m->sync1, x, nullptr, nullptr, nullptr);
    if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_plan_update(m->plain1, x, nullptr, nullptr, nullptr);
  }
  if (y && rc == CUSYNC_SUCCESS) {
    m->desc.y = y;
    rc = cusync_gemm_plan_update(m->sync2, nullptr, nullptr, nullptr, y);
    if (rc == CUSYNC_SUCCESS) rc = cusync_gemm_plan_update(m->plain2, nullptr, nullptr, nullptr, y);
  }
  return rc;
}

cusync_stage_t* cusync_mlp_stage(cusync_mlp_t* m, int which) {
  if (!m) return nullptr;
  return which == 0 ? m->prod : m->cons;
}

int cusync_mlp_set_trace(cusync_mlp_t* m, void* t1, uint32_t c1, void* t2, uint32_t c2) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  cusync_gemm_plan_set_trace(m->sync1, t1, c1);
  return cusync_gemm_plan_set_trace(m->sync2, t2, c2);
}

int cusync_mlp_config(const cusync_mlp_t* m, int32_t* out6) {
  if (!m || !out6) return CUSYNC_ERROR_NOT_INITIALIZED;
  out6[0] = m->tile_n1; out6[1] = m->tile_n2;
  out6[2] = static_cast<int32_t>(cusync_gemm_plan_num_ctas(m->sync1));
  out6[3] = static_cast<int32_t>(cusync_gemm_plan_num_ctas(m->sync2));
  out6[4] = m->split_k1; out6[5] = m->split_k2;
  return CUSYNC_SUCCESS;
}

int cusync_mlp_post_x_rows(cusync_mlp_t* m, uint32_t first_tile, uint32_t num_tiles, cusync_stream_t stream) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!m->input) return CUSYNC_ERROR_NOT_PRODUCER;
  cusync_stage_view_t v;
  cusync_stage_get_view(m->input, &v);
  if (num_tiles == 0 || first_tile + num_tiles > v.grid.y) return CUSYNC_ERROR_INVALID_ARGUMENT;
  // Run r waits for its row semaphores to reach r, and every tile is posted once per run: the j-th post of a
  // tile is the one for run j, whether it is enqueued before or after that run's launch.
  int rc = CUSYNC_SUCCESS;
  uint32_t t = first_tile;
  while (t < first_tile + num_tiles && rc == CUSYNC_SUCCESS) {
    uint32_t n = 1;
    const uint32_t value = m->x_posted[t] + 1u;
    while (t + n < first_tile + num_tiles && m->x_posted[t + n] + 1u == value) n++;
    rc = cusync_stream_write_values(v.sems_post + t, n, value, stream);
    if (rc == CUSYNC_SUCCESS) for (uint32_t i = 0; i < n; i++) m->x_posted[t + i] = value;
    t += n;
  }
  return rc;
}

int cusync_mlp_wait_rows(cusync_mlp_t* m, uint32_t first_tile, uint32_t num_tiles, cusync_stream_t stream) {
  if (!m) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (!m->desc.post_rows) return CUSYNC_ERROR_NOT_PRODUCER;
  cusync_stage_view_t v;
  cusync_stage_get_view(m->cons, &v);
  if (num_tiles == 0 || first_tile + num_tiles > v.grid.y) return CUSYNC_ERROR_INVALID_ARGUMENT;
  // run_cusync has already incremented the iteration: the run to wait for is the previous one.  With split-K
  // only the finishing slice of a tile posts, so a row is complete after grid.x posts per run.
  const uint32_t runs = v.iter - 1u;
  int rc = cusync_stream_wait_values(v.sems_post + first_tile, num_tiles, runs * v.grid.x, stream);
  if (rc == CUSYNC_ERROR_UNSUPPORTED)   // no stream memory operations: a wait kernel, which needs a free SM
    rc = cusync_wait_kernel_range(v.sems_post + first_tile, num_tiles, runs * v.grid.x, stream, v.status, v.timeout_ns);
  return rc;
}

int cusync_mlp_choose_config(int32_t model, int32_t batch, int32_t hidden, int32_t ffn, cusync_mlp_choice_t* out) {
  if (!out || batch <= 0 || hidden <= 0 || ffn <= 0) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const ConfigRow* row = config_row(model, batch);
  if (!row) return CUSYNC_ERROR_INVALID_ARGUMENT;
  const int epi1 = model == CUSYNC_MLP_LLAMA ? CUSYNC_EPILOGUE_SILU_MUL_DUAL : CUSYNC_EPILOGUE_GELU_ERF;
  out->policy = row->policy;
  out->single_grid = row->single_grid;
  out->group_rows1 = row->group_rows1;
  out->group_rows2 = row->group_rows2;
  out->tail_split1 = row->tail_split1;
  out->tile_n1 = cusync_gemm_default_tile_n(batch, ffn, hidden, epi1);
  out->tile_n2 = cusync_gemm_default_tile_n(batch, hidden, ffn, CUSYNC_EPILOGUE_NONE);
  out->split_k1 = cusync_gemm_default_split_k(batch, ffn, hidden, epi1, out->tile_n1, 0);
  out->split_k2 = cusync_gemm_default_split_k(batch, hidden, ffn, CUSYNC_EPILOGUE_NONE, out->tile_n2, 0);
  out->stream_wait = (batch + 127) / 128 <= 4 ? 1 : 0;
  return CUSYNC_SUCCESS;
}

int cusync_mlp_uses_single_grid(const cusync_mlp_t* m) { return m && m->single_grid ? 1 : 0; }

int cusync_mlp_tail_splits(const cusync_mlp_t* m, int32_t* out4) {
  if (!m || !out4) return CUSYNC_ERROR_NOT_INITIALIZED;
  out4[0] = cusync_gemm_plan_tail_split(m->sync1); out4[1] = cusync_gemm_plan_tail_split(m->sync2);
  out4[2] = cusync_gemm_plan_tail_split(m->plain1); out4[3] = cusync_gemm_plan_tail_split(m->plain2);
  return CUSYNC_SUCCESS;
}

}  // extern "C"
