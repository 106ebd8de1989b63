/*
 * CPU oracle for the CuSync hot path -- see cusync_oracle.h.
 * TEST INFRASTRUCTURE ONLY; never linked into the product library.
 * Parity pinning is described in the header: integer side pinned to the
 * reference's own policy code and test known-answers; arithmetic side pinned
 * to CUTLASS's host reference kernels and activation functors (the decode
 * attention's softmax alone stays unpinned: the reference has none).
 */
#include "cusync_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ======================================================================== */
/* Integer side                                                             */
/* ======================================================================== */

/* tile-orders.h:52-54 and :68-70 -- both orders linearise the launch grid
 * x-fastest; they differ only in tileToBlock. */
uint32_t orc_block_index(int order, orc_dim3 grid, orc_dim3 block) {
  (void)order;
  return block.x + block.y * grid.x + block.z * grid.x * grid.y;
}

/* tile-orders.h:57-59 (transpose: {x,y,z} -> {y,x,z}) and :73-75 (identity). */
orc_dim3 orc_tile_to_block(int order, orc_dim3 tile) {
  orc_dim3 b = tile;
  if (order == ORC_ORDER_TRANSPOSE_XY) { b.x = tile.y; b.y = tile.x; }
  return b;
}

/* GenericTileOrder::tileIndex, tile-orders.h:38-42. */
uint32_t orc_order_tile_index(int order, orc_dim3 tile, orc_dim3 grid) {
  return orc_block_index(order, grid, orc_tile_to_block(order, tile));
}

uint32_t orc_policy_wait_value(const orc_policy* p, orc_dim3 tile, orc_dim3 grid) {
  (void)tile; (void)grid;
  switch (p->kind) {
    case ORC_ROWSYNC:          /* policies.h:66-68 */
    case ORC_TILESYNC:         /* policies.h:122-124 */
    case ORC_CONV2DTILESYNC:   /* policies.h:181-183 */
      return p->wait_value;
    case ORC_STRIDEDSYNC:      /* mlp.cu:83-85 */
      return p->p1;
    case ORC_CONSECUTIVESYNC:  /* attention.cu:55-57 */
      return (p->p0 / 8) / p->tile_n;
    default:                   /* NoSync, policies.h:24 */
      return 0;
  }
}

uint32_t orc_policy_post_value(const orc_policy* p, orc_dim3 tile, orc_dim3 grid) {
  (void)tile; (void)grid;
  switch (p->kind) {
    case ORC_ROWSYNC:          /* policies.h:91-93 */
    case ORC_TILESYNC:         /* policies.h:130-131 */
    case ORC_CONV2DTILESYNC:   /* policies.h:189-190 */
      return p->post_value;
    case ORC_STRIDEDSYNC:      /* mlp.cu:87-88 */
    case ORC_CONSECUTIVESYNC:  /* attention.cu:59-60 */
      return 1;
    default:
      return 0;
  }
}

uint32_t orc_policy_tile_index(const orc_policy* p, orc_dim3 tile, orc_dim3 grid) {
  orc_dim3 t = {0, 0, 0};
  switch (p->kind) {
    case ORC_ROWSYNC:          /* policies.h:74-76 */
      return tile.x / p->tile_m;
    case ORC_TILESYNC:         /* policies.h:136-138 */
      t.x = tile.x / p->tile_m; t.y = tile.y / p->tile_n;
      return orc_order_tile_index(p->order, t, grid);
    case ORC_CONV2DTILESYNC:   /* policies.h:196-198 */
      t.x = tile.x / p->tile_m; t.y = (tile.y / p->tile_n) / p->p0;
      return orc_order_tile_index(p->order, t, grid);
    case ORC_STRIDEDSYNC: {    /* mlp.cu:90-96 */
      uint32_t ty = tile.y / p->tile_n;
      uint32_t half = p->p0 / p->tile_n;
      if (ty >= half) ty -= half;
      t.x = tile.x / p->tile_m; t.y = ty;
      return orc_order_tile_index(p->order, t, grid);
    }
    case ORC_CONSECUTIVESYNC: {/* attention.cu:62-65 */
      uint32_t group = (p->p0 / 8) / p->tile_n;
      orc_dim3 g = {grid.x / group, grid.y, grid.z};
      t.x = tile.x / p->tile_m; t.y = (tile.y / p->tile_n) / group;
      return orc_order_tile_index(p->order, t, g);
    }
    default:
      return 0;
  }
}

int orc_policy_is_sync(const orc_policy* p, orc_dim3 tile, orc_dim3 grid) {
  (void)grid;
  switch (p->kind) {
    case ORC_ROWSYNC:          /* policies.h:83-85 */
    case ORC_CONSECUTIVESYNC:  /* attention.cu:67-69 */
      return tile.z == 1;
    case ORC_TILESYNC:         /* policies.h:144-146 */
    case ORC_STRIDEDSYNC:      /* mlp.cu:98-100 */
      return tile.y % p->tile_n == 0;
    case ORC_CONV2DTILESYNC:   /* policies.h:205-207 */
      return (tile.y / p->tile_n) % p->p0 == 0;
    default:                   /* policies.h:28 */
      return 0;
  }
}

/* cusync.h:125-157: every slot starts invalid; walking the grid z,y,x, block
 * (x,y,z) is stored at slot blockIndex(grid, block); a slot hit twice is the
 * "invalid linear block index" error. */
int orc_build_tile_order(int order, orc_dim3 grid, orc_dim3* out) {
  uint32_t n = grid.x * grid.y * grid.z;
  int bad = 0;
  for (uint32_t i = 0; i < n; i++) { out[i].x = n; out[i].y = 0; out[i].z = 0; }
  for (uint32_t z = 0; z < grid.z; z++)
    for (uint32_t y = 0; y < grid.y; y++)
      for (uint32_t x = 0; x < grid.x; x++) {
        orc_dim3 b = {x, y, z};
        uint32_t id = orc_block_index(order, grid, b);
        if (id >= n) { bad = 1; continue; }
        if (out[id].x == n) out[id] = b; else bad = 1;
      }
  return bad;
}

int orc_producer_semaphores(const orc_policy* op, orc_dim3 grid, uint32_t tile_m,
                            uint32_t tile_n, int opts, uint32_t iters,
                            uint32_t* sems, uint32_t num_sems) {
  int oob = 0;
  for (uint32_t it = 1; it <= iters; it++)
    for (uint32_t y = 0; y < grid.y; y++)
      for (uint32_t x = 0; x < grid.x; x++) {
        /* only the last split-K slice posts: cusyncgemm.h:374-398 */
        orc_dim3 tile = {y * tile_m, x * tile_n, grid.z - 1};
        uint32_t idx = orc_policy_tile_index(op, tile, grid);
        uint32_t pv = orc_policy_post_value(op, tile, grid);
        if (idx >= num_sems) { oob++; continue; }
        if (opts & ORC_OPT_NO_ATOMIC_ADD) sems[idx] = pv * it;  /* device_defs.h:64-66 */
        else                              sems[idx] += pv;      /* device_defs.h:61-63 */
      }
  return oob;
}

uint32_t orc_consumer_tile_waits(const orc_policy* ip, orc_dim3 prod_grid,
                                 uint32_t row_off, uint32_t k_extent,
                                 uint32_t block_k, uint32_t iter,
                                 uint32_t* idx_out, uint32_t* expect_out,
                                 uint32_t cap) {
  uint32_t n = 0;
  for (uint32_t k = 0; k < k_extent; k += block_k) {
    orc_dim3 tile = {row_off, k, k == 0 ? 1u : 0u};
    if (!orc_policy_is_sync(ip, tile, prod_grid)) continue;
    if (n < cap) {
      idx_out[n] = orc_policy_tile_index(ip, tile, prod_grid);
      /* cusync_device_defs.h:41: spin while sem < iter * waitValue */
      expect_out[n] = iter * orc_policy_wait_value(ip, tile, prod_grid);
    }
    n++;
  }
  return n;
}

/* ======================================================================== */
/* Arithmetic side                                                          */
/* ======================================================================== */

float orc_half_to_float(uint16_t h) {
  _Float16 v; memcpy(&v, &h, 2); return (float)v;
}
uint16_t orc_float_to_half(float f) {
  _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h;
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static inline float epi_apply(float x, int epilogue) {
  switch (epilogue) {
    case ORC_EPI_GELU_ERF: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case ORC_EPI_RELU:     return x > 0.0f ? x : 0.0f;
    default:               return x;
  }
}

#define ORC_MB 16   /* rows kept in flight per task */
#define ORC_NB 256  /* columns per task */

/* Accumulate acc[mb][nb] += A[i0.., :] * B[:, j0..] with each output element
 * summed over k = 0..K-1 in order, as ref_cpumatmul does (common.h:96-98).
 * Row/column blocking only changes which elements are computed together, not
 * the order of additions inside one element. */
static void gemm_block_f16(int mb, int nb, int K, const _Float16* A, int lda,
                           const _Float16* B, int ldb, float* acc) {
  float brow[ORC_NB] __attribute__((aligned(32)));
  for (int i = 0; i < mb; i++)
    for (int j = 0; j < nb; j++) acc[i * ORC_NB + j] = 0.0f;
  for (int k = 0; k < K; k++) {
    const _Float16* bsrc = B + (size_t)k * ldb;
    int j = 0;
    for (; j + 8 <= nb; j += 8)   /* exact fp16 -> fp32 widening, 8 at a time */
      _mm256_store_ps(brow + j, _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(bsrc + j))));
    for (; j < nb; j++) brow[j] = (float)bsrc[j];
    for (int i = 0; i < mb; i++) {
      float a = (float)A[(size_t)i * lda + k];
      float* arow = acc + i * ORC_NB;
      for (int jj = 0; jj < nb; jj++) arow[jj] += a * brow[jj];
    }
  }
}

void orc_gemm_f16(int M, int N, int K, const uint16_t* A_, int lda,
                  const uint16_t* B_, int ldb, uint16_t* C_, int ldc, int epilogue) {
  const _Float16* A = (const _Float16*)A_;
  const _Float16* B = (const _Float16*)B_;
  _Float16* C = (_Float16*)C_;
  int mt = (M + ORC_MB - 1) / ORC_MB, nt = (N + ORC_NB - 1) / ORC_NB;
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * ORC_MB * ORC_NB);
#pragma omp for collapse(2) schedule(dynamic)
    for (int bi = 0; bi < mt; bi++)
      for (int bj = 0; bj < nt; bj++) {
        int i0 = bi * ORC_MB, j0 = bj * ORC_NB;
        int mb = M - i0 < ORC_MB ? M - i0 : ORC_MB;
        int nb = N - j0 < ORC_NB ? N - j0 : ORC_NB;
        gemm_block_f16(mb, nb, K, A + (size_t)i0 * lda, lda, B + j0, ldb, acc);
        for (int i = 0; i < mb; i++)
          for (int j = 0; j < nb; j++)
            C[(size_t)(i0 + i) * ldc + j0 + j] =
                (_Float16)epi_apply(acc[i * ORC_NB + j], epilogue);
      }
    free(acc);
  }
}

void orc_gemm_dual_silu_mul_f16(int M, int N, int K, const uint16_t* A_, int lda,
                                const uint16_t* B1_, const uint16_t* B2_, int ldb,
                                uint16_t* G_, int ldg) {
  const _Float16* A = (const _Float16*)A_;
  const _Float16* B1 = (const _Float16*)B1_;
  const _Float16* B2 = (const _Float16*)B2_;
  _Float16* G = (_Float16*)G_;
  int mt = (M + ORC_MB - 1) / ORC_MB, nt = (N + ORC_NB - 1) / ORC_NB;
#pragma omp parallel
  {
    float* acc1 = (float*)malloc(sizeof(float) * ORC_MB * ORC_NB);
    float* acc2 = (float*)malloc(sizeof(float) * ORC_MB * ORC_NB);
#pragma omp for collapse(2) schedule(dynamic)
    for (int bi = 0; bi < mt; bi++)
      for (int bj = 0; bj < nt; bj++) {
        int i0 = bi * ORC_MB, j0 = bj * ORC_NB;
        int mb = M - i0 < ORC_MB ? M - i0 : ORC_MB;
        int nb = N - j0 < ORC_NB ? N - j0 : ORC_NB;
        gemm_block_f16(mb, nb, K, A + (size_t)i0 * lda, lda, B1 + j0, ldb, acc1);
        gemm_block_f16(mb, nb, K, A + (size_t)i0 * lda, lda, B2 + j0, ldb, acc2);
        for (int i = 0; i < mb; i++)
          for (int j = 0; j < nb; j++) {
            float a = acc1[i * ORC_NB + j], b = acc2[i * ORC_NB + j];
            float silu = a / (1.0f + expf(-a));
            G[(size_t)(i0 + i) * ldg + j0 + j] = (_Float16)(silu * b);
          }
      }
    free(acc1); free(acc2);
  }
}

void orc_gemm_f32(int M, int N, int K, const float* A, const float* B, float* C) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; i++) {
    float* c = C + (size_t)i * N;
    for (int j = 0; j < N; j++) c[j] = 0.0f;
    for (int k = 0; k < K; k++) {
      float a = A[(size_t)i * K + k];
      const float* b = B + (size_t)k * N;
      for (int j = 0; j < N; j++) c[j] += a * b[j];
    }
  }
}

void orc_conv2d_3x3_nhwc_f16(int N, int H, int W, int C, int K,
                             const uint16_t* x_, const uint16_t* w_, uint16_t* y_,
                             int relu) {
  const _Float16* x = (const _Float16*)x_;
  const _Float16* w = (const _Float16*)w_;
  _Float16* y = (_Float16*)y_;
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; n++)
    for (int p = 0; p < H; p++)
      for (int q = 0; q < W; q++)
        for (int k = 0; k < K; k++) {
          float acc = 0.0f;
          for (int r = 0; r < 3; r++)
            for (int s = 0; s < 3; s++) {
              int h = p + r - 1, ww = q + s - 1;
              if (h < 0 || h >= H || ww < 0 || ww >= W) continue;
              const _Float16* xp = x + (((size_t)n * H + h) * W + ww) * C;
              const _Float16* wp = w + (((size_t)k * 3 + r) * 3 + s) * C;
              for (int c = 0; c < C; c++) acc += (float)xp[c] * (float)wp[c];
            }
          if (relu && acc < 0.0f) acc = 0.0f;
          y[(((size_t)n * H + p) * W + q) * K + k] = (_Float16)acc;
        }
}

void orc_attention_decode_f16(int B, int S, int heads, int d, const uint16_t* q_,
                              int ldq, const uint16_t* k_, const uint16_t* v_,
                              uint16_t* o_, int ldo) {
  const _Float16* q = (const _Float16*)q_;
  const _Float16* kc = (const _Float16*)k_;
  const _Float16* vc = (const _Float16*)v_;
  _Float16* o = (_Float16*)o_;
  float scale = 1.0f / sqrtf((float)d);
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; b++)
    for (int h = 0; h < heads; h++) {
      float* p = (float*)malloc(sizeof(float) * (size_t)S);
      float* acc = (float*)malloc(sizeof(float) * (size_t)d);
      const _Float16* qv = q + (size_t)b * ldq + (size_t)h * d;
      float mx = -INFINITY;
      for (int s = 0; s < S; s++) {
        const _Float16* kv = kc + (((size_t)b * S + s) * heads + h) * d;
        float dot = 0.0f;
        for (int e = 0; e < d; e++) dot += (float)qv[e] * (float)kv[e];
        p[s] = dot * scale;
        if (p[s] > mx) mx = p[s];
      }
      float sum = 0.0f;
      for (int s = 0; s < S; s++) { p[s] = expf(p[s] - mx); sum += p[s]; }
      for (int e = 0; e < d; e++) acc[e] = 0.0f;
      for (int s = 0; s < S; s++) {
        const _Float16* vv = vc + (((size_t)b * S + s) * heads + h) * d;
        for (int e = 0; e < d; e++) acc[e] += p[s] * (float)vv[e];
      }
      for (int e = 0; e < d; e++)
        o[(size_t)b * ldo + (size_t)h * d + e] = (_Float16)(acc[e] / sum);
      free(p); free(acc);
    }
}

double orc_max_rel_err_f16(size_t n, const uint16_t* got, const uint16_t* ref,
                           double floor_frac) {
  double mx = 0.0;
  for (size_t i = 0; i < n; i++) {
    double r = fabs((double)orc_half_to_float(ref[i]));
    if (r > mx) mx = r;
  }
  double floor = mx * floor_frac;
  if (floor <= 0.0) floor = 1e-30;
  double worst = 0.0;
  for (size_t i = 0; i < n; i++) {
    double g = orc_half_to_float(got[i]), r = orc_half_to_float(ref[i]);
    if (isnan(g) || isnan(r)) return INFINITY;
    double den = fabs(r) > floor ? fabs(r) : floor;
    double e = fabs(g - r) / den;
    if (e > worst) worst = e;
  }
  return worst;
}
