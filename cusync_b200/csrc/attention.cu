// Decode attention as a CuSync middle stage: one query token per batch row attends over the cached
// keys/values plus its own new key/value, per head, with an fp32 softmax.
//
// In the reference's attention chain (src/ml-bench/transformer/attention.cu:105-118, 706-833) the stages
// between the QKV projection and the output projection are two plain GEMMs without softmax; a stage there
// both waits on its producer and posts to its consumer (CuStage holds tileStatusRead_ and tileStatusWrite_,
// cusync.h:116-117).  This kernel takes that place in the chain:
//   wait : the Q, K and V thirds of row panel b / 128 of the QKV projection's output
//          (ConsecutiveSync, attention.cu:51-70: one semaphore per third, reached when its column tiles posted);
//   work : scores = q . k / sqrt(d) over the S cached keys and the new one, softmax in fp32, o = p . v;
//          the key range can be split over several blocks (partials combined by the last to finish);
//   post : RowSync on the row panel of the attention output, once every (row, head) of the panel is written.
// The work is HBM-bound (it streams the K/V cache once), so it is plain coalesced loads, no tensor cores.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <new>

#include "common.cuh"

namespace {

constexpr int kAttnThreads = 128;      // also the head dimension: thread t owns output element t
constexpr int kHeadDim = 128;

struct AttnParams {
  int32_t batch, seq, heads, splits;
  const __half* qkv; long long ld_qkv;       // [batch, 3 * heads * 128]: Q | K | V
  const __half* k_cache; const __half* v_cache;   // [batch, seq, heads, 128]
  __half* out; long long ld_out;             // [batch, heads * 128]
  float* partial;                            // [batch, heads, splits, 130]: m, l, acc[128]
  uint32_t* split_arrivals;                  // [batch * heads]
  uint32_t* panel_arrivals;                  // [ceil(batch / 128)]
  int32_t is_producer, is_consumer;
  cusync_stage_view_t stage;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(kAttnThreads)
cusync_attn_decode_kernel(const AttnParams p) {
  extern __shared__ float smem[];
  float* q_s = smem;                    // [128] query, pre-scaled
  float* red = smem + kHeadDim;         // [8] block reductions
  float* scores = smem + kHeadDim + 8;  // [keys of this block]
  __shared__ int s_flag;

  const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const cusync_stage_view_t& st = p.stage;

  cusync::allowDependentLaunch();       // this block is resident: a dependent consumer may be launched
  if (tid == 0 && p.is_producer) {
    // "started" words for the wait kernel of the next stage
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) cusync::storeRelease(st.started, st.iter);
    cusync::addRelease(st.started + 1, 1u);
  }

  // ---- wait for this row's Q, K and V thirds -------------------------------------------------
  if (p.is_consumer) {
    if (tid == 0) {
      int ok = 1;
      const uint32_t target = st.iter * cusync::eval::waitValue(st.in_policy);
      for (int third = 0; third < 3 && ok; third++) {
        // first column of this head inside the third, rounded down to the producer's tile
        uint32_t col = static_cast<uint32_t>(third * p.heads * kHeadDim + h * kHeadDim);
        col -= col % st.in_policy.tile_n;
        if (!cusync::eval::isSync(st.in_policy, col, 1u)) continue;
        const uint32_t idx = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(b), col, st.prod_grid.x,
                                                     st.prod_grid.y);
        uint32_t seen = 0;
        if (!cusync::spinUntilAtLeast(st.sems_wait + idx, target, st.timeout_ns, &seen)) {
          cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(b), col, 1u, idx, seen, target);
          ok = 0;
        }
      }
      s_flag = ok;
    }
    __syncthreads();
    if (!s_flag) {            // bounded wait expired: leave without touching the output ...
      // ... and without posting: release what waits on this stage without a bound of its own
      if (p.is_producer) {
        cusync::releaseWaitersOnAbort(st.sems_post, st.grid.x * st.grid.y * st.grid.z, tid, blockDim.x);
        __syncthreads();
        if (tid == 0) cusync::countBlockFinished(st.started);
      }
      return;
    }
  }

  // ---- query ----------------------------------------------------------------------------------
  const int hd = p.heads * kHeadDim;
  const __half* qrow = p.qkv + static_cast<size_t>(b) * p.ld_qkv + h * kHeadDim;
  q_s[tid] = __half2float(qrow[tid]) * rsqrtf(static_cast<float>(kHeadDim));
  __syncthreads();

  // keys of this block: [k0, k1) out of seq cached keys + the new one (index seq)
  const int total = p.seq + 1;
  const int per = (total + p.splits - 1) / p.splits;
  const int k0 = z * per, k1 = min(total, k0 + per);
  const int nkeys = max(k1 - k0, 0);

  // Thread layout for the two passes over the cache: 16 threads cover one key's 128 elements with a 16-byte
  // load each (thread `sub` holds elements [8 sub, 8 sub + 8)); the block's 8 such groups take every eighth
  // key; `kInFlight` keys per group are loaded before any is used, so 16 KB are in flight per block.
  constexpr int kGroups = kAttnThreads / 16, kInFlight = 8;
  const int grp = tid >> 4, sub = tid & 15;
  float qf[8];
#pragma unroll
  for (int e = 0; e < 8; e++) qf[e] = q_s[8 * sub + e];
  const size_t kv_row = static_cast<size_t>(p.heads) * kHeadDim;                     // elements between keys
  const __half* knew = p.qkv + static_cast<size_t>(b) * p.ld_qkv + hd + h * kHeadDim + 8 * sub;
  const __half* vnew = p.qkv + static_cast<size_t>(b) * p.ld_qkv + 2 * hd + h * kHeadDim + 8 * sub;
  const __half* kbase = p.k_cache + (static_cast<size_t>(b) * p.seq * p.heads + h) * kHeadDim + 8 * sub;
  const __half* vbase = p.v_cache + (static_cast<size_t>(b) * p.seq * p.heads + h) * kHeadDim + 8 * sub;

  // ---- scores -----------------------------------------------------------------------------------
  float mx = -INFINITY;
  // the trip count is the same for every thread of the block (the shuffles below need whole warps)
  for (int base = 0; base < nkeys; base += kGroups * kInFlight) {
    const int i0 = base + grp;
    uint4 raw[kInFlight];
#pragma unroll
    for (int j = 0; j < kInFlight; j++) {
      const int i = i0 + j * kGroups;
      if (i < nkeys) {
        const int s = k0 + i;
        raw[j] = *reinterpret_cast<const uint4*>(s < p.seq ? kbase + static_cast<size_t>(s) * kv_row : knew);
      }
    }
#pragma unroll
    for (int j = 0; j < kInFlight; j++) {
      const int i = i0 + j * kGroups;
      float d = 0.f;
      if (i < nkeys) {
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
        for (int e = 0; e < 4; e++) d += qf[2 * e] * __low2float(h2[e]) + qf[2 * e + 1] * __high2float(h2[e]);
      }
      // sum over the 16 threads of the group (both halves of the warp take part in every shuffle)
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (i < nkeys) {
        if (sub == 0) scores[i] = d;
        mx = fmaxf(mx, d);
      }
    }
  }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();

  // ---- softmax numerators and their sum ------------------------------------------------------------
  float sum = 0.f;
  for (int i = tid; i < nkeys; i += kAttnThreads) {
    const float e = __expf(scores[i] - mx);
    scores[i] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) red[4 + warp] = sum;
  __syncthreads();
  sum = red[4] + red[5] + red[6] + red[7];

  // ---- values: group g accumulates its keys' contribution to elements [8 sub, 8 sub + 8) -----------
  float pv[8];
#pragma unroll
  for (int e = 0; e < 8; e++) pv[e] = 0.f;
  for (int base = 0; base < nkeys; base += kGroups * kInFlight) {
    const int i0 = base + grp;
    uint4 raw[kInFlight];
#pragma unroll
    for (int j = 0; j < kInFlight; j++) {
      const int i = i0 + j * kGroups;
      if (i < nkeys) {
        const int s = k0 + i;
        raw[j] = *reinterpret_cast<const uint4*>(s < p.seq ? vbase + static_cast<size_t>(s) * kv_row : vnew);
      }
    }
#pragma unroll
    for (int j = 0; j < kInFlight; j++) {
      const int i = i0 + j * kGroups;
      if (i < nkeys) {
        const float w = scores[i];
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
        for (int e = 0; e < 4; e++) { pv[2 * e] += w * __low2float(h2[e]); pv[2 * e + 1] += w * __high2float(h2[e]); }
      }
    }
  }
  // sum the 8 groups: pv_s[group][128] in shared memory, then thread t adds up element t
  __syncthreads();                       // everyone is done reading scores[], which pv_s may overlap
  float* pv_s = smem + kHeadDim + 8;     // reuses the score buffer when it is large enough, see host side
#pragma unroll
  for (int e = 0; e < 8; e++) pv_s[grp * kHeadDim + 8 * sub + e] = pv[e];
  __syncthreads();
  float acc = 0.f;
#pragma unroll
  for (int g2 = 0; g2 < kGroups; g2++) acc += pv_s[g2 * kHeadDim + tid];

  __half* orow = p.out + static_cast<size_t>(b) * p.ld_out + h * kHeadDim;
  bool wrote = false;
  if (p.splits == 1) {
    orow[tid] = __float2half_rn(acc / sum);
    wrote = true;
  } else {
    // partial (m, l, acc) of this key range; the block that brings the last one combines them
    float* part = p.partial + ((static_cast<size_t>(b) * p.heads + h) * p.splits + z) * (kHeadDim + 2);
    if (tid == 0) { part[0] = mx; part[1] = sum; }
    part[2 + tid] = acc;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const uint32_t before = atomicAdd(p.split_arrivals + b * p.heads + h, 1u);
      const int last = before == static_cast<uint32_t>(p.splits) - 1u;
      if (last) { p.split_arrivals[b * p.heads + h] = 0u; __threadfence(); }
      s_flag = last;
    }
    __syncthreads();
    if (s_flag) {
      const float* base = p.partial + (static_cast<size_t>(b) * p.heads + h) * p.splits * (kHeadDim + 2);
      float gm = -INFINITY;
      for (int j = 0; j < p.splits; j++) gm = fmaxf(gm, __ldcg(base + j * (kHeadDim + 2)));
      float l = 0.f, o = 0.f;
      for (int j = 0; j < p.splits; j++) {
        const float* pj = base + j * (kHeadDim + 2);
        const float lj = __ldcg(pj + 1);
        if (lj == 0.f) continue;                       // an empty key range
        const float w = __expf(__ldcg(pj) - gm);
        l += lj * w;
        o += __ldcg(pj + 2 + tid) * w;
      }
      orow[tid] = __float2half_rn(o / l);
      wrote = true;
    }
  }

  // ---- post: the row panel is published once all of its (row, head) outputs are written -------------------
  if (p.is_producer) {
    __syncthreads();
    if (tid == 0 && wrote) {
      const int panel = b / 128;
      const int rows = min(128, p.batch - panel * 128);
      __threadfence();
      const uint32_t before = atomicAdd(p.panel_arrivals + panel, 1u);
      if (before == static_cast<uint32_t>(rows * p.heads) - 1u) {
        p.panel_arrivals[panel] = 0u;
        const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(panel * 128), 0u, st.grid.x,
                                                     st.grid.y);
        const uint32_t pv = cusync::eval::postValue(st.out_policy);
        __threadfence();
        if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
        else                                    cusync::addRelease(st.sems_post + idx, pv);
      }
    }
    if (tid == 0) cusync::countBlockFinished(st.started);     // after this block's post, if it had one
  }
}

}  // namespace

struct cusync_attn_plan {
  cusync_attn_desc_t desc;
  AttnParams params;
  int splits;
  cusync_stage_t* own_stage;
  cusync_stage_t* stage;
  uint32_t* counters;      // split_arrivals followed by panel_arrivals
  float* partial;
  size_t smem;
};

extern "C" {

int cusync_attn_default_splits(int32_t batch, int32_t seq, int32_t heads) {
  int sms = cusync_b200_sm_count();
  if (sms <= 0) sms = 148;
  const int blocks = batch * heads;
  if (blocks <= 0) return 1;
  int s = (2 * sms + blocks - 1) / blocks;       // about two blocks per SM keep the HBM queues full
  const int by_len = (seq + 1) / 128;            // at least 128 keys per block
  if (s > by_len) s = by_len;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

int cusync_attn_plan_create(cusync_attn_plan_t** out, const cusync_attn_desc_t* desc) {
  if (!out || !desc) return CUSYNC_ERROR_INVALID_ARGUMENT;
  *out = nullptr;
  const cusync_attn_desc_t& d = *desc;
  if (d.batch <= 0 || d.seq < 0 || d.heads <= 0 || !d.qkv || !d.out || (d.seq > 0 && (!d.k_cache || !d.v_cache)))
    return CUSYNC_ERROR_INVALID_ARGUMENT;
  if (d.head_dim != kHeadDim || d.seq > 16384) return CUSYNC_ERROR_UNSUPPORTED;
  // 16-byte loads of the query's key/value and of the cache rows
  if (d.ld_qkv < 3ll * d.heads * kHeadDim || d.ld_out < 1ll * d.heads * kHeadDim || d.ld_qkv % 8) return CUSYNC_ERROR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(d.qkv) | reinterpret_cast<uintptr_t>(d.k_cache) | reinterpret_cast<uintptr_t>(d.v_cache)) & 15u)
    return CUSYNC_ERROR_UNSUPPORTED;
  if (d.kv_splits < 0 || d.kv_splits > 64) return CUSYNC_ERROR_INVALID_ARGUMENT;

  cusync_attn_plan* pl = new (std::nothrow) cusync_attn_plan();
  if (!pl) return CUSYNC_ERROR_CUDA;
  std::memset(pl, 0, sizeof(*pl));
  pl->desc = d;
  pl->splits = d.kv_splits ? d.kv_splits : cusync_attn_default_splits(d.batch, d.seq, d.heads);
  if (pl->splits > d.seq + 1) pl->splits = d.seq + 1;
  AttnParams& p = pl->params;
  p.batch = d.batch; p.seq = d.seq; p.heads = d.heads; p.splits = pl->splits;
  p.qkv = static_cast<const __half*>(d.qkv); p.ld_qkv = d.ld_qkv;
  p.k_cache = static_cast<const __half*>(d.k_cache); p.v_cache = static_cast<const __half*>(d.v_cache);
  p.out = static_cast<__half*>(d.out); p.ld_out = d.ld_out;

  // The stage grid of the attention step is (heads, batch, key-range splits).
  pl->stage = d.stage;
  int rc = CUSYNC_SUCCESS;
  if (pl->stage == nullptr) {
    cusync_dim3_t grid = {static_cast<uint32_t>(d.heads), static_cast<uint32_t>(d.batch), static_cast<uint32_t>(pl->splits)};
    cusync_dim3_t ts = {1, 1, 1};
    rc = cusync_stage_create(&pl->own_stage, grid, ts, CUSYNC_ORDER_IDENTITY, nullptr, nullptr, CUSYNC_OPT_NONE);
    pl->stage = pl->own_stage;
  }
  cusync_stage_view_t view;
  if (rc == CUSYNC_SUCCESS) {
    cusync_stage_get_view(pl->stage, &view);
    if (view.grid.x != static_cast<uint32_t>(d.heads) || view.grid.y != static_cast<uint32_t>(d.batch) ||
        view.grid.z != static_cast<uint32_t>(pl->splits))
      rc = CUSYNC_ERROR_INVALID_ARGUMENT;
    else if (view.in_policy.kind != CUSYNC_POLICY_NOSYNC && view.sems_wait == nullptr)
      rc = CUSYNC_ERROR_NOT_INITIALIZED;
    else if (view.in_policy.kind == CUSYNC_POLICY_CUSTOM || view.out_policy.kind == CUSYNC_POLICY_CUSTOM)
      rc = CUSYNC_ERROR_UNSUPPORTED;
  }
  if (rc == CUSYNC_SUCCESS) {
    const size_t n_split = static_cast<size_t>(d.batch) * d.heads, n_panel = (d.batch + 127) / 128;
    const size_t part = n_split * pl->splits * (kHeadDim + 2) * sizeof(float);
    if (cudaMalloc(&pl->counters, (n_split + n_panel) * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(pl->counters, 0, (n_split + n_panel) * sizeof(uint32_t)) != cudaSuccess ||
        cudaMalloc(&pl->partial, part) != cudaSuccess) {
      (void)cudaGetLastError();
      rc = CUSYNC_ERROR_CUDA;
    }
    p.split_arrivals = pl->counters;
    p.panel_arrivals = pl->counters + n_split;
    p.partial = pl->partial;
    const int per = (d.seq + 1 + pl->splits - 1) / pl->splits;
    pl->smem = (kHeadDim + 8 + (per > 8 * kHeadDim ? per : 8 * kHeadDim)) * sizeof(float);
    if (rc == CUSYNC_SUCCESS && pl->smem > 48 * 1024 &&
        cudaFuncSetAttribute(cusync_attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(pl->smem)) != cudaSuccess) {
      (void)cudaGetLastError();
      rc = CUSYNC_ERROR_CUDA;
    }
  }
  if (rc != CUSYNC_SUCCESS) {
    if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
    cudaFree(pl->counters); cudaFree(pl->partial);
    delete pl;
    return rc;
  }
  *out = pl;
  return CUSYNC_SUCCESS;
}

int cusync_attn_plan_destroy(cusync_attn_plan_t* pl) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  if (pl->own_stage) cusync_stage_destroy(pl->own_stage);
  cudaFree(pl->counters); cudaFree(pl->partial);
  delete pl;
  return CUSYNC_SUCCESS;
}

int cusync_attn_plan_splits(const cusync_attn_plan_t* pl) { return pl ? pl->splits : 0; }

namespace {
int attn_launch(cusync_attn_plan_t* pl, cusync_stream_t stream, bool dependent);
}

int cusync_attn_run(cusync_attn_plan_t* pl, cusync_stream_t stream) { return attn_launch(pl, stream, false); }

int cusync_attn_run_dependent(cusync_attn_plan_t* pl, cusync_stream_t stream) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  cusync_stage_view_t v;
  cusync_stage_get_view(pl->stage, &v);
  if (v.in_policy.kind == CUSYNC_POLICY_NOSYNC) return CUSYNC_ERROR_NOT_CONSUMER;
  return attn_launch(pl, stream, true);
}

namespace {
int attn_launch(cusync_attn_plan_t* pl, cusync_stream_t stream, bool dependent) {
  if (!pl) return CUSYNC_ERROR_NOT_INITIALIZED;
  AttnParams p = pl->params;
  cusync_stage_get_view(pl->stage, &p.stage);
  p.is_producer = p.stage.out_policy.kind != CUSYNC_POLICY_NOSYNC;
  p.is_consumer = p.stage.in_policy.kind != CUSYNC_POLICY_NOSYNC;
  dim3 grid(pl->desc.heads, pl->desc.batch, pl->splits);
  if (p.is_producer) cusync_stage_note_launch(pl->stage, grid.x * grid.y * grid.z);
  if (dependent) {
    if (launchDependent(cusync_attn_decode_kernel, grid, dim3(kAttnThreads), pl->smem,
                        reinterpret_cast<cudaStream_t>(stream), p) != cudaSuccess) {
      (void)cudaGetLastError();
      return CUSYNC_ERROR_CUDA;
    }
    return CUSYNC_SUCCESS;
  }
  cusync_attn_decode_kernel<<<grid, kAttnThreads, pl->smem, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? CUSYNC_SUCCESS : CUSYNC_ERROR_CUDA;
}
}  // namespace

}  // extern "C"
