// cusync_gemm_pair_kernel: the CTA-pair (tcgen05 cta_group::2) GEMM kernel and its cluster-level PTX wrappers.
#pragma once

#include "sm100_device.cuh"

namespace {

// ---------------------------------------------------------------------------
// CTA-pair variant: tcgen05.mma.cta_group::2
// ---------------------------------------------------------------------------
// Two CTAs of a cluster (the two SMs of a TPC) compute one 256 x 256 output tile.  CTA r owns rows
// [r*128, r*128+128) of it: it loads its own A rows and HALF of the B tile (128 of the 256 columns),
// and holds its 128 x 256 accumulator in its own tensor memory.  The leader (rank 0) issues one
// M=256 MMA per K step that reads A and the B halves from both CTAs' shared memory.  Per CTA and 64 of K
// that is 32 KB from L2 instead of 48 KB; the ring holds three stages of 128 of K (64 KB each).
// No multicast loads: the only cluster-wide traffic is mbarrier signalling (TMA completion on the
// leader's barrier, tcgen05.commit to both CTAs, remote arrives) and the scheduler's tile broadcast.
// Semaphores stay per 128-row tile: each CTA waits for, and posts, its own rows.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on a LOCAL barrier that a peer CTA may have signalled.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = cusync::globalTimerNs();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++polls & 31u) == 0u) {
      if (*ctx.abort) return false;
      if (cusync::globalTimerNs() - t0 > ctx.timeout_ns) {
        *ctx.abort = 1u;
        cusync::recordTimeout(ctx.status, 2u, blockIdx.x, threadIdx.x, parity, smem_u32(bar), 0u, 0u);
        return false;
      }
    }
  }
}
// TMA load whose completion may be signalled on the peer CTA's barrier (`bar_cluster_addr` is a
// shared::cluster address); the data lands in this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair when the MMAs retire.
__device__ __forceinline__ void umma_commit_pair_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair_local(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// K depth of one ring stage of the pair kernel: two 64-element swizzle chunks.  A barrier wait, a commit and
// each MMA issue cost the issuing thread of the order of a hundred cycles whatever the MMA's size, so a stage
// carries eight MMAs (and two TMA boxes) per wait/commit instead of four to stay under the tensor time.
constexpr int kPairBlockK = 128;
constexpr int kPairChunkBytes = kBlockM * 128;     // one 64-deep chunk of 128 rows
struct PairCfg {
  static constexpr int kABytes = kBlockM * kPairBlockK * 2;            // this CTA's 128 A rows
  static constexpr int kBHalfBytes = (kPairBN / 2) * kPairBlockK * 2;  // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBHalfBytes;
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kStages = ((int)kSmemLimit - 1024 - kStagingBytes - kBarrierBytes) / kStageBytes;
  static constexpr int kAccCols = kPairBN;
  static constexpr int kTmemCols = 2 * kAccCols;
  static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarrierBytes;
  static_assert(kStages >= 3 && kStages <= 8, "ring depth out of range");
  static_assert(kSmemBytes <= kSmemLimit, "shared memory over budget");
};

// The kernel body serves one GEMM (kChain = false) or a chain of two dependent GEMMs run by ONE persistent grid
// (kChain = true): the work units of the first GEMM take the tickets [0, units of GEMM 0), those of the second
// the tickets after them, from one shared counter.  A pair that finds no unit of the first GEMM left goes
// straight on to units of the second, whose waits on the first GEMM's semaphores are the usual ones; no second
// launch, no wait kernel, and no pair sits idle while the first GEMM's last round runs.  It cannot deadlock:
// every pair of the grid is resident, tickets are drawn in order, a pair works through its tickets in order,
// and a unit only ever waits for units with lower tickets.
template <bool kChain>
__device__ __forceinline__ void pair_kernel_body(const CUtensorMap* mA0, const CUtensorMap* mB0, const CUtensorMap* mD0,
                                                 const CUtensorMap* mWS0, const CUtensorMap* mA1, const CUtensorMap* mB1,
                                                 const CUtensorMap* mD1, const CUtensorMap* mWS1, const GemmParams& p0,
                                                 const GemmParams& p1, const CUtensorMap* mB2_0, const CUtensorMap* mB2_1) {
  using C = PairCfg;
  constexpr int BN = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(staging + C::kStagingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader: draws tickets, issues the MMAs
  const bool leader = rank == 0;
  // Bounded barrier waits record into the first GEMM's stage.
  WaitCtx ctx{&bars->abort, p0.stage.status, 2 * p0.stage.timeout_ns + 1000000000ull};
  const uint32_t units0 = static_cast<uint32_t>(p0.num_pairs);
  const uint32_t total_units = units0 + (kChain ? static_cast<uint32_t>(p1.num_pairs) : 0u);

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; i++) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 2 * kEpilogueWarps);           // leader's: epilogue warps of both CTAs
    }
    for (int i = 0; i < kSchedSlots; i++) {
      mbar_init(&bars->sched_full[i], 1);
      mbar_init(&bars->sched_empty[i], 2 * (1 + kEpilogueWarps));    // leader's: MMA + peer loader + all epilogue warps
    }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->post, kEpilogueWarps);
    mbar_init(&bars->splitk_counted, 1);
    mbar_init(&bars->splitk_done, kEpilogueWarps);
    bars->abort = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    for (int gi = 0; gi < (kChain ? 2 : 1); gi++) {
      const GemmParams& pg = gi ? p1 : p0;
      if (pg.is_producer) {
        if (blockIdx.x == 0) cusync::storeRelease(pg.stage.started, pg.stage.iter);
        cusync::addRelease(pg.stage.started + 1, 1u);
      }
    }
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(mA0); prefetch_tensormap(mB0); prefetch_tensormap(mD0);
    if (kChain) { prefetch_tensormap(mA1); prefetch_tensormap(mB1); prefetch_tensormap(mD1); }
  }
  if (warp == 2) {
    tmem_alloc_pair(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  cusync::allowDependentLaunch();      // this pair is resident: a dependent consumer may be launched

  // Cluster addresses of the leader's barriers that the peer signals.
  const uint32_t leader_full0 = map_to_cta(smem_u32(&bars->full[0]), 0);
  const uint32_t leader_tmem_empty0 = map_to_cta(smem_u32(&bars->tmem_empty[0]), 0);
  const uint32_t leader_sched_empty0 = map_to_cta(smem_u32(&bars->sched_empty[0]), 0);

  if (warp == 0) {
    // =====================================================================
    // Scheduler (leader) + TMA loader (both CTAs)
    // =====================================================================
    if (lane == 0) {
      uint32_t fills = 0, sched_it = 0;
      bool ok = true;
      const uint32_t total_draws = total_units + gridDim.x / 2;
      uint32_t* const ticket_counter = p0.stage.tile_counter;     // one counter for the whole chain
      const uint32_t peer_sched_tile0 = map_to_cta(smem_u32(&bars->sched_tile[0][0]), 1);
      const uint32_t peer_sched_time0 = map_to_cta(smem_u32(&bars->sched_time[0]), 1);
      const uint32_t peer_sched_full0 = map_to_cta(smem_u32(&bars->sched_full[0]), 1);
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        int32_t tn, tpm, valid, tz_slice = 0, nslices = 1, gi = 0;
        if (leader) {
          if (!mbar_wait_cluster(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
          const uint32_t drawn = atomicAdd(ticket_counter, 1u);
          if (drawn == total_draws - 1u) atomicExch(ticket_counter, 0u);   // last draw of the launch
          valid = drawn < total_units ? 1 : 0;
          gi = (kChain && drawn >= units0) ? 1 : 0;
          const uint32_t ticket = gi ? drawn - units0 : drawn;              // index in that GEMM's own schedule
          PairUnit t = {0, 0, 1u << 16, 0};
          if (valid) t = (gi ? p1 : p0).pair_order[ticket];
          tn = static_cast<int32_t>(t.x); tpm = static_cast<int32_t>(t.y);
          tz_slice = static_cast<int32_t>(t.slice_of & 0xffffu); nslices = static_cast<int32_t>(t.slice_of >> 16);
          const unsigned long long now = (p0.trace || (kChain && p1.trace)) ? cusync::globalTimerNs() : 0ull;
          bars->sched_tile[slot][0] = tn; bars->sched_tile[slot][1] = tpm;
          bars->sched_tile[slot][2] = valid; bars->sched_tile[slot][3] = static_cast<int32_t>(ticket);
          bars->sched_tile[slot][4] = tz_slice; bars->sched_tile[slot][5] = nslices;
          bars->sched_tile[slot][6] = static_cast<int32_t>(t.ws_tile);
          bars->sched_tile[slot][7] = gi;
          bars->sched_time[slot] = now;
          // the same record into the peer's ring, then signal both
          const uint32_t pt = peer_sched_tile0 + slot * 32;
          st_cluster_u32(pt, static_cast<uint32_t>(tn)); st_cluster_u32(pt + 4, static_cast<uint32_t>(tpm));
          st_cluster_u32(pt + 8, static_cast<uint32_t>(valid)); st_cluster_u32(pt + 12, ticket);
          st_cluster_u32(pt + 16, static_cast<uint32_t>(tz_slice)); st_cluster_u32(pt + 20, static_cast<uint32_t>(nslices));
          st_cluster_u32(pt + 24, t.ws_tile);
          st_cluster_u32(pt + 28, static_cast<uint32_t>(gi));
          st_cluster_u32(peer_sched_time0 + slot * 8, static_cast<uint32_t>(now));
          st_cluster_u32(peer_sched_time0 + slot * 8 + 4, static_cast<uint32_t>(now >> 32));
          mbar_arrive(&bars->sched_full[slot]);
          mbar_arrive_cluster(peer_sched_full0 + slot * 8);
        } else {
          if (!mbar_wait_cluster(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
          tn = bars->sched_tile[slot][0]; tpm = bars->sched_tile[slot][1]; valid = bars->sched_tile[slot][2];
          tz_slice = bars->sched_tile[slot][4]; nslices = bars->sched_tile[slot][5];
          gi = kChain ? bars->sched_tile[slot][7] : 0;
          mbar_arrive_cluster(leader_sched_empty0 + slot * 8);
        }
        sched_it++;
        if (!valid) break;

        // The GEMM this unit belongs to: its parameters, stage and tensor maps.
        const GemmParams& p = gi ? p1 : p0;
        const cusync_stage_view_t& st = p.stage;
        const CUtensorMap* const tmA = gi ? mA1 : mA0;
        const CUtensorMap* const tmB = gi ? mB1 : mB0;
        const uint32_t wait_target = p.is_consumer ? st.iter * cusync::eval::waitValue(st.in_policy) : 0u;
        uint32_t sync_stride = 0;
        if (p.is_consumer) {
          const int kind = st.in_policy.kind;
          if (kind == CUSYNC_POLICY_TILESYNC || kind == CUSYNC_POLICY_STRIDEDTILESYNC) sync_stride = st.in_policy.tile_n;
          else if (kind == CUSYNC_POLICY_CONV2DTILESYNC) sync_stride = st.in_policy.tile_n * st.in_policy.p0;
        }
        // Dual GEMM (SiLU(A B) (.) (A B2)): the pair's 256-column MMA is [A B | A B2] of ONE 128-column output tile;
        // the leader CTA supplies the B half, its peer the B2 half, each the tile's own 128 columns.
        const bool dual = p.epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL;
        const CUtensorMap* const tmBr = dual && rank ? (gi ? mB2_1 : mB2_0) : tmB;
        const int n_off = dual ? tn * (BN / 2) : tn * BN;
        const int m_off = tpm * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;   // this CTA's 128 rows
        const int nb_off = dual ? n_off : n_off + static_cast<int>(rank) * (BN / 2);   // this CTA's half of B
        uint32_t ready_end = 0;
        long long wait_empty = 0;
        const int kb_per_slice = (p.num_k_blocks + nslices - 1) / nslices;
        const int kb_begin = tz_slice * kb_per_slice;
        const int kb_end = kb_begin + kb_per_slice < p.num_k_blocks ? kb_begin + kb_per_slice : p.num_k_blocks;
        for (int kb = kb_begin; kb < kb_end; kb++) {
          const uint32_t s = fills % C::kStages, ph = (fills / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait_cluster(&bars->empty[s], ph ^ 1u, ctx)) { ok = false; break; }
          if (p.trace) wait_empty += clock64() - c0;
          uint8_t* sa = ring + s * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          const uint32_t full_addr = leader_full0 + s * 8;
          const int k_base = kb * kPairBlockK;
          // A B operand that an earlier stage produces (the K^T and V operands of the attention GEMMs) is waited
          // for by 128-row blocks of the B matrix: this CTA's 128 n rows once per unit, or the stage's 128 k rows.
          if (p.b_sems != nullptr && (!p.b_kmajor || kb == kb_begin)) {
            const uint32_t block = static_cast<uint32_t>(p.b_kmajor ? nb_off : k_base) / kBlockM;
            const uint32_t bidx = p.b_sem_first + block * p.b_sem_stride;
            const uint32_t target = st.iter * p.b_sem_value;
            const bool in_range = p.b_kmajor ? nb_off < p.n : k_base < p.k;
            uint32_t seen = 0;
            if (in_range && !cusync::spinUntilAtLeast(p.b_sems + bidx, target, st.timeout_ns, &seen)) {
              bars->abort = 1u;
              cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_base), 3u, bidx,
                                    seen, target);
              ok = false;
              break;              // nothing of this stage is armed yet
            }
            fence_proxy_async_global();
          }
          // The leader's barrier collects the bytes of both CTAs.
          if (leader) mbar_expect_tx(&bars->full[s], 2 * C::kStageBytes);
          // B half: one 3-D box.  [k,n] weights: {64 columns, 128 k rows, 2 column chunks};
          // [n,k] weights: {64 k, 128 n rows, 2 k chunks}.
          if (p.b_kmajor) tma_load_3d_pair(sb, tmBr, full_addr, 0, nb_off, k_base / 64);
          else            tma_load_3d_pair(sb, tmBr, full_addr, 0, k_base, nb_off / 64);
          // The stage spans two 64-deep K chunks; each may open a new producer tile.
#pragma unroll 1
          for (int sub = 0; sub < kPairBlockK / kBlockK && ok; sub++) {
          const int k_off = k_base + sub * kBlockK;
          if (p.is_consumer && m_off < p.m && k_off < p.k) {
            const uint32_t tz = (kb == kb_begin && sub == 0) ? 1u : 0u;
            // A K slice may begin in the middle of a producer tile: its first K block is a sync point of the
            // K-walking policies as well, on the tile that contains it.
            if (static_cast<uint32_t>(k_off) >= ready_end &&
                (cusync::eval::isSync(st.in_policy, static_cast<uint32_t>(k_off), tz) || (tz && sync_stride))) {
              const uint32_t idx = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(k_off), st.prod_grid.x,
                                                           st.prod_grid.y);
              const uint32_t k_sync = sync_stride ? static_cast<uint32_t>(k_off) / sync_stride * sync_stride
                                                  : static_cast<uint32_t>(k_off);
              // Probe first: the tile's own semaphore and the next producer tiles along K are read with
              // independent relaxed loads (one memory round trip for all of them); only if the tile's own is
              // not there yet does the thread go on to wait for it.  How far the finished prefix reaches is
              // remembered, so later K-blocks skip the wait.  One fence makes the relaxed loads acquiring.
              uint32_t vals[kLookahead];
              uint32_t v_first = 0;
              if (sync_stride) {
                // TileSync / Conv2DTileSync number the producer tiles of a row with a constant step along K
                // (both orders are affine in the column), so one more evaluation gives every later index
                // without its integer divisions; the wrapping policies are evaluated one by one.
                const bool affine = st.in_policy.kind == CUSYNC_POLICY_TILESYNC ||
                                    st.in_policy.kind == CUSYNC_POLICY_CONV2DTILESYNC;
                uint32_t step = 0;
                if (affine && k_sync + sync_stride < static_cast<uint32_t>(p.k))
                  step = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off),
                                                 k_sync + sync_stride, st.prod_grid.x,
                                                 st.prod_grid.y) - idx;
                v_first = cusync::loadRelaxed(st.sems_wait + idx);
#pragma unroll
                for (int j = 0; j < kLookahead; j++) {
                  const uint32_t kk = k_sync + (j + 1) * sync_stride;
                  vals[j] = kk < static_cast<uint32_t>(p.k)
                                ? cusync::loadRelaxed(st.sems_wait + (affine ? idx + (j + 1) * step
                                      : cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off), kk,
                                                                st.prod_grid.x, st.prod_grid.y)))
                                : 0u;
                }
              }
              const bool probed_ready = sync_stride != 0 && v_first >= wait_target;
              uint32_t seen = 0;
              if (!probed_ready && !cusync::spinUntilAtLeast(st.sems_wait + idx, wait_target, st.timeout_ns, &seen)) {
                bars->abort = 1u;
                cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_off), tz,
                                      idx, seen, wait_target);
                ok = false;
                break;
              }
              if (sync_stride) {
                uint32_t ahead = 0;
#pragma unroll
                for (int j = 0; j < kLookahead; j++) {
                  if (ahead == static_cast<uint32_t>(j) && vals[j] >= wait_target) ahead++;
                }
                ready_end = k_sync + (ahead + 1) * sync_stride;
                if (ahead || probed_ready) cusync::fenceAcqRel();
              }
              fence_proxy_async_global();
            }
          }
          }
          // A: {64 k, 128 rows, 2 k chunks}.  Issued on the abort path too, so that the armed barrier
          // completes and the drain below terminates.
          tma_load_3d_pair(sa, tmA, full_addr, 0, m_off, k_base / 64);
          fills++;
          if (!ok) break;
        }
        if (p.trace) {
          const uint32_t tk = static_cast<uint32_t>(bars->sched_tile[slot][3]);
          if (2 * tk + rank < p.trace_capacity)
            p.trace[8ull * (2 * tk + rank) + 5] = static_cast<unsigned long long>(wait_empty);
        }
      }
      if (!ok) {
        bars->abort = 1u;
        if (leader) {
          // wait (bounded) for the copies of both CTAs that were armed on this CTA's barriers
          const uint32_t live = fills < static_cast<uint32_t>(C::kStages) ? fills : static_cast<uint32_t>(C::kStages);
          for (uint32_t j = 0; j < live; j++) {
            const uint32_t f = fills - 1u - j;
            const uint32_t s = f % C::kStages, ph = (f / C::kStages) & 1u;
            const uint64_t t0 = cusync::globalTimerNs();
            while (!mbar_try_wait_cluster(&bars->full[s], ph)) {
              if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
            }
          }
        } else {
          // the peer's copies complete on the leader's barriers, which it cannot wait on: give
          // them time to land before this CTA's shared memory goes away
          const uint64_t t0 = cusync::globalTimerNs();
          while (cusync::globalTimerNs() - t0 < 100000ull) __nanosleep(1000);
        }
      }
    }
  } else if (warp == 1) {
    // =====================================================================
    // MMA issuer (leader only)
    // =====================================================================
    if (lane == 0 && leader) {
      uint32_t drains = 0, sched_it = 0, acc_it = 0;
      bool ok = true, issued = false;
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
        const int valid = bars->sched_tile[slot][2];
        const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
        const int slice = bars->sched_tile[slot][4];
        const int nslices = bars->sched_tile[slot][5];
        const GemmParams& p = (kChain && bars->sched_tile[slot][7]) ? p1 : p0;
        mbar_arrive(&bars->sched_empty[slot]);
        sched_it++;
        if (!valid) break;
        // instruction descriptor: M = 256 across the pair, N = 256
        const uint32_t idesc = (1u << 4) | ((p.b_kmajor ? 0u : 1u) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                               (static_cast<uint32_t>((2 * kBlockM) >> 4) << 24);
        const uint32_t b_lbo = p.b_lbo, b_sbo = p.b_sbo, b_kstep = p.b_kstep;
        const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
        const long long t_tile0 = p.trace ? clock64() : 0;
        if (!mbar_wait_cluster(&bars->tmem_empty[acc], aph ^ 1u, ctx)) { ok = false; break; }
        tc_fence_after();
        const long long t_acc = p.trace ? clock64() : 0;
        long long wait_full = 0;
        const uint32_t d_tmem = tmem_base + acc * C::kAccCols;
        const int kb_per_slice = (p.num_k_blocks + nslices - 1) / nslices;
        const int kb_first = slice * kb_per_slice;
        const int kb_count = kb_first + kb_per_slice < p.num_k_blocks ? kb_per_slice : p.num_k_blocks - kb_first;
        for (int kb = 0; kb < kb_count; kb++) {
          const uint32_t s = drains % C::kStages, ph = (drains / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait_cluster(&bars->full[s], ph, ctx)) { ok = false; break; }
          if (p.trace) wait_full += clock64() - c0;
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + s * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int kk = 0; kk < kPairBlockK / kUmmaK; kk++) {
            // K-major operands: 64-deep chunks of 128 rows, 32 bytes per K step inside a chunk.
            // [k,n] B: 2048 bytes (16 rows) per K step, column chunks one leading offset apart.
            const uint32_t a_off = (kk >> 2) * kPairChunkBytes + (kk & 3) * 32;
            const uint32_t b_off = p.b_kmajor ? a_off : kk * b_kstep;
            const uint64_t adesc = make_smem_desc(sa + a_off, 16u, 1024u);
            const uint64_t bdesc = make_smem_desc(sb + b_off, b_lbo, b_sbo);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair_both(&bars->empty[s]);     // frees the ring slot in both CTAs
          issued = true;
          drains++;
        }
        if (!ok) break;
        umma_commit_pair_both(&bars->tmem_full[acc]);
        if (p.trace && 2 * ticket < p.trace_capacity) {
          p.trace[8ull * (2 * ticket) + 4] = static_cast<unsigned long long>(wait_full);
          p.trace[8ull * (2 * ticket) + 6] = static_cast<unsigned long long>(clock64() - t_tile0);
          p.trace[8ull * (2 * ticket) + 7] = static_cast<unsigned long long>(t_acc - t_tile0);
        }
        acc_it++;
      }
      if (!ok && issued) {
        umma_commit_pair_local(&bars->drain);
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(&bars->drain, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // =====================================================================
    // Epilogue (both CTAs, each for its own 128 rows)
    // =====================================================================
    const int ew = warp - kEpilogueWarp0;
    const int quarter = ew & 3;
    const int half = ew >> 2;
    uint8_t* buf = staging + ew * (32 * 128);
    uint32_t sched_it = 0, acc_it = 0, post_it = 0, split_it = 0;
    bool ok = true;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait_cluster(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_n = bars->sched_tile[slot][0];
      const int pair_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      const uint32_t nslices = static_cast<uint32_t>(bars->sched_tile[slot][5]);
      const uint32_t ws_slot = static_cast<uint32_t>(bars->sched_tile[slot][6]) * nslices;   // the tile's first slot
      const uint32_t slice = static_cast<uint32_t>(bars->sched_tile[slot][4]);
      const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
      const unsigned long long t_draw = bars->sched_time[slot];
      const int gi = kChain ? bars->sched_tile[slot][7] : 0;
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_sched_empty0 + slot * 8);
      sched_it++;
      if (!valid) break;
      const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
      const GemmParams& p = gi ? p1 : p0;
      const cusync_stage_view_t& st = p.stage;
      const CUtensorMap* const tmD = gi ? mD1 : mD0;
      const CUtensorMap* const tmWS = gi ? mWS1 : mWS0;
      if (!mbar_wait_cluster(&bars->tmem_full[acc], aph, ctx)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_mma_done = p.trace ? cusync::globalTimerNs() : 0ull;
      const bool dual = p.epilogue == CUSYNC_EPILOGUE_SILU_MUL_DUAL;       // a 128-column output tile from both halves
      const int n_off = dual ? tile_n * (BN / 2) : tile_n * BN;
      const int m_off = pair_m * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kAccCols;

      if (nslices > 1u) {
        // One K slice of the tile: add it to the workspace; the pair that brings the last slice finalises.
        // `post` is also used by unsplit tiles, the two split-K barriers only here: separate phase counters.
        bool last = false;
        ok = splitk_epilogue<BN>(p, tmWS, buf, bars, ctx, t_row, n_off, m_off, quarter, half, ew, lane, post_it & 1u,
                                 split_it & 1u, nslices, nullptr, leader_tmem_empty0 + acc * 8,
                                 static_cast<__half*>(p.d), p.ldd, &last,
                                 reinterpret_cast<float4*>(p.splitk_ws) + static_cast<size_t>(ws_slot) * kPairSlotVec4 +
                                     rank * (kPairSlotVec4 / 2),
                                 slice, tmD);
        acc_it++;
        if (ew == 0 && lane == 0) {
          if (!mbar_wait(&bars->splitk_done, split_it & 1u, ctx)) ok = false;
          else if (last && p.is_producer) {
            const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                         static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
            const uint32_t pv = cusync::eval::postValue(st.out_policy);
            __threadfence();
            if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
            else                                    cusync::addRelease(st.sems_post + idx, pv);
          }
        }
        post_it++;
        split_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (p.trace && ew == 0 && lane == 0 && 2 * ticket + rank < p.trace_capacity) {
          uint32_t smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          unsigned long long* rec = p.trace + 8ull * (2 * ticket + rank);
          rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
          rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
        }
        continue;
      }
      if (dual) epilogue_store_rows<BN / 2, true>(p, tmD, buf, t_row, n_off, m_off + quarter * 32, half, lane);
      else      epilogue_store_rows<BN, false>(p, tmD, buf, t_row, n_off, m_off + quarter * 32, half, lane);

      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tmem_empty0 + acc * 8);
      acc_it++;

      if (p.is_producer && m_off < p.m) {     // a pair's second half may lie past the last row tile
        if (lane == 0) {
          tma_store_wait_all();        // the bulk stores' writes are complete and visible to this thread
          // Epilogue warps run at their own pace: one that is a tile ahead must not arrive on `post`
          // while the previous tile's phase is still open (its arrival would close that phase early).
          if (!mbar_wait(&bars->post, (post_it & 1u) ^ 1u, ctx)) ok = false;
          mbar_arrive(&bars->post);
          if (ew == 0) {
            if (!mbar_wait(&bars->post, post_it & 1u, ctx)) ok = false;
            else {
              const uint32_t idx = cusync::eval::tileIndex(st.out_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(n_off), st.grid.x, st.grid.y);
              const uint32_t pv = cusync::eval::postValue(st.out_policy);
              cusync::fenceAcqRel();
              if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
              else                                    cusync::addRelease(st.sems_post + idx, pv);
            }
          }
        }
        post_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      if (p.trace && ew == 0 && lane == 0 && 2 * ticket + rank < p.trace_capacity) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long* rec = p.trace + 8ull * (2 * ticket + rank);
        rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
        rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // Teardown: nobody may leave while the peer can still signal its barriers or read its operands.
  tc_fence_before();
  __syncthreads();
  // A block that gave up does not post its tiles: release what waits on this stage without a bound of its own.
  if (bars->abort != 0u) {
    for (int gi = 0; gi < (kChain ? 2 : 1); gi++) {
      const cusync_stage_view_t& sg = (gi ? p1 : p0).stage;
      if ((gi ? p1 : p0).is_producer)
        cusync::releaseWaitersOnAbort(sg.sems_post, sg.grid.x * sg.grid.y * sg.grid.z, threadIdx.x, blockDim.x);
    }
  }
  // every post of this block happened before the barrier above: the block counts itself finished in each stage
  // it produced for
  if (threadIdx.x == 0) {
    if (p0.is_producer) cusync::countBlockFinished(p0.stage.started);
    if (kChain && p1.is_producer) cusync::countBlockFinished(p1.stage.started);
  }
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
cusync_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmWS,
                        const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  pair_kernel_body<false>(&tmA, &tmB, &tmD, &tmWS, &tmA, &tmB, &tmD, &tmWS, p, p, &tmB2, &tmB2);
}

// Two dependent GEMMs (both on CTA pairs) in one persistent grid; see pair_kernel_body.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
cusync_gemm_pair_chain_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                              const __grid_constant__ CUtensorMap tmD0, const __grid_constant__ CUtensorMap tmWS0,
                              const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                              const __grid_constant__ CUtensorMap tmD1, const __grid_constant__ CUtensorMap tmWS1,
                              const __grid_constant__ CUtensorMap tmB2_0, const __grid_constant__ CUtensorMap tmB2_1,
                              const __grid_constant__ GemmParams p0, const __grid_constant__ GemmParams p1) {
  pair_kernel_body<true>(&tmA0, &tmB0, &tmD0, &tmWS0, &tmA1, &tmB1, &tmD1, &tmWS1, p0, p1, &tmB2_0, &tmB2_1);
}

}  // namespace
