// cusync_gemm_kernel<BN, DUAL, CONV>: the one-CTA-per-tile persistent GEMM / implicit-GEMM convolution kernel
// (roles and protocol are described at the top of gemm_sm100.cu).
#pragma once

#include "sm100_device.cuh"

namespace {

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <int BN, bool DUAL, bool CONV = false>
__global__ void __launch_bounds__(kThreads, 1)
cusync_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmD,
                   const __grid_constant__ CUtensorMap tmWS, const GemmParams p) {
  using C = Cfg<BN, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle patterns repeat every 1024 bytes: align the ring to that.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(staging + C::kStagingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const cusync_stage_view_t& st = p.stage;
  WaitCtx ctx{&bars->abort, st.status, 2 * st.timeout_ns + 1000000000ull};

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; i++) { mbar_init(&bars->tmem_full[i], 1); mbar_init(&bars->tmem_empty[i], kEpilogueWarps); }
    for (int i = 0; i < kSchedSlots; i++) { mbar_init(&bars->sched_full[i], 1); mbar_init(&bars->sched_empty[i], 1 + kEpilogueWarps); }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->post, kEpilogueWarps);
    mbar_init(&bars->splitk_counted, 1);
    mbar_init(&bars->splitk_done, kEpilogueWarps);
    bars->abort = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    // "Kernel started" words the wait kernel polls: [0] follows the reference
    // (block 0 stores iter, cusync_device_defs.h:78-83); [1] counts resident blocks.
    if (p.is_producer) {
      if (blockIdx.x == 0) cusync::storeRelease(st.started, st.iter);
      cusync::addRelease(st.started + 1, 1u);
    }
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA); prefetch_tensormap(&tmB); prefetch_tensormap(&tmD);
    if (DUAL) prefetch_tensormap(&tmB2);
  }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  cusync::allowDependentLaunch();      // this block is resident: a dependent consumer may be launched

  if (warp == 0) {
    // =====================================================================
    // Scheduler + TMA loader
    // =====================================================================
    if (lane == 0) {
      uint32_t fills = 0, sched_it = 0;
      bool ok = true;
      // Once the producer kernel of this run has finished altogether there is nothing left to wait for: the
      // tiles that follow skip their semaphore probes (checked once per tile until it is so).
      bool prod_done = false;
      const uint32_t total_draws = static_cast<uint32_t>(p.num_tiles) + gridDim.x;
      const uint32_t wait_target = p.is_consumer ? st.iter * cusync::eval::waitValue(st.in_policy) : 0u;
      // Distance along K between two sync points of the input policy (0: it syncs once per tile).
      uint32_t sync_stride = 0;
      if (p.is_consumer) {
        const int kind = st.in_policy.kind;
        if (kind == CUSYNC_POLICY_TILESYNC || kind == CUSYNC_POLICY_STRIDEDTILESYNC) sync_stride = st.in_policy.tile_n;
        else if (kind == CUSYNC_POLICY_CONV2DTILESYNC) sync_stride = st.in_policy.tile_n * st.in_policy.p0;
      }
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
        const uint32_t ticket = atomicAdd(st.tile_counter, 1u);
        // Every block draws exactly one ticket past the end, so the draw
        // numbered total_draws-1 is the launch's last: it re-arms the counter
        // (the reference resets on the last tile, cusync_device_defs.h:87-90).
        if (ticket == total_draws - 1u) atomicExch(st.tile_counter, 0u);
        const bool valid = ticket < static_cast<uint32_t>(p.num_tiles);
        cusync_dim3_t t = {0, 0, 0};
        if (valid) t = st.tile_order[ticket];
        bars->sched_tile[slot][0] = static_cast<int32_t>(t.x);
        bars->sched_tile[slot][1] = static_cast<int32_t>(t.y);
        bars->sched_tile[slot][2] = valid ? 1 : 0;
        bars->sched_tile[slot][3] = static_cast<int32_t>(ticket);
        bars->sched_tile[slot][4] = static_cast<int32_t>(t.z);
        if (p.trace) bars->sched_time[slot] = cusync::globalTimerNs();
        mbar_arrive(&bars->sched_full[slot]);
        sched_it++;
        if (!valid) break;

        const int n_off = static_cast<int>(t.x) * BN;
        // Row offset of the tile: 128 matrix rows, or for a convolution conv_rows image rows of output pixels.
        const int m_off = CONV ? static_cast<int>(t.y) * p.conv_rows * p.conv_w : static_cast<int>(t.y) * kBlockM;
        const int img = CONV ? static_cast<int>(t.y) / p.conv_tiles_per_image : 0;
        const int h0 = CONV ? (static_cast<int>(t.y) % p.conv_tiles_per_image) * p.conv_rows : 0;
        // K slice of this work unit (the whole K walk without split-K)
        const int kb_begin = static_cast<int>(t.z) * p.k_blocks_per_split;
        const int kb_end = kb_begin + p.k_blocks_per_split < p.num_k_blocks ? kb_begin + p.k_blocks_per_split
                                                                           : p.num_k_blocks;
        uint32_t ready_end = 0;   // K offset below which this tile's producer tiles are known finished
        long long wait_empty = 0;
        if (p.is_consumer && !prod_done && cusync::producerFinished(st.prod_finished, st.prod_finish_target)) {
          prod_done = true;
          fence_proxy_async_global();     // the acquire (generic proxy) before every later TMA read (async proxy)
        }
        for (int kb = kb_begin; kb < kb_end; kb++) {
          const uint32_t s = fills % C::kStages, ph = (fills / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u, ctx)) { ok = false; break; }
          if (p.trace) wait_empty += clock64() - c0;
          uint8_t* sa = ring + s * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          // A convolution's A box holds conv_rows * conv_w pixel rows of 128 bytes, not the full 128.
          mbar_expect_tx(&bars->full[s], CONV ? static_cast<uint32_t>(p.conv_rows * p.conv_w * 128 + C::kNumB * C::kBBytes)
                                              : static_cast<uint32_t>(C::kStageBytes));
          const int k_off = kb * kBlockK;
          // Convolution: K block kb is channel chunk kb / 9, filter tap (r, s) = kb % 9; the filter is
          // [k_out][r][s][c], so its K offset is tap * C + chunk * 64.
          const int tap = CONV ? kb % 9 : 0, chunk = CONV ? kb / 9 : 0;
          // Weights first: they never depend on the producer kernel.
          if (CONV) {
            tma_load_2d(sb, &tmB, &bars->full[s], tap * p.conv_c + chunk * kBlockK, n_off);
          } else if (p.b_kmajor) {
            tma_load_2d(sb, &tmB, &bars->full[s], k_off, n_off);
            if (DUAL) tma_load_2d(sb + C::kBBytes, &tmB2, &bars->full[s], k_off, n_off);
          } else if (p.b_chunked3d) {
            // one box {64 columns, kBlockK rows, BN/64 chunks}: a TMA instruction costs the issuing
            // thread over a hundred cycles, so fewer and larger boxes keep the loader ahead of the MMAs
            tma_load_3d(sb, &tmB, &bars->full[s], 0, k_off, n_off / 64);
            if (DUAL) tma_load_3d(sb + C::kBBytes, &tmB2, &bars->full[s], 0, k_off, n_off / 64);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; j++)
              tma_load_2d(sb + j * (kBlockK * 128), &tmB, &bars->full[s], n_off + j * 64, k_off);
            if (DUAL) {
#pragma unroll
              for (int j = 0; j < BN / 64; j++)
                tma_load_2d(sb + C::kBBytes + j * (kBlockK * 128), &tmB2, &bars->full[s], n_off + j * 64, k_off);
            }
          }
          // Consumer wait, at the load of the dependent A K-block.
          if (p.is_consumer && !prod_done) {
            const uint32_t tz = kb == kb_begin ? 1u : 0u;
            // A K slice (split-K) may begin in the middle of a producer tile: its first K block is a sync point
            // of the K-walking policies as well, on the tile that contains it.
            if (static_cast<uint32_t>(k_off) >= ready_end &&
                (cusync::eval::isSync(st.in_policy, static_cast<uint32_t>(k_off), tz) || (tz && sync_stride))) {
              const uint32_t idx = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off),
                                                           static_cast<uint32_t>(k_off), st.prod_grid.x,
                                                           st.prod_grid.y);
              // K offset at which the producer tile holding k_off begins
              const uint32_t k_sync = sync_stride ? static_cast<uint32_t>(k_off) / sync_stride * sync_stride
                                                  : static_cast<uint32_t>(k_off);
              uint32_t seen = 0;
              bool wait_ok = true;
              if (CONV) {
                // A 3x3 stencil reads, besides the tile's own producer tile, the image rows just above and below
                // it: they belong to the neighbouring producer tiles of the same image, which the reference's
                // policy does not wait for (it relies on tile order).  All three are needed at EVERY channel
                // chunk of the K walk.  One probe covers this chunk and the ones after it: the three rows'
                // semaphores of up to kConvProbe chunks are read with independent relaxed loads (one memory round
                // trip for all), one fence makes them acquiring, and ready_end remembers how far all three rows
                // were finished, so the later chunks of the tile pass without touching memory.
                constexpr int kConvProbe = 8;
                const int tin = static_cast<int>(t.y) % p.conv_tiles_per_image;
                const int span = p.conv_rows * p.conv_w;
                const bool has_up = tin > 0, has_dn = tin + 1 < p.conv_tiles_per_image;
                const uint32_t i_up = has_up ? cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off - span),
                                                   static_cast<uint32_t>(k_off), st.prod_grid.x, st.prod_grid.y) : idx;
                const uint32_t i_dn = has_dn ? cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off + span),
                                                   static_cast<uint32_t>(k_off), st.prod_grid.x, st.prod_grid.y) : idx;
                // the tile orders are affine in the column: one more evaluation per row gives its step along K
                uint32_t step = 0, step_up = 0, step_dn = 0;
                if (k_sync + sync_stride < static_cast<uint32_t>(p.k)) {
                  const uint32_t kn = k_sync + sync_stride;
                  step = cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off), kn, st.prod_grid.x,
                                                 st.prod_grid.y) - idx;
                  step_up = has_up ? cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off - span), kn,
                                                             st.prod_grid.x, st.prod_grid.y) - i_up : step;
                  step_dn = has_dn ? cusync::eval::tileIndex(st.in_policy, static_cast<uint32_t>(m_off + span), kn,
                                                             st.prod_grid.x, st.prod_grid.y) - i_dn : step;
                }
                uint32_t v[kConvProbe][3];
#pragma unroll
                for (int j = 0; j < kConvProbe; j++) {
                  const bool in = k_sync + static_cast<uint32_t>(j) * sync_stride < static_cast<uint32_t>(p.k);
                  v[j][0] = in ? cusync::loadRelaxed(st.sems_wait + idx + j * step) : 0u;
                  v[j][1] = in ? cusync::loadRelaxed(st.sems_wait + i_up + j * step_up) : 0u;
                  v[j][2] = in ? cusync::loadRelaxed(st.sems_wait + i_dn + j * step_dn) : 0u;
                }
                uint32_t chunks_ready = 0;
#pragma unroll
                for (int j = 0; j < kConvProbe; j++) {
                  if (chunks_ready == static_cast<uint32_t>(j) && v[j][0] >= wait_target && v[j][1] >= wait_target &&
                      v[j][2] >= wait_target)
                    chunks_ready++;
                }
                if (chunks_ready == 0) {
                  // this chunk is not there yet: wait (bounded) for the tile itself and its two neighbours
                  const uint32_t need[3] = {idx, i_up, i_dn};
                  for (int e = 0; e < 3 && wait_ok; e++) {
                    if (!cusync::spinUntilAtLeast(st.sems_wait + need[e], wait_target, st.timeout_ns, &seen)) {
                      cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_off),
                                            e == 0 ? tz : 2u, need[e], seen, wait_target);
                      wait_ok = false;
                    }
                  }
                  chunks_ready = 1;
                } else {
                  cusync::fenceAcqRel();
                }
                ready_end = k_sync + chunks_ready * sync_stride;
              } else {
                // Probe first: the tile's own semaphore and the next producer tiles along K are read with
                // independent relaxed loads (one memory round trip for all of them); only if the tile's own is
                // not there yet does the thread go on to wait for it.  How far the finished prefix reaches is
                // remembered, so later K-blocks skip the wait.  One fence makes the relaxed loads acquiring.
                uint32_t vals[kLookahead];
                uint32_t v_first = 0;
                if (sync_stride) {
                  // TileSync numbers the producer tiles of a row with a constant step along K (the orders are
                  // affine in the column), so one more evaluation gives every later index without its integer
                  // divisions; the wrapping policies are evaluated one by one.
                  const bool affine = st.in_policy.kind == CUSYNC_POLICY_TILESYNC;
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
                if (!probed_ready && !cusync::spinUntilAtLeast(st.sems_wait + idx, wait_target, st.timeout_ns, &seen)) {
                  cusync::recordTimeout(st.status, 1u, static_cast<uint32_t>(m_off), static_cast<uint32_t>(k_off), tz,
                                        idx, seen, wait_target);
                  wait_ok = false;
                }
                if (wait_ok && sync_stride) {
                  uint32_t ahead = 0;
#pragma unroll
                  for (int j = 0; j < kLookahead; j++) {
                    if (ahead == static_cast<uint32_t>(j) && vals[j] >= wait_target) ahead++;
                  }
                  ready_end = k_sync + (ahead + 1) * sync_stride;
                  if (ahead || probed_ready) cusync::fenceAcqRel();
                }
              }
              if (!wait_ok) {
                bars->abort = 1u;
                // The stage was armed: give it its A bytes anyway so the
                // barrier completes and the drain below terminates.
                if (CONV) tma_load_4d(sa, &tmA, &bars->full[s], chunk * kBlockK, tap % 3 - 1, h0 + tap / 3 - 1, img);
                else      tma_load_2d(sa, &tmA, &bars->full[s], k_off, m_off);
                fills++;
                ok = false;
                break;
              }
              // Order the acquire (generic proxy) before the TMA read (async proxy).
              fence_proxy_async_global();
            }
          }
          // Convolution: the box {64 channels, W pixels, conv_rows rows, 1 image} shifted by the tap; the
          // TMA zero-fills what falls outside the image, which is the padding.
          if (CONV) tma_load_4d(sa, &tmA, &bars->full[s], chunk * kBlockK, tap % 3 - 1, h0 + tap / 3 - 1, img);
          else      tma_load_2d(sa, &tmA, &bars->full[s], k_off, m_off);
          fills++;
        }
        if (p.trace && ticket < p.trace_capacity) p.trace[8ull * ticket + 5] = static_cast<unsigned long long>(wait_empty);
      }
      if (!ok) {
        // Abort path: wait (bounded) for every copy still in flight before the
        // block's shared memory goes away.
        bars->abort = 1u;
        const uint32_t live = fills < static_cast<uint32_t>(C::kStages) ? fills : static_cast<uint32_t>(C::kStages);
        for (uint32_t j = 0; j < live; j++) {
          const uint32_t f = fills - 1u - j;
          const uint32_t s = f % C::kStages, ph = (f / C::kStages) & 1u;
          const uint64_t t0 = cusync::globalTimerNs();
          while (!mbar_try_wait(&bars->full[s], ph)) {
            if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // =====================================================================
    // MMA issuer
    // =====================================================================
    if (lane == 0) {
      // Dual-B tiles sit back to back in the ring (second operand right after the first, same chunking), so
      // while both fit one instruction they are multiplied as a single 2*BN-wide B: accumulator columns
      // [0, BN) are A*B, [BN, 2BN) are A*B2.
      constexpr bool kFusedDual = DUAL && 2 * BN <= 256;
      const uint32_t idesc = make_idesc(kFusedDual ? 2 * BN : BN, !p.b_kmajor);
      const uint32_t b_lbo = p.b_lbo, b_sbo = p.b_sbo, b_kstep = p.b_kstep;
      uint32_t drains = 0, sched_it = 0, acc_it = 0;
      bool ok = true;
      bool issued = false;
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
        const int valid = bars->sched_tile[slot][2];
        const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
        const int slice = bars->sched_tile[slot][4];
        mbar_arrive(&bars->sched_empty[slot]);
        sched_it++;
        if (!valid) break;
        const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
        const long long t_tile0 = p.trace ? clock64() : 0;
        if (!mbar_wait(&bars->tmem_empty[acc], aph ^ 1u, ctx)) { ok = false; break; }
        tc_fence_after();
        const long long t_acc = p.trace ? clock64() : 0;
        long long wait_full = 0;
        const uint32_t d_tmem = tmem_base + acc * C::kAccCols;
        const int kb_first = slice * p.k_blocks_per_split;
        const int kb_count = kb_first + p.k_blocks_per_split < p.num_k_blocks ? p.k_blocks_per_split
                                                                             : p.num_k_blocks - kb_first;
        for (int kb = 0; kb < kb_count; kb++) {
          const uint32_t s = drains % C::kStages, ph = (drains / C::kStages) & 1u;
          const long long c0 = p.trace ? clock64() : 0;
          if (!mbar_wait(&bars->full[s], ph, ctx)) { ok = false; break; }
          if (p.trace) wait_full += clock64() - c0;
          tc_fence_after();
          const uint32_t sa = smem_u32(ring + s * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; kk++) {
            const uint64_t adesc = make_smem_desc(sa + kk * 32, 16u, 1024u);
            const uint64_t bdesc = make_smem_desc(sb + kk * b_kstep, b_lbo, b_sbo);
            const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
            umma_f16(d_tmem, adesc, bdesc, idesc, accumulate);
            if (DUAL && !kFusedDual) {
              const uint64_t b2desc = make_smem_desc(sb + C::kBBytes + kk * b_kstep, b_lbo, b_sbo);
              umma_f16(d_tmem + BN, adesc, b2desc, idesc, accumulate);
            }
          }
          umma_commit(&bars->empty[s]);   // frees the ring slot when these MMAs retire
          issued = true;
          drains++;
        }
        if (!ok) break;
        umma_commit(&bars->tmem_full[acc]);
        if (p.trace && ticket < p.trace_capacity) {
          p.trace[8ull * ticket + 4] = static_cast<unsigned long long>(wait_full);
          p.trace[8ull * ticket + 6] = static_cast<unsigned long long>(clock64() - t_tile0);
          p.trace[8ull * ticket + 7] = static_cast<unsigned long long>(t_acc - t_tile0);
        }
        acc_it++;
      }
      if (!ok && issued) {
        // Let outstanding MMAs retire before tensor memory is released.
        umma_commit(&bars->drain);
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(&bars->drain, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // =====================================================================
    // Epilogue
    // =====================================================================
    const int ew = warp - kEpilogueWarp0;
    const int quarter = ew & 3;                        // == warp % 4: the TMEM lanes this warp may read
    const int half = ew >> 2;                          // which 64-column chunks of the tile it takes
    uint8_t* buf = staging + ew * (32 * 128);
    uint32_t sched_it = 0, acc_it = 0, post_it = 0;
    bool ok = true;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_n = bars->sched_tile[slot][0];
      const int tile_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
      const unsigned long long t_draw = p.trace ? bars->sched_time[slot] : 0ull;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->sched_empty[slot]);
      sched_it++;
      if (!valid) break;
      const uint32_t acc = acc_it & 1u, aph = (acc_it >> 1) & 1u;
      if (!mbar_wait(&bars->tmem_full[acc], aph, ctx)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_mma_done = p.trace ? cusync::globalTimerNs() : 0ull;
      const int n_off = tile_n * BN, m_off = CONV ? tile_m * p.conv_rows * p.conv_w : tile_m * kBlockM;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kAccCols;

      if (CONV) {
        // One output pixel per lane: its BN channels are contiguous in NHWC, so each lane stores its own
        // 128-byte pieces directly.  Rows past conv_rows * conv_w are padding of the 128-row MMA.
        const int row = quarter * 32 + lane;
        const bool row_in = row < p.conv_rows * p.conv_w;
#pragma unroll 1
        for (int c = half; c < BN / kStoreCols; c += 2) {
          uint32_t v[64];
          tmem_ld_32x32b_x32(t_row + c * 64, v);
          tmem_ld_32x32b_x32(t_row + c * 64 + 32, v + 32);
          tmem_ld_wait();
          if (row_in) {
            __half* dst = static_cast<__half*>(p.d) + static_cast<size_t>(m_off + row) * p.ldd + n_off + c * 64;
#pragma unroll
            for (int q = 0; q < 8; q++) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; e++) {
                float x0 = __uint_as_float(v[8 * q + 2 * e]), x1 = __uint_as_float(v[8 * q + 2 * e + 1]);
                if (p.epilogue == CUSYNC_EPILOGUE_RELU) { x0 = fmaxf(x0, 0.0f); x1 = fmaxf(x1, 0.0f); }
                w[e] = pack_half2(x0, x1);
              }
              *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
        acc_it++;
        if (p.is_producer) {
          // Every lane's stores are ordered before lane 0's arrival by the warp barrier above, the arrival (a
          // release) before the posting lane's wait (an acquire), and that lane's fence + release publish them
          // device-wide (releases are cumulative): no device-wide fence per warp.
          if (lane == 0) {
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
                // (the release below is the fence: no separate one, which costs the whole SM's stores a wait)
                if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
                else                                    cusync::addRelease(st.sems_post + idx, pv);
              }
            }
          }
          post_it++;
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
          uint32_t smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          unsigned long long* rec = p.trace + 8ull * ticket;
          rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
          rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
        }
        continue;
      }
      if (!DUAL && p.split_k > 1) {
        // Split-K: add this slice's part; the block that brings the last slice finalises and posts.
        bool last = false;
        ok = splitk_epilogue<BN>(p, &tmWS, buf, bars, ctx, t_row, n_off, m_off, quarter, half, ew, lane, post_it & 1u,
                                 post_it & 1u, static_cast<uint32_t>(p.split_k), &bars->tmem_empty[acc], 0u,
                                 static_cast<__half*>(p.d), p.ldd, &last);
        acc_it++;
        if (ew == 0 && lane == 0) {
          if (!mbar_wait(&bars->splitk_done, post_it & 1u, ctx)) ok = false;
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
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
          uint32_t smid;
          asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
          unsigned long long* rec = p.trace + 8ull * ticket;
          rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
          rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
        }
        continue;
      }
      epilogue_store_rows<BN, DUAL>(p, &tmD, buf, t_row, n_off, m_off + quarter * 32, half, lane);
      // Accumulator buffer is free for the MMA warp again.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
      acc_it++;

      if (p.is_producer) {
        // Publish the tile only after every store of it has fully completed:
        // each warp's issuing lane waits for its own bulk stores, then arrives
        // on `post`; the first epilogue warp's lane collects the four arrivals
        // (bounded) and performs the single release.
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
              cusync::fenceAcqRel();      // (one per tile of a GEMM: cheap; the tiles' writes came from bulk stores)
              if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
              else                                    cusync::addRelease(st.sems_post + idx, pv);
            }
          }
        }
        post_it++;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long* rec = p.trace + 8ull * ticket;
        rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
        rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // Teardown (normal and abort paths alike).
  tc_fence_before();
  __syncthreads();
  // A block that gave up does not post its tiles: release what waits on this stage without a bound of its own.
  if (bars->abort != 0u && p.is_producer)
    cusync::releaseWaitersOnAbort(st.sems_post, st.grid.x * st.grid.y * st.grid.z, threadIdx.x, blockDim.x);
  // every post of this block happened before the barrier above: the block counts itself finished
  if (p.is_producer && threadIdx.x == 0) cusync::countBlockFinished(st.started);
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

}  // namespace
