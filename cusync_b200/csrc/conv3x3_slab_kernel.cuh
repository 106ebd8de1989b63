// cusync_conv3x3_slab_kernel: the 64 -> 64 channel 3x3 convolution with a resident filter and one input slab per
// tile.
#pragma once

#include "sm100_device.cuh"

namespace {

// ---------------------------------------------------------------------------
// 3x3 convolution, 64 -> 64 channels: the slab kernel
// ---------------------------------------------------------------------------
// The implicit-GEMM path (gemm_kernel_1cta.cuh, CONV) fetches one shifted copy of the input rows per filter tap (nine TMA boxes and
// nine barrier round trips per tile) and re-reads the 3x3 filter for every tile.  For the layer the conv chain
// is measured on (C = K = 64, src/ml-bench/volta_conv2d/ resnet sizes) both fit on chip:
//
//   * the whole filter (9 taps x 64 x 64 fp16 = 72 KB) is loaded ONCE per CTA and stays in shared memory;
//   * per tile ONE 4-D TMA box brings the input slab: conv_rows + 2 image rows of W + 2 pixels (the halo is the
//     box's out-of-range part, zero-filled = the padding), 64 channels = one 128-byte swizzle row per pixel;
//   * the MMA's M index runs over the slab's pixels in memory order (padded width W + 2), so tap (r, s) is the
//     same slab read from (r * (W + 2) + s) pixel rows further on: 36 tcgen05.mma per tile, back to back, with a
//     shared-memory descriptor whose start address moves by whole 128-byte rows (the 128-byte swizzle is a
//     function of the shared-memory address, so a start that is not a multiple of 8 rows needs nothing else;
//     the descriptor's base-offset field stays 0 - setting it to the start row's phase gave wrong products).
//     M rows that fall on the two padding columns of a slab row, or past conv_rows rows, are computed and dropped.
//
// Tile shape, stage grid, semaphores and policies are those of the general path: one tile = conv_rows whole image
// rows, waits on its own and the two neighbouring producer tiles, posts once.
//
// The scheduler works in groups of four tickets, one group ahead: the ticket draw, the schedule look-up and the
// semaphore probes of a tile are three dependent memory round trips (about 2 us, as long as two tiles' math
// here), and the fence that makes the probes acquiring costs over a thousand cycles, so all of it is issued for
// four tiles at once while the previous four are being loaded.  Every CTA draws exactly two groups past the end.
constexpr int kSlabStages = 4;
constexpr int kSlabBytes = 256 * 128;          // room for 256 pixel rows: the last tap reads up to row 2(W+2)+2+127
constexpr int kSlabFilterBytes = 9 * 64 * 128; // nine taps of [64 n][64 c]
constexpr int kSlabBN = 64;
constexpr uint32_t kSlabSmemBytes = 1024 + kSlabStages * kSlabBytes + kSlabFilterBytes + 1024;
constexpr int kSlabGroup = 4;                  // most tickets a block draws at a time
constexpr int kSlabIssuers = 2;                // threads that issue MMAs, alternating tiles

__global__ void __launch_bounds__(kThreads, 1)
cusync_conv3x3_slab_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmF,
                           const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slabs = smem;
  uint8_t* filt = smem + kSlabStages * kSlabBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(filt + kSlabFilterBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const cusync_stage_view_t& st = p.stage;
  WaitCtx ctx{&bars->abort, st.status, 2 * st.timeout_ns + 1000000000ull};
  const int wp = p.conv_w + 2;                         // padded slab width
  uint64_t* filt_full = &bars->splitk_counted;         // (split-K is not used by this kernel)
  // Four accumulators, one per slab stage: tile j of this CTA uses slab j % 4 and accumulator j % 4, and is
  // issued by MMA thread j % 2 (see below).  Their barriers live in the upper half of the ring's arrays.
  uint64_t* acc_full = &bars->full[kSlabStages];
  uint64_t* acc_empty = &bars->empty[kSlabStages];

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlabStages; i++) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < kSlabStages; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpilogueWarps); }
    for (int i = 0; i < kSchedSlots; i++) { mbar_init(&bars->sched_full[i], 1); mbar_init(&bars->sched_empty[i], kSlabIssuers + kEpilogueWarps + 1); }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->splitk_done, 1);     // the second MMA thread's drain barrier
    for (int i = 0; i < kSchedSlots; i++) mbar_init(&bars->post_slot[i], kEpilogueWarps);
    mbar_init(filt_full, 1);
    bars->abort = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
    if (p.is_producer) {
      if (blockIdx.x == 0) cusync::storeRelease(st.started, st.iter);
      cusync::addRelease(st.started + 1, 1u);
    }
  }
  if (warp == 0 && lane == 0) { prefetch_tensormap(&tmX); prefetch_tensormap(&tmF); }
  if (warp == 2) {
    tmem_alloc(&bars->tmem_base, kSlabStages * kSlabBN);
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
      // The filter: nine boxes {64 c, 64 n}, tap t at K offset t * C of the [k_out][r][s][c] matrix.
      mbar_expect_tx(filt_full, kSlabFilterBytes);
      for (int tap = 0; tap < 9; tap++) tma_load_2d(filt + tap * (64 * 128), &tmF, filt_full, tap * p.conv_c, 0);

      const uint32_t num_tiles = static_cast<uint32_t>(p.num_tiles);
      // Tickets are drawn in groups, and a group ahead, only as far as the grid can afford: a block that holds
      // tickets it is not yet working on keeps them from idle blocks.  With at most two tiles per block there is
      // no drawing ahead; groups grow to kSlabGroup tickets from sixteen tiles per block.  Every block draws
      // exactly one group that lies wholly past the end (two when it draws ahead), so the launch's last draw
      // starts at last_base.
      const bool ahead = num_tiles > 2u * gridDim.x;
      uint32_t group = num_tiles / (4u * gridDim.x);
      group = group < 1u ? 1u : (group > kSlabGroup ? kSlabGroup : group);
      const uint32_t groups_total = (num_tiles + group - 1u) / group + (ahead ? 2u : 1u) * gridDim.x;
      const uint32_t last_base = group * (groups_total - 1u);
      const uint32_t wait_target = p.is_consumer ? st.iter * cusync::eval::waitValue(st.in_policy) : 0u;
      const int span = p.conv_rows * p.conv_w;           // output pixels per tile
      uint32_t fills = 0, sched_it = 0;
      bool ok = true;

      // The policy's tile index is affine in the tile row (the column is always 0 here); when it is the row itself
      // (any x-fastest or transposed order over a one-column producer grid) the three integer divisions per
      // evaluation are skipped.
      auto policy_index = [&](uint32_t row) {
        return cusync::eval::tileIndex(st.in_policy, row * static_cast<uint32_t>(span), 0u, st.prod_grid.x, st.prod_grid.y);
      };
      const bool index_is_row = p.is_consumer && policy_index(0u) == 0u && policy_index(1u) == 1u &&
                                policy_index(num_tiles - 1u) == num_tiles - 1u;
      // semaphores a tile depends on: its own producer tile and the neighbours holding its halo rows
      auto sem_indices = [&](uint32_t ty, uint32_t* idx) {
        const int tin = static_cast<int>(ty) % p.conv_tiles_per_image;
        if (index_is_row) {
          idx[0] = ty;
          idx[1] = tin > 0 ? ty - 1u : ty;
          idx[2] = tin + 1 < p.conv_tiles_per_image ? ty + 1u : ty;
          return;
        }
        idx[0] = policy_index(ty);
        idx[1] = tin > 0 ? policy_index(ty - 1u) : idx[0];
        idx[2] = tin + 1 < p.conv_tiles_per_image ? policy_index(ty + 1u) : idx[0];
      };
      // Probes the dependencies of a group of tiles with relaxed loads (all in flight together), then ONE fence
      // makes them acquiring: the fence is the expensive part (over a thousand cycles here) and is paid once
      // per group, a tile ahead of need.  ready[j] tells whether tile j may be loaded without waiting.
      // Once the producer kernel of this run has finished altogether there is nothing left to probe.
      bool prod_done = false;
      auto probe_group = [&](uint32_t base, const uint32_t* ys, bool* ready) {
        if (!prod_done && cusync::producerFinished(st.prod_finished, st.prod_finish_target)) {
          prod_done = true;
          fence_proxy_async_global();     // the acquire (generic proxy) before every later TMA read (async proxy)
        }
        if (prod_done) {
#pragma unroll
          for (int j = 0; j < kSlabGroup; j++) ready[j] = true;
          return;
        }
        uint32_t v[kSlabGroup][3];
#pragma unroll
        for (int j = 0; j < kSlabGroup; j++) {
          if (j < static_cast<int>(group) && base + j < num_tiles) {
            uint32_t idx[3];
            sem_indices(ys[j], idx);
#pragma unroll
            for (int e = 0; e < 3; e++) v[j][e] = cusync::loadRelaxed(st.sems_wait + idx[e]);
          }
        }
#pragma unroll
        for (int j = 0; j < kSlabGroup; j++)
          ready[j] = j < static_cast<int>(group) && base + j < num_tiles && v[j][0] >= wait_target &&
                     v[j][1] >= wait_target && v[j][2] >= wait_target;
        cusync::fenceAcqRel();
        fence_proxy_async_global();     // acquire (generic proxy) before the TMA reads (async proxy)
      };

      // Pipeline: group 0 is being loaded, group 1 has its tickets (schedule entries and probes follow while
      // group 0 is worked on), group 2 is drawn at the top of the iteration.
      uint32_t base0 = atomicAdd(st.tile_counter, group);
      uint32_t base1 = ahead ? atomicAdd(st.tile_counter, group) : 0u;
      uint32_t y0[kSlabGroup], y1[kSlabGroup];
      bool ready0[kSlabGroup], ready1[kSlabGroup];
#pragma unroll
      for (int j = 0; j < kSlabGroup; j++) {
        y0[j] = j < static_cast<int>(group) && base0 + j < num_tiles ? st.tile_order[base0 + j].y : 0u;
        ready0[j] = !p.is_consumer;
        ready1[j] = !p.is_consumer;
      }
      if (p.is_consumer && base0 < num_tiles) probe_group(base0, y0, ready0);

      while (ok) {
        if (base0 >= num_tiles) {
          // this block's groups past the end are base0 and, when drawing ahead, base1; the launch's last draw
          // re-arms the counter (the reference resets on the last tile, cusync_device_defs.h:87-90)
          if (base0 == last_base || (ahead && base1 == last_base)) atomicExch(st.tile_counter, 0u);
          const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
          if (!mbar_wait(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
          bars->sched_tile[slot][2] = 0;
          bars->sched_tile[slot][3] = static_cast<int32_t>(base0);
          mbar_arrive(&bars->sched_full[slot]);
          sched_it++;
          break;
        }
        // for later groups: the draw of group 2 and the schedule entries of group 1 (both in flight while
        // group 0 is loaded)
        uint32_t base2 = 0u;
        if (ahead) {
          base2 = atomicAdd(st.tile_counter, group);
#pragma unroll
          for (int j = 0; j < kSlabGroup; j++)
            y1[j] = j < static_cast<int>(group) && base1 + j < num_tiles ? st.tile_order[base1 + j].y : 0u;
        }

#pragma unroll 1
        for (int j = 0; j < static_cast<int>(group) && ok; j++) {
          const uint32_t ticket = base0 + j;
          if (ticket >= num_tiles) break;
          const long long lc0 = p.trace ? clock64() : 0;
          const uint32_t ty = y0[j];
          if (p.is_consumer && !ready0[j]) {
            // not finished when probed: wait (bounded) for the tile itself and its two halo neighbours
            uint32_t idx[3];
            sem_indices(ty, idx);
            for (int e = 0; e < 3 && ok; e++) {
              uint32_t seen = 0;
              if (!cusync::spinUntilAtLeast(st.sems_wait + idx[e], wait_target, st.timeout_ns, &seen)) {
                bars->abort = 1u;
                cusync::recordTimeout(st.status, 1u, ty * static_cast<uint32_t>(span), 0u, static_cast<uint32_t>(e), idx[e],
                                      seen, wait_target);
                ok = false;
              }
            }
            fence_proxy_async_global();
          }
          const long long lc1 = p.trace ? clock64() : 0;
          const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
          if (!mbar_wait(&bars->sched_empty[slot], sph ^ 1u, ctx)) { ok = false; break; }
          bars->sched_tile[slot][0] = 0;
          bars->sched_tile[slot][1] = static_cast<int32_t>(ty);
          bars->sched_tile[slot][2] = 1;
          bars->sched_tile[slot][3] = static_cast<int32_t>(ticket);
          if (p.trace) bars->sched_time[slot] = cusync::globalTimerNs();
          mbar_arrive(&bars->sched_full[slot]);
          sched_it++;
          if (!ok) break;      // published, so that the other threads see the abort instead of a missing tile

          const int img = static_cast<int>(ty) / p.conv_tiles_per_image;
          const int h0 = (static_cast<int>(ty) % p.conv_tiles_per_image) * p.conv_rows;
          const long long lc2 = p.trace ? clock64() : 0;
          const uint32_t s = fills % kSlabStages, ph = (fills / kSlabStages) & 1u;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u, ctx)) { ok = false; break; }
          const long long lc3 = p.trace ? clock64() : 0;
          const uint32_t slab_bytes = static_cast<uint32_t>((p.conv_rows + 2) * wp * 128);
          mbar_expect_tx(&bars->full[s], slab_bytes);
          // box {64 channels, W + 2 pixels, conv_rows + 2 rows, 1 image} from pixel (-1, h0 - 1)
          tma_load_4d(slabs + s * kSlabBytes, &tmX, &bars->full[s], 0, -1, h0 - 1, img);
          fills++;
          if (p.trace && ticket < p.trace_capacity) {
            // loader's cycles for this tile: dependencies | schedule slot | free slab | TMA issue
            auto cap = [](long long v) { return static_cast<unsigned long long>(v < 0 ? 0 : (v > 4095 ? 4095 : v)); };
            p.trace[8ull * ticket + 5] = cap(lc1 - lc0) | (cap(lc2 - lc1) << 12) | (cap(lc3 - lc2) << 24) |
                                         (cap(clock64() - lc3) << 36);
          }
        }
        if (!ok) break;
        if (!ahead) {
          // the next group is drawn only now that this one is under way
          base1 = atomicAdd(st.tile_counter, group);
#pragma unroll
          for (int j = 0; j < kSlabGroup; j++)
            y1[j] = j < static_cast<int>(group) && base1 + j < num_tiles ? st.tile_order[base1 + j].y : 0u;
        }
        // group 1's dependencies, one group ahead of need
        if (p.is_consumer && base1 < num_tiles) probe_group(base1, y1, ready1);
        base0 = base1; base1 = base2;
#pragma unroll
        for (int j = 0; j < kSlabGroup; j++) { y0[j] = y1[j]; ready0[j] = ready1[j]; }
      }
      if (!ok) {
        bars->abort = 1u;
        // wait (bounded) for the copies in flight before the block's shared memory goes away
        const uint32_t live = fills < static_cast<uint32_t>(kSlabStages) ? fills : static_cast<uint32_t>(kSlabStages);
        for (uint32_t j = 0; j < live; j++) {
          const uint32_t f = fills - 1u - j;
          const uint32_t s = f % kSlabStages, ph = (f / kSlabStages) & 1u;
          const uint64_t t0 = cusync::globalTimerNs();
          while (!mbar_try_wait(&bars->full[s], ph)) {
            if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
          }
        }
      }
      // the filter copy must have landed too
      {
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(filt_full, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // =====================================================================
    // MMA issuers.  A 128 x 64 x 16 MMA keeps the tensor pipe busy for about a third of the time one thread
    // needs to issue it, so two threads issue: warp 1 the CTA's even tiles, warp 3 the odd ones, each into
    // its own accumulators.  Both walk the whole schedule ring to stay in step.
    // =====================================================================
    if (lane == 0) {
      const uint32_t me = warp == 1 ? 0u : 1u;
      const uint32_t idesc = make_idesc(kSlabBN, false);
      uint32_t drains = 0, sched_it = 0;
      bool ok = mbar_wait(filt_full, 0u, ctx);
      bool issued = false;
      const uint32_t filt_addr = smem_u32(filt);
      while (ok) {
        const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
        if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
        const int valid = bars->sched_tile[slot][2];
        const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
        mbar_arrive(&bars->sched_empty[slot]);
        sched_it++;
        if (!valid) break;
        const uint32_t s = drains % kSlabStages, ph = (drains / kSlabStages) & 1u;   // slab and accumulator of tile j
        const bool mine = (drains & 1u) == me;
        if (!mine) { drains++; continue; }
        const uint32_t acc = s;
        const long long t_tile0 = p.trace ? clock64() : 0;
        if (!mbar_wait(&acc_empty[acc], ph ^ 1u, ctx)) { ok = false; break; }
        const long long t_acc = p.trace ? clock64() : 0;
        if (!mbar_wait(&bars->full[s], ph, ctx)) { ok = false; break; }
        const long long t_full = p.trace ? clock64() : 0;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kSlabBN;
        const uint32_t slab_addr = smem_u32(slabs + s * kSlabBytes);
#pragma unroll 1
        for (int tap = 0; tap < 9; tap++) {
          const uint32_t a_row = static_cast<uint32_t>((tap / 3) * wp + tap % 3);     // first pixel row of this tap
          const uint32_t a_addr = slab_addr + a_row * 128u;
          const uint32_t b_addr = filt_addr + static_cast<uint32_t>(tap) * (64u * 128u);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; kk++) {
            const uint64_t adesc = make_smem_desc(a_addr + kk * 32, 16u, 1024u);
            const uint64_t bdesc = make_smem_desc(b_addr + kk * 32, 16u, 1024u);
            umma_f16(d_tmem, adesc, bdesc, idesc, (tap > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bars->empty[s]);
        umma_commit(&acc_full[acc]);
        issued = true;
        drains++;
        if (p.trace && ticket < p.trace_capacity) {
          p.trace[8ull * ticket + 4] = static_cast<unsigned long long>(t_full - t_acc);
          p.trace[8ull * ticket + 6] = static_cast<unsigned long long>(clock64() - t_tile0);
          p.trace[8ull * ticket + 7] = static_cast<unsigned long long>(t_acc - t_tile0);
        }
      }
      if (!ok && issued) {
        uint64_t* drain = me ? &bars->splitk_done : &bars->drain;
        umma_commit(drain);
        const uint64_t t0 = cusync::globalTimerNs();
        while (!mbar_try_wait(drain, 0u)) {
          if (cusync::globalTimerNs() - t0 > 1000000000ull) break;
        }
      }
    }
  } else if (warp >= kEpilogueWarp0) {
    // =====================================================================
    // Epilogue: lane = one M row = one slab pixel; warp (quarter, half) takes 32 of its 64 channels
    // =====================================================================
    const int ew = warp - kEpilogueWarp0;
    const int quarter = ew & 3;
    const int half = ew >> 2;
    uint32_t sched_it = 0, acc_it = 0;
    bool ok = true;
    const int mrow = quarter * 32 + lane;
    const int prow = mrow / wp, pcol = mrow % wp;       // image row within the tile, column
    const bool px_in = prow < p.conv_rows && pcol < p.conv_w;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      const uint32_t ticket = static_cast<uint32_t>(bars->sched_tile[slot][3]);
      const unsigned long long t_draw = p.trace ? bars->sched_time[slot] : 0ull;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->sched_empty[slot]);
      sched_it++;
      if (!valid) break;
      const uint32_t acc = acc_it % kSlabStages, aph = (acc_it / kSlabStages) & 1u;
      if (!mbar_wait(&acc_full[acc], aph, ctx)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_mma_done = p.trace ? cusync::globalTimerNs() : 0ull;
      const int m_off = tile_m * p.conv_rows * p.conv_w;      // first output pixel of the tile
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kSlabBN + half * 32, v);
      tmem_ld_wait();
      if (px_in) {
        __half* dst = static_cast<__half*>(p.d) + static_cast<size_t>(m_off + prow * p.conv_w + pcol) * p.ldd + half * 32;
#pragma unroll
        for (int q = 0; q < 4; q++) {
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      acc_it++;
      if (p.is_producer) {
        // Hand the tile to the posting thread (warp 2) and go on: the warp barrier above orders every lane's
        // stores before lane 0's arrival, the arrival (release) before the poster's wait (acquire), and the
        // poster's fence + release publish them device-wide.  The barrier belongs to the tile's schedule
        // slot, which the poster gives back only after it has posted: no warp can be a phase ahead on it.
        if (lane == 0) mbar_arrive(&bars->post_slot[slot]);
      }
      if (p.trace && ew == 0 && lane == 0 && ticket < p.trace_capacity) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        unsigned long long* rec = p.trace + 8ull * ticket;
        rec[0] = t_draw; rec[1] = t_mma_done; rec[2] = cusync::globalTimerNs();
        rec[3] = (static_cast<unsigned long long>(smid) << 32) | blockIdx.x;
      }
    }
  }

  else if (warp == 2 && lane == 0) {
    // =====================================================================
    // Poster: publishes each finished tile (CuStage::post, cusync_device_defs.h:55-72) so that the epilogue
    // warps do not sit out the device-wide fence.  Walks the schedule ring like everybody else.
    // =====================================================================
    uint32_t sched_it = 0;
    bool ok = true;
    while (ok) {
      const uint32_t slot = sched_it % kSchedSlots, sph = (sched_it / kSchedSlots) & 1u;
      if (!mbar_wait(&bars->sched_full[slot], sph, ctx)) { ok = false; break; }
      const int tile_m = bars->sched_tile[slot][1];
      const int valid = bars->sched_tile[slot][2];
      sched_it++;
      if (!valid || !p.is_producer) {
        mbar_arrive(&bars->sched_empty[slot]);
        if (!valid) break;
        continue;
      }
      {
        if (!mbar_wait(&bars->post_slot[slot], sph, ctx)) { ok = false; break; }
        const uint32_t m_off = static_cast<uint32_t>(tile_m * p.conv_rows * p.conv_w);
        const uint32_t idx = cusync::eval::tileIndex(st.out_policy, m_off, 0u, st.grid.x, st.grid.y);
        const uint32_t pv = cusync::eval::postValue(st.out_policy);
        // (the release below is the fence: no separate one)
        if (st.opts & CUSYNC_OPT_NO_ATOMIC_ADD) cusync::storeRelease(st.sems_post + idx, pv * st.iter);
        else                                    cusync::addRelease(st.sems_post + idx, pv);
        mbar_arrive(&bars->sched_empty[slot]);      // only now may the slot (and its post barrier) be reused
      }
    }
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
    tmem_dealloc(tmem_base, kSlabStages * kSlabBN);
  }
}

}  // namespace
