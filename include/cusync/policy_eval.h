// Run-time evaluation of a sync policy held as data (cusync_policy_t).
// One evaluator serves the typed policy classes of <cusync/policies.h>, the
// pre-compiled GEMM / conv kernels of the library, and host-side checks.
// The arithmetic is the reference's (src/include/cusync/policies.h:37-210,
// tile-orders.h:50-76, mlp.cu:76-101, attention.cu:51-70).
#pragma once

#include <stdint.h>
#include "../cusync_b200.h"
#include "cusync_defines.h"

namespace cusync {
namespace eval {

// Linear index of a block in a launch grid: x fastest for both orders.
CUSYNC_DEVICE_HOST uint32_t blockIndex(uint32_t gx, uint32_t gy, uint32_t bx, uint32_t by, uint32_t bz) {
  return bx + by * gx + bz * gx * gy;
}

// Linear index of block (bx, by, bz) under the grouped-rows order: groups of `rows` grid rows, the row
// index fastest inside a group, then the column; z outermost.
CUSYNC_DEVICE_HOST uint32_t groupedBlockIndex(uint32_t rows, uint32_t gx, uint32_t gy, uint32_t bx, uint32_t by,
                                              uint32_t bz) {
  const uint32_t group = by / rows;
  const uint32_t first = group * rows;
  const uint32_t height = gy - first < rows ? gy - first : rows;   // the last group may be short
  return bz * gx * gy + first * gx + bx * height + (by - first);
}

// Semaphore index of tile (tx, ty) under `order`: TransposeXY swaps the tile's
// coordinates before linearising, Identity does not.
CUSYNC_DEVICE_HOST uint32_t orderTileIndex(int order, uint32_t tx, uint32_t ty, uint32_t gx, uint32_t gy) {
  return order == CUSYNC_ORDER_TRANSPOSE_XY ? blockIndex(gx, gy, ty, tx, 0) : blockIndex(gx, gy, tx, ty, 0);
}

CUSYNC_DEVICE_HOST uint32_t waitValue(const cusync_policy_t& p) {
  switch (p.kind) {
    case CUSYNC_POLICY_ROWSYNC:
    case CUSYNC_POLICY_TILESYNC:
    case CUSYNC_POLICY_CONV2DTILESYNC:      return p.wait_value;
    case CUSYNC_POLICY_STRIDEDTILESYNC:     return p.p1;
    case CUSYNC_POLICY_CONSECUTIVETILESYNC: return (p.p0 / 8) / p.tile_n;
    default:                                return 0;
  }
}

CUSYNC_DEVICE_HOST uint32_t postValue(const cusync_policy_t& p) {
  switch (p.kind) {
    case CUSYNC_POLICY_ROWSYNC:
    case CUSYNC_POLICY_TILESYNC:
    case CUSYNC_POLICY_CONV2DTILESYNC:      return p.post_value;
    case CUSYNC_POLICY_STRIDEDTILESYNC:
    case CUSYNC_POLICY_CONSECUTIVETILESYNC: return 1;
    default:                                return 0;
  }
}

// tile = {row offset (elements), column / K offset (elements), z}; grid = the
// PRODUCER's tile grid (N tiles, M tiles, split-K).
CUSYNC_DEVICE_HOST uint32_t tileIndex(const cusync_policy_t& p, uint32_t tx, uint32_t ty,
                                      uint32_t gx, uint32_t gy) {
  switch (p.kind) {
    case CUSYNC_POLICY_ROWSYNC:
      return tx / p.tile_m;
    case CUSYNC_POLICY_TILESYNC:
      return orderTileIndex(p.order, tx / p.tile_m, ty / p.tile_n, gx, gy);
    case CUSYNC_POLICY_CONV2DTILESYNC:
      return orderTileIndex(p.order, tx / p.tile_m, (ty / p.tile_n) / p.p0, gx, gy);
    case CUSYNC_POLICY_STRIDEDTILESYNC: {
      uint32_t col = ty / p.tile_n, wrap = p.p0 / p.tile_n;
      if (col >= wrap) col -= wrap;
      return orderTileIndex(p.order, tx / p.tile_m, col, gx, gy);
    }
    case CUSYNC_POLICY_CONSECUTIVETILESYNC: {
      uint32_t group = (p.p0 / 8) / p.tile_n;
      return orderTileIndex(p.order, tx / p.tile_m, (ty / p.tile_n) / group, gx / group, gy);
    }
    default:
      return 0;
  }
}

CUSYNC_DEVICE_HOST bool isSync(const cusync_policy_t& p, uint32_t ty, uint32_t tz) {
  switch (p.kind) {
    case CUSYNC_POLICY_ROWSYNC:
    case CUSYNC_POLICY_CONSECUTIVETILESYNC: return tz == 1;
    case CUSYNC_POLICY_TILESYNC:
    case CUSYNC_POLICY_STRIDEDTILESYNC:     return ty % p.tile_n == 0;
    case CUSYNC_POLICY_CONV2DTILESYNC:      return (ty / p.tile_n) % p.p0 == 0;
    default:                                return false;
  }
}

}  // namespace eval
}  // namespace cusync
