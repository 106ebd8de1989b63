// Tile orders: how tiles are numbered (the order blocks take them in) and how a
// tile maps to a block of the launch grid.  API of the reference's
// src/include/cusync/tile-orders.h (GenericTileOrder, TransposeXYOrder,
// IdentityOrder); the arithmetic lives in policy_eval.h so the pre-compiled
// kernels and these classes cannot disagree.
//
// A user-defined order derives from GenericTileOrder<Itself> and provides
//   uint32_t blockIndex(const dim3& grid, const dim3& block);
//   dim3     tileToBlock(const dim3& tile);
// Such orders work with kernels compiled against these headers; the library's
// pre-compiled GEMM kernels accept the two built-in orders only.
#pragma once

#include <stdint.h>
#include "cusync_defines.h"
#include "policy_eval.h"

namespace cusync {

template <typename Child>
struct GenericTileOrder {
  // Built-in orders override this with their CUSYNC_ORDER_* value.
  static constexpr int kOrderKind = -1;

  CUSYNC_DEVICE_HOST uint32_t tileIndex(const dim3& tile, const dim3& grid) {
    Child self;
    return self.blockIndex(grid, self.tileToBlock(tile));
  }
};

// Tile {x, y, z} runs on block {y, x, z}; blocks are numbered x-fastest.
struct TransposeXYOrder : public GenericTileOrder<TransposeXYOrder> {
  static constexpr int kOrderKind = CUSYNC_ORDER_TRANSPOSE_XY;
  CUSYNC_DEVICE_HOST uint32_t blockIndex(const dim3& grid, const dim3& block) {
    return eval::blockIndex(grid.x, grid.y, block.x, block.y, block.z);
  }
  CUSYNC_DEVICE_HOST dim3 tileToBlock(const dim3& tile) { return dim3(tile.y, tile.x, tile.z); }
};

// Tile {x, y, z} runs on block {x, y, z}; blocks are numbered x-fastest.
struct IdentityOrder : public GenericTileOrder<IdentityOrder> {
  static constexpr int kOrderKind = CUSYNC_ORDER_IDENTITY;
  CUSYNC_DEVICE_HOST uint32_t blockIndex(const dim3& grid, const dim3& block) {
    return eval::blockIndex(grid.x, grid.y, block.x, block.y, block.z);
  }
  CUSYNC_DEVICE_HOST dim3 tileToBlock(const dim3& tile) { return dim3(tile.x, tile.y, tile.z); }
};

// Addition: blocks are taken in groups of Rows grid rows, row index fastest inside a group (see
// CUSYNC_ORDER_GROUPED).  Tiles map to blocks like TransposeXYOrder.
template <uint32_t Rows>
struct GroupedRowsOrder : public GenericTileOrder<GroupedRowsOrder<Rows>> {
  static_assert(Rows >= 1, "group height must be positive");
  static constexpr int kOrderKind = CUSYNC_ORDER_GROUPED(Rows);
  CUSYNC_DEVICE_HOST uint32_t blockIndex(const dim3& grid, const dim3& block) {
    return eval::groupedBlockIndex(Rows, grid.x, grid.y, block.x, block.y, block.z);
  }
  CUSYNC_DEVICE_HOST dim3 tileToBlock(const dim3& tile) { return dim3(tile.y, tile.x, tile.z); }
};

}  // namespace cusync
