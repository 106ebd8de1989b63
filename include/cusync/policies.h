// Synchronisation policies.  A policy answers four questions about a tile
// {x = row offset, y = column (or K) offset, z}:
//   waitValue(tile, grid)  value the semaphore must reach (times the run count)
//   postValue(tile, grid)  value a finished tile adds
//   tileIndex(tile, grid)  which semaphore
//   isSync(tile, grid)     whether this wait call synchronises at all
// Class names, template parameters and constructors are those of the reference
// (src/include/cusync/policies.h; StridedSync from ml-bench/transformer/mlp.cu,
// ConsecutiveSync from ml-bench/transformer/attention.cu).  Here every built-in
// policy is a typed wrapper around a cusync_policy_t record: desc() returns the
// record, and the four methods evaluate it with the shared evaluator, which is
// also what the library's pre-compiled kernels run.
//
// User-written policies with the same four methods work in kernels compiled
// against these headers.  To hand one to a pre-compiled library kernel it must
// also provide `cusync_policy_t desc() const`.
#pragma once

#include <stdint.h>
#include "cusync_defines.h"
#include "policy_eval.h"
#include "tile-orders.h"

namespace cusync {

namespace detail {
// Common body of the built-in policies: evaluate the record.
template <typename Derived>
struct RecordPolicy {
  CUSYNC_DEVICE_HOST uint32_t waitValue(const dim3&, const dim3&) const {
    return eval::waitValue(static_cast<const Derived*>(this)->desc());
  }
  CUSYNC_DEVICE_HOST uint32_t postValue(const dim3&, const dim3&) const {
    return eval::postValue(static_cast<const Derived*>(this)->desc());
  }
  CUSYNC_DEVICE_HOST uint32_t tileIndex(const dim3& tile, const dim3& grid) const {
    return eval::tileIndex(static_cast<const Derived*>(this)->desc(), tile.x, tile.y, grid.x, grid.y);
  }
  CUSYNC_DEVICE_HOST bool isSync(const dim3& tile, const dim3&) const {
    return eval::isSync(static_cast<const Derived*>(this)->desc(), tile.y, tile.z);
  }
};
}  // namespace detail

// No synchronisation: a stage with NoSync input is not a consumer, with NoSync
// output not a producer.
struct NoSync : public detail::RecordPolicy<NoSync> {
  CUSYNC_DEVICE_HOST NoSync() {}
  CUSYNC_DEVICE_HOST cusync_policy_t desc() const {
    return cusync_policy_t{CUSYNC_POLICY_NOSYNC, CUSYNC_ORDER_IDENTITY, 1, 1, 0, 0, 0, 0};
  }
};

// One semaphore per row panel of TileM rows; a consumer tile waits once, at
// its first K step, until all column tiles of the panel have posted.
template <uint32_t TileM>
struct RowSync : public detail::RecordPolicy<RowSync<TileM>> {
  uint32_t waitValue_, postValue_;
  CUSYNC_DEVICE_HOST RowSync() : waitValue_(0), postValue_(0) {}
  CUSYNC_DEVICE_HOST RowSync(uint32_t waitValue) : waitValue_(waitValue), postValue_(1) {}
  CUSYNC_DEVICE_HOST RowSync(uint32_t waitValue, uint32_t postValue) : waitValue_(waitValue), postValue_(postValue) {}
  CUSYNC_DEVICE_HOST cusync_policy_t desc() const {
    return cusync_policy_t{CUSYNC_POLICY_ROWSYNC, CUSYNC_ORDER_TRANSPOSE_XY, TileM, 1, waitValue_, postValue_, 0, 0};
  }
};

// One semaphore per TileM x TileN producer tile; a consumer waits every time
// its K walk enters a new producer tile.
template <typename TileOrder, uint32_t TileM, uint32_t TileN>
struct TileSync : public detail::RecordPolicy<TileSync<TileOrder, TileM, TileN>> {
  static_assert(TileOrder::kOrderKind == CUSYNC_ORDER_IDENTITY || TileOrder::kOrderKind == CUSYNC_ORDER_TRANSPOSE_XY,
                "TileSync numbers its semaphores with IdentityOrder or TransposeXYOrder");
  uint32_t waitValue_, postValue_;
  CUSYNC_DEVICE_HOST TileSync() : waitValue_(1), postValue_(1) {}
  CUSYNC_DEVICE_HOST TileSync(uint32_t waitValue, uint32_t postValue) : waitValue_(waitValue), postValue_(postValue) {}
  CUSYNC_DEVICE_HOST cusync_policy_t desc() const {
    return cusync_policy_t{CUSYNC_POLICY_TILESYNC, TileOrder::kOrderKind, TileM, TileN, waitValue_, postValue_, 0, 0};
  }
};

// Column tiles j and j + GridN/TileN share a semaphore that must reach
// `stride`: the consumer's K tile needs both halves of a [X*W1 | X*V] output.
template <typename TileOrder, uint32_t GridN, uint32_t TileM, uint32_t TileN, uint32_t stride>
struct StridedTileSync : public detail::RecordPolicy<StridedTileSync<TileOrder, GridN, TileM, TileN, stride>> {
  static_assert(TileOrder::kOrderKind == CUSYNC_ORDER_IDENTITY || TileOrder::kOrderKind == CUSYNC_ORDER_TRANSPOSE_XY,
                "StridedTileSync numbers its semaphores with IdentityOrder or TransposeXYOrder");
  CUSYNC_DEVICE_HOST StridedTileSync() {}
  CUSYNC_DEVICE_HOST cusync_policy_t desc() const {
    return cusync_policy_t{CUSYNC_POLICY_STRIDEDTILESYNC, TileOrder::kOrderKind, TileM, TileN, 0, 0, GridN, stride};
  }
};
template <typename TileOrder, uint32_t GridN, uint32_t TileM, uint32_t TileN, uint32_t stride>
using StridedSync = StridedTileSync<TileOrder, GridN, TileM, TileN, stride>;

// The (H/8)/TileN adjacent column tiles of one of Q, K, V share a semaphore.
template <typename TileOrder, uint32_t H, uint32_t TileM, uint32_t TileN>
struct ConsecutiveTileSync : public detail::RecordPolicy<ConsecutiveTileSync<TileOrder, H, TileM, TileN>> {
  static_assert(TileOrder::kOrderKind == CUSYNC_ORDER_IDENTITY || TileOrder::kOrderKind == CUSYNC_ORDER_TRANSPOSE_XY,
                "ConsecutiveTileSync numbers its semaphores with IdentityOrder or TransposeXYOrder");
  CUSYNC_DEVICE_HOST ConsecutiveTileSync() {}
  CUSYNC_DEVICE_HOST cusync_policy_t desc() const {
    return cusync_policy_t{CUSYNC_POLICY_CONSECUTIVETILESYNC, TileOrder::kOrderKind, TileM, TileN, 0, 0, H, 0};
  }
};
template <typename TileOrder, uint32_t H, uint32_t TileM, uint32_t TileN>
using ConsecutiveSync = ConsecutiveTileSync<TileOrder, H, TileM, TileN>;

// Implicit-GEMM convolution with an R x S filter: the consumer's K walk is
// channel-chunk outermost, (r, s) innermost, so K tile y depends on producer
// column tile y / (R*S).
template <typename TileOrder, uint32_t R, uint32_t S, uint32_t TileM, uint32_t TileN>
struct Conv2DTileSync : public detail::RecordPolicy<Conv2DTileSync<TileOrder, R, S, TileM, TileN>> {
  static_assert(TileOrder::kOrderKind == CUSYNC_ORDER_IDENTITY || TileOrder::kOrderKind == CUSYNC_ORDER_TRANSPOSE_XY,
                "Conv2DTileSync numbers its semaphores with IdentityOrder or TransposeXYOrder");
  uint32_t waitValue_, postValue_;
  CUSYNC_DEVICE_HOST Conv2DTileSync() : waitValue_(1), postValue_(1) {}
  CUSYNC_DEVICE_HOST Conv2DTileSync(uint32_t waitValue, uint32_t postValue)
      : waitValue_(waitValue), postValue_(postValue) {}
  CUSYNC_DEVICE_HOST cusync_policy_t desc() const {
    return cusync_policy_t{CUSYNC_POLICY_CONV2DTILESYNC, TileOrder::kOrderKind, TileM, TileN, waitValue_, postValue_,
                           R * S, 0};
  }
};

}  // namespace cusync
