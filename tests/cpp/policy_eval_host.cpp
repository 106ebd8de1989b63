// Host build of the PRODUCT's policy evaluator (include/cusync/policy_eval.h),
// so CPU tests can compare it with the golden vectors taken from the reference.
#include <stdint.h>
#include <cusync/policy_eval.h>

#define API extern "C" __attribute__((visibility("default")))

API void pe_eval(const cusync_policy_t* p, uint32_t tx, uint32_t ty, uint32_t tz, uint32_t gx, uint32_t gy,
                 uint32_t* out4) {
  out4[0] = cusync::eval::waitValue(*p);
  out4[1] = cusync::eval::postValue(*p);
  out4[2] = cusync::eval::tileIndex(*p, tx, ty, gx, gy);
  out4[3] = cusync::eval::isSync(*p, ty, tz) ? 1u : 0u;
}
API uint32_t pe_block_index(uint32_t gx, uint32_t gy, uint32_t bx, uint32_t by, uint32_t bz) {
  return cusync::eval::blockIndex(gx, gy, bx, by, bz);
}
API uint32_t pe_order_tile_index(int order, uint32_t tx, uint32_t ty, uint32_t gx, uint32_t gy) {
  return cusync::eval::orderTileIndex(order, tx, ty, gx, gy);
}
API uint32_t pe_grouped_block_index(uint32_t rows, uint32_t gx, uint32_t gy, uint32_t bx, uint32_t by, uint32_t bz) {
  return cusync::eval::groupedBlockIndex(rows, gx, gy, bx, by, bz);
}
