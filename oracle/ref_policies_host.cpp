// Host-callable view of the REFERENCE's own sync policies and tile orders.
// TEST INFRASTRUCTURE ONLY.  This file contains no policy logic: it includes
// the reference's headers where they lie (-I<reference>/src/include, never
// copied into this repository), turns their __device__ qualifiers into
// nothing so g++ can compile them for the CPU, and exposes each function
// through a C symbol.  Built by `make _ref` into oracle/_ref/; used to pin the
// C restatement in cusync_oracle.c and to generate tests/golden/policies.json.
#include <stdint.h>

struct dim3 {
  unsigned int x, y, z;
  dim3(unsigned int x_ = 1, unsigned int y_ = 1, unsigned int z_ = 1) : x(x_), y(y_), z(z_) {}
};

// The reference guards its policy bodies with `#if defined(__CUDACC__)`.
#define __CUDACC__ 1
#define __device__
#define __host__
#define __forceinline__ inline
#include "cusync/cusync_defines.h"
#include "cusync/tile-orders.h"
#include "cusync/policies.h"
#undef __CUDACC__

using namespace cusync;

// Policies that live in the reference's benchmark drivers rather than in its
// headers are exercised through small fixed instantiations below; their
// source (mlp.cu:76-101, attention.cu:51-70) cannot be included because the
// drivers pull in CUTLASS, which is absent.  They are restated in
// cusync_oracle.c and checked against the reference's call sites by the tests.

template <class Order> static uint32_t order_block_index(dim3 g, dim3 b) { return Order().blockIndex(g, b); }
template <class Order> static uint32_t order_tile_index(dim3 t, dim3 g) { return Order().tileIndex(t, g); }

// One instantiation per (policy, order, TileM, TileN[, R*S]) the tests use.
#define DEFINE_POLICY(NAME, TYPE, CTOR)                                                     \
  extern "C" void ref_##NAME(uint32_t wv, uint32_t pv, uint32_t tx, uint32_t ty, uint32_t tz,\
                             uint32_t gx, uint32_t gy, uint32_t gz, uint32_t* out4) {       \
    (void)wv; (void)pv;                                                                      \
    TYPE p CTOR;                                                                             \
    dim3 t(tx, ty, tz), g(gx, gy, gz);                                                       \
    out4[0] = p.waitValue(t, g); out4[1] = p.postValue(t, g);                                \
    out4[2] = p.tileIndex(t, g); out4[3] = p.isSync(t, g) ? 1u : 0u;                         \
  }

typedef RowSync<128> Row128;  typedef RowSync<1> Row1;  typedef RowSync<32> Row32;  typedef RowSync<256> Row256;
DEFINE_POLICY(rowsync_128, Row128, (wv, pv))
DEFINE_POLICY(rowsync_256, Row256, (wv, pv))
DEFINE_POLICY(rowsync_32, Row32, (wv, pv))
DEFINE_POLICY(rowsync_1, Row1, (wv, pv))
typedef TileSync<IdentityOrder, 1, 1> TileI_1_1;
typedef TileSync<IdentityOrder, 32, 32> TileI_32_32;
typedef TileSync<TransposeXYOrder, 128, 128> TileT_128_128;
typedef TileSync<TransposeXYOrder, 128, 256> TileT_128_256;
typedef TileSync<TransposeXYOrder, 256, 128> TileT_256_128;
typedef TileSync<IdentityOrder, 128, 128> TileI_128_128;
DEFINE_POLICY(tilesync_identity_1_1, TileI_1_1, (wv, pv))
DEFINE_POLICY(tilesync_identity_32_32, TileI_32_32, (wv, pv))
DEFINE_POLICY(tilesync_identity_128_128, TileI_128_128, (wv, pv))
DEFINE_POLICY(tilesync_transpose_128_128, TileT_128_128, (wv, pv))
DEFINE_POLICY(tilesync_transpose_128_256, TileT_128_256, (wv, pv))
DEFINE_POLICY(tilesync_transpose_256_128, TileT_256_128, (wv, pv))
typedef Conv2DTileSync<TransposeXYOrder, 3, 3, 64, 32> ConvT_3_3_64_32;
typedef Conv2DTileSync<TransposeXYOrder, 3, 3, 128, 64> ConvT_3_3_128_64;
typedef Conv2DTileSync<IdentityOrder, 3, 3, 64, 32> ConvI_3_3_64_32;
DEFINE_POLICY(conv2dtilesync_transpose_3_3_64_32, ConvT_3_3_64_32, (wv, pv))
DEFINE_POLICY(conv2dtilesync_transpose_3_3_128_64, ConvT_3_3_128_64, (wv, pv))
DEFINE_POLICY(conv2dtilesync_identity_3_3_64_32, ConvI_3_3_64_32, (wv, pv))

extern "C" uint32_t ref_block_index(int order, uint32_t gx, uint32_t gy, uint32_t gz,
                                    uint32_t bx, uint32_t by, uint32_t bz) {
  dim3 g(gx, gy, gz), b(bx, by, bz);
  return order ? order_block_index<TransposeXYOrder>(g, b) : order_block_index<IdentityOrder>(g, b);
}
extern "C" uint32_t ref_order_tile_index(int order, uint32_t gx, uint32_t gy, uint32_t gz,
                                         uint32_t tx, uint32_t ty, uint32_t tz) {
  dim3 g(gx, gy, gz), t(tx, ty, tz);
  return order ? order_tile_index<TransposeXYOrder>(t, g) : order_tile_index<IdentityOrder>(t, g);
}
extern "C" void ref_tile_to_block(int order, uint32_t tx, uint32_t ty, uint32_t tz, uint32_t* out3) {
  dim3 t(tx, ty, tz);
  dim3 b = order ? TransposeXYOrder().tileToBlock(t) : IdentityOrder().tileToBlock(t);
  out3[0] = b.x; out3[1] = b.y; out3[2] = b.z;
}
