"""Generates tests/golden/policies.json from the REFERENCE's own policy and
tile-order code (oracle/_ref/libcusync_ref_policies.so, built by
`make -C oracle _ref` from the reference headers).  Run in a container that
has the reference tree; the JSON it writes is the committed fixture.

    python tests/golden/make_policy_golden.py
"""
import ctypes as C
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SO = os.path.join(ROOT, "oracle", "_ref", "libcusync_ref_policies.so")

# name -> (kind, order, tile_m, tile_n, p0) in the oracle's vocabulary
POLICIES = {
    "rowsync_128": ("row", 1, 128, 1, 0),
    "rowsync_256": ("row", 1, 256, 1, 0),
    "rowsync_32": ("row", 1, 32, 1, 0),
    "rowsync_1": ("row", 1, 1, 1, 0),
    "tilesync_identity_1_1": ("tile", 0, 1, 1, 0),
    "tilesync_identity_32_32": ("tile", 0, 32, 32, 0),
    "tilesync_identity_128_128": ("tile", 0, 128, 128, 0),
    "tilesync_transpose_128_128": ("tile", 1, 128, 128, 0),
    "tilesync_transpose_128_256": ("tile", 1, 128, 256, 0),
    "tilesync_transpose_256_128": ("tile", 1, 256, 128, 0),
    "conv2dtilesync_transpose_3_3_64_32": ("conv2d", 1, 64, 32, 9),
    "conv2dtilesync_transpose_3_3_128_64": ("conv2d", 1, 128, 64, 9),
    "conv2dtilesync_identity_3_3_64_32": ("conv2d", 0, 64, 32, 9),
}
GRIDS = [(1, 1, 1), (8, 2, 1), (48, 16, 1), (24, 16, 1), (3, 5, 2), (64, 1, 1), (1, 49, 1)]


def main():
    L = C.CDLL(SO)
    out = {"policies": [], "orders": []}
    for name, (kind, order, tm, tn, p0) in POLICIES.items():
        f = getattr(L, "ref_" + name)
        f.argtypes = [C.c_uint32] * 8 + [C.POINTER(C.c_uint32)]
        rows = []
        for grid in GRIDS:
            for wv, pv in ((1, 1), (7, 3)):
                for mi in range(min(grid[1], 3)):
                    for step in (0, 1, 2, 3, 9, 18):
                        for z in (0, 1):
                            # element offsets the GEMM/conv main loops would pass
                            tx = mi * tm + (0 if mi % 2 == 0 else tm // 2)
                            ty = step * max(tn // 2, 1)
                            buf = (C.c_uint32 * 4)()
                            f(wv, pv, tx, ty, z, grid[0], grid[1], grid[2], buf)
                            rows.append([wv, pv, tx, ty, z, *grid, *list(buf)])
        out["policies"].append({"name": name, "kind": kind, "order": order, "tile_m": tm,
                                "tile_n": tn, "p0": p0,
                                "columns": ["wait_ctor", "post_ctor", "tile_x", "tile_y", "tile_z",
                                            "grid_x", "grid_y", "grid_z",
                                            "waitValue", "postValue", "tileIndex", "isSync"],
                                "rows": rows})
    L.ref_block_index.restype = C.c_uint32
    L.ref_block_index.argtypes = [C.c_int] + [C.c_uint32] * 6
    L.ref_order_tile_index.restype = C.c_uint32
    L.ref_order_tile_index.argtypes = [C.c_int] + [C.c_uint32] * 6
    L.ref_tile_to_block.argtypes = [C.c_int] + [C.c_uint32] * 3 + [C.POINTER(C.c_uint32)]
    for order in (0, 1):
        for grid in GRIDS:
            rows = []
            for z in range(grid[2]):
                for y in range(min(grid[1], 5)):
                    for x in range(min(grid[0], 5)):
                        b3 = (C.c_uint32 * 3)()
                        L.ref_tile_to_block(order, x, y, z, b3)
                        rows.append([x, y, z, L.ref_block_index(order, *grid, x, y, z),
                                     L.ref_order_tile_index(order, *grid, x, y, z), *list(b3)])
            out["orders"].append({"order": order, "grid": list(grid),
                                  "columns": ["x", "y", "z", "blockIndex", "tileIndex",
                                              "tileToBlock_x", "tileToBlock_y", "tileToBlock_z"],
                                  "rows": rows})
    with open(os.path.join(HERE, "policies.json"), "w") as fh:
        json.dump(out, fh, separators=(",", ":"))
    print("wrote", sum(len(p["rows"]) for p in out["policies"]), "policy rows,",
          sum(len(o["rows"]) for o in out["orders"]), "order rows")


if __name__ == "__main__":
    main()
