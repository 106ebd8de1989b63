"""Runs the REFERENCE's own L1 (CuStage wait/post/tile, wait kernel), compiled
for sm_100a from the reference tree into oracle/_ref/ref_l1_driver, and compares
what it produced -- schedule buffer, semaphores after k runs, the (index,
expected) pair of every consumer wait -- bit-exactly with the oracle and with
this library's stages."""
import json
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as o
import cusync_b200 as cs
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CASES = {
    # name: (oracle policy kind, order, tile_m, tile_n, wait ctor, opts)
    "tilesync_identity_1_1": (o.TILESYNC, 0, 1, 1, 1, 0),
    "tilesync_identity_1_1_noatomic": (o.TILESYNC, 0, 1, 1, 1, o.OPT_NO_ATOMIC_ADD),
    "tilesync_identity_1_1_nocustomorder": (o.TILESYNC, 0, 1, 1, 1, 0),
    "rowsync_128": (o.ROWSYNC, 1, 128, 128, 8, 0),
    "rowsync_128_wide": (o.ROWSYNC, 1, 128, 256, 6, 0),
    "tilesync_transpose_128_128": (o.TILESYNC, 1, 128, 128, 1, 0),
    "tilesync_transpose_128_128_noatomic": (o.TILESYNC, 1, 128, 128, 1, o.OPT_NO_ATOMIC_ADD),
    "tilesync_transpose_128_256": (o.TILESYNC, 1, 128, 256, 1, 0),
}


@pytest.fixture(scope="module")
def reference_records():
    if not os.path.exists(o.REF_L1_DRIVER):
        pytest.skip("reference L1 build absent (built where the reference tree is present)")
    out = subprocess.run([o.REF_L1_DRIVER], capture_output=True, timeout=120)
    assert out.returncode == 0, out.stderr.decode()[-500:]
    recs = [json.loads(line) for line in out.stdout.decode().splitlines() if line.startswith("{")]
    assert len(recs) >= 17
    return recs


def test_reference_tile_order_and_semaphores_match_oracle_and_library(reference_records):
    import ctypes as C
    OL = o.lib()
    for r in reference_records:
        kind, order, tm, tn, wv, opts = CASES[r["case"]]
        grid_p, grid_c, it = tuple(r["grid_p"]), tuple(r["grid_c"]), r["iter"]
        pol = o.policy(kind, order, tm, tn, wv, 1)
        # schedule buffer
        exp_order, bad = o.tile_order(order, grid_p)
        assert bad == 0
        assert (np.array(r["tile_order"], dtype=np.uint32) == exp_order).all(), r["case"]
        # semaphores after `it` runs
        if r["gemm_shaped"]:
            exp, oob = o.producer_semaphores(pol, grid_p, tm, tn, opts, it)
        else:  # copy-kernel protocol: tile {x,0,0} posted as is -> semaphore x
            exp = np.full(grid_p[0], it, dtype=np.uint32); oob = 0
        assert oob == 0
        assert (np.array(r["sems"], dtype=np.uint32) == exp).all(), (r["case"], it)
        # consumer waits
        waits = {}
        for t, w, idx, expect, seen in r["waits"]:
            if idx != 0xFFFFFFFF:
                waits.setdefault(t, []).append((w, idx, expect, seen))
        for t in range(grid_c[0] * grid_c[1]):
            if r["gemm_shaped"]:
                row = (t // grid_c[0]) * tm
                oi, oe = o.consumer_tile_waits(pol, grid_p, row, grid_p[0] * tn, r["bk"], it)
                # the driver records every K step; keep the steps where the policy synchronises
                got = []
                for (w, idx, expect, seen) in sorted(waits.get(t, [])):
                    tile = o.Dim3(row, w * r["bk"], 1 if w == 0 else 0)
                    if OL.orc_policy_is_sync(C.byref(pol), tile, o.Dim3(*grid_p)):
                        got.append((idx, expect * it))
                        assert seen >= expect * it
                assert got == list(zip(oi.tolist(), oe.tolist())), (r["case"], t)
            else:
                (w, idx, expect, seen), = waits[t]
                assert idx == t and expect == 1 and seen == it
        # this library's stage builds the same schedule buffer
        mine = cs.CuStage(order, grid_p, (1, 1, 1), cs.NoSync(), cs.TileSync(order, max(tm, 1), max(tn, 1)))
        assert (mine.tile_order() == exp_order).all()
        mine.destroy()
