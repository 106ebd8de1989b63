"""CPU tests of the oracle: pinned against the reference's own policy code
(committed golden vectors, and the live reference build when it is present)
and against the known answers of the reference's tests."""
import ctypes as C
import json
import math
import os

import numpy as np
import pytest

import oracle_lib as o

HERE = os.path.dirname(os.path.abspath(__file__))
KIND = {"row": o.ROWSYNC, "tile": o.TILESYNC, "conv2d": o.CONV2DTILESYNC}


def _golden():
    with open(os.path.join(HERE, "golden", "policies.json")) as fh:
        return json.load(fh)


def test_policies_match_reference_golden():
    L = o.lib()
    n = 0
    for pol in _golden()["policies"]:
        for wv, pv, tx, ty, tz, gx, gy, gz, e_wait, e_post, e_idx, e_sync in pol["rows"]:
            p = o.policy(KIND[pol["kind"]], pol["order"], pol["tile_m"], pol["tile_n"], wv, pv, pol["p0"])
            t, g = o.Dim3(tx, ty, tz), o.Dim3(gx, gy, gz)
            assert L.orc_policy_wait_value(C.byref(p), t, g) == e_wait
            assert L.orc_policy_post_value(C.byref(p), t, g) == e_post
            assert L.orc_policy_tile_index(C.byref(p), t, g) == e_idx, (pol["name"], tx, ty, tz, gx, gy, gz)
            assert bool(L.orc_policy_is_sync(C.byref(p), t, g)) == bool(e_sync)
            n += 1
    assert n > 1000


def test_tile_orders_match_reference_golden():
    L = o.lib()
    for rec in _golden()["orders"]:
        g = o.Dim3(*rec["grid"])
        for x, y, z, e_block, e_tile, bx, by, bz in rec["rows"]:
            t = o.Dim3(x, y, z)
            assert L.orc_block_index(rec["order"], g, t) == e_block
            assert L.orc_order_tile_index(rec["order"], t, g) == e_tile
            assert L.orc_tile_to_block(rec["order"], t).tup() == (bx, by, bz)


@pytest.mark.skipif(not os.path.exists(o.REF_POLICIES_SO), reason="reference build absent")
def test_golden_is_what_the_reference_build_gives_now():
    """The committed fixture is regenerated from the live reference build and compared."""
    import subprocess, sys, tempfile, shutil
    gold = os.path.join(HERE, "golden", "policies.json")
    before = open(gold).read()
    with tempfile.TemporaryDirectory() as td:
        shutil.copy(gold, os.path.join(td, "keep.json"))
        subprocess.check_call([sys.executable, os.path.join(HERE, "golden", "make_policy_golden.py")],
                              stdout=subprocess.DEVNULL)
        after = open(gold).read()
        shutil.copy(os.path.join(td, "keep.json"), gold)
    assert before == after


def test_schedule_buffer_is_row_major_over_the_launch_grid():
    # cusync.h:138-147 with either order: slot i holds block (i % gx, (i / gx) % gy, i / (gx*gy))
    for order in (o.ORDER_IDENTITY, o.ORDER_TRANSPOSE_XY):
        for grid in ((8, 2, 1), (3, 5, 2), (1, 1, 1), (48, 16, 1)):
            got, bad = o.tile_order(order, grid)
            assert bad == 0
            i = np.arange(len(got))
            assert (got[:, 0] == i % grid[0]).all()
            assert (got[:, 1] == (i // grid[0]) % grid[1]).all()
            assert (got[:, 2] == i // (grid[0] * grid[1])).all()


def test_simple_test_known_answer_all_semaphores_equal_iter():
    # tests/simple-test.cu:59-66,96 + tests/cusync-test.h:19-27: TileSync<IdentityOrder,1,1> on a 1-D
    # grid of 8192 blocks; after `iters` runs every semaphore equals expectedWaitValue * iter = iter.
    grid = (8192, 1, 1)
    pol = o.policy(o.TILESYNC, o.ORDER_IDENTITY, 1, 1, 1, 1)
    for opts in (0, o.OPT_NO_ATOMIC_ADD):
        for iters in (1, 2):
            # the copy kernel's tile is the block itself: {x, 0, 0}; expressed in GEMM coordinates that
            # is grid (1, 8192) with tile_m = 1, i.e. row offset = block index
            pol_rows = o.policy(o.TILESYNC, o.ORDER_TRANSPOSE_XY, 1, 1, 1, 1)
            sems, oob = o.producer_semaphores(pol_rows, (1, 8192, 1), 1, 1, opts, iters)
            assert oob == 0 and (sems == iters).all()
    L = o.lib()
    for x in (0, 1, 4097, 8191):
        assert L.orc_policy_tile_index(C.byref(pol), o.Dim3(x, 0, 0), o.Dim3(*grid)) == x
        assert L.orc_policy_is_sync(C.byref(pol), o.Dim3(x, 0, 0), o.Dim3(*grid)) == 1


def test_two_matmuls_known_answer():
    # src/examples/twoMatMuls/matrixMul.cu:149-152,235-272: A = 1, B = D = 0.01, 256^3 fp32:
    # every C element is 2.56, every E element 6.5536, within 1e-5 * dot length relative.
    n = 256
    a = np.ones((n, n), np.float32); b = np.full((n, n), 0.01, np.float32)
    c = o.gemm_f32(a, b)
    e = o.gemm_f32(c, b)
    assert np.abs(c - 2.56).max() / 2.56 / n < 1e-5
    assert np.abs(e - 6.5536).max() / 6.5536 / n < 1e-5


def test_two_matmuls_semaphores_and_waits():
    # matrixMul.cu:36-39,91-92,120: TileSync<IdentityOrder,32,32>, grid 8x8; consumer waits
    # {k, by*32, 1} for k = 0,32,..; producer posts {bx*32, by*32, 0}.  With IdentityOrder the wait on
    # (x = k, y = by*32) resolves to semaphore k/32 + by*8, the tile the producer posted as (bx = k/32, by).
    L = o.lib()
    pol = o.policy(o.TILESYNC, o.ORDER_IDENTITY, 32, 32, 1, 1)
    grid = o.Dim3(8, 8, 1)
    posted = set()
    for by in range(8):
        for bx in range(8):
            posted.add(L.orc_policy_tile_index(C.byref(pol), o.Dim3(bx * 32, by * 32, 0), grid))
    assert posted == set(range(64))
    for by in range(8):
        for k in range(0, 256, 32):
            t = o.Dim3(k, by * 32, 1)
            assert L.orc_policy_is_sync(C.byref(pol), t, grid) == 1
            assert L.orc_policy_tile_index(C.byref(pol), t, grid) == k // 32 + by * 8


def test_gemm_chain_semaphores_rowsync_and_tilesync():
    # GPT-3 shard at B=2048 with 128x128 tiles: GEMM1 grid (48, 16, 1) (mlp.cu:1026-1039)
    grid = (48, 16, 1)
    row = o.policy(o.ROWSYNC, o.ORDER_TRANSPOSE_XY, 128, 128, 48, 1)
    sems, oob = o.producer_semaphores(row, grid, 128, 128, 0, 3)
    assert oob == 0 and (sems[:16] == 3 * 48).all() and (sems[16:] == 0).all()
    idx, exp = o.consumer_tile_waits(row, grid, 5 * 128, 6144, 64, 3)
    assert list(idx) == [5] and list(exp) == [3 * 48]
    tile = o.policy(o.TILESYNC, o.ORDER_TRANSPOSE_XY, 128, 128, 1, 1)
    sems, oob = o.producer_semaphores(tile, grid, 128, 128, o.OPT_NO_ATOMIC_ADD, 2)
    assert oob == 0 and (sems == 2).all()
    idx, exp = o.consumer_tile_waits(tile, grid, 5 * 128, 6144, 64, 2)
    assert list(idx) == [n + 5 * 48 for n in range(48)] and (exp == 2).all()


def test_strided_and_consecutive_sync_follow_their_call_sites():
    L = o.lib()
    # mlp.cu:107-108: StridedSync<TransposeXYOrder, 2816, TM, TN, 2>: N-tiles j and j + 2816/TN share a
    # semaphore; wait value 2, post 1.
    p = o.policy(o.STRIDEDSYNC, o.ORDER_TRANSPOSE_XY, 128, 128, 0, 0, p0=2816, p1=2)
    grid = o.Dim3(44, 4, 1)
    for m in range(4):
        for j in range(22):
            a = L.orc_policy_tile_index(C.byref(p), o.Dim3(m * 128, j * 128, 0), grid)
            b = L.orc_policy_tile_index(C.byref(p), o.Dim3(m * 128, (j + 22) * 128, 0), grid)
            assert a == b == j + m * 44
    assert L.orc_policy_wait_value(C.byref(p), o.Dim3(0, 0, 0), grid) == 2
    assert L.orc_policy_post_value(C.byref(p), o.Dim3(0, 0, 0), grid) == 1
    sems, oob = o.producer_semaphores(p, (44, 4, 1), 128, 128, 0, 1)
    assert oob == 0
    s = sems.reshape(4, 44)
    assert (s[:, :22] == 2).all() and (s[:, 22:] == 0).all()
    # attention.cu:105-110: ConsecutiveSync<TransposeXYOrder, 12288, TM, TN=128>: the 12 N-tiles of one
    # of Q, K, V (1536 columns) share a semaphore that reaches 12.
    c = o.policy(o.CONSECUTIVESYNC, o.ORDER_TRANSPOSE_XY, 128, 128, 0, 0, p0=12288)
    grid = o.Dim3(36, 2, 1)
    assert L.orc_policy_wait_value(C.byref(c), o.Dim3(0, 0, 1), grid) == 12
    for m in range(2):
        for j in range(36):
            assert L.orc_policy_tile_index(C.byref(c), o.Dim3(m * 128, j * 128, 0), grid) == j // 12 + m * 3
    assert L.orc_policy_is_sync(C.byref(c), o.Dim3(0, 0, 1), grid) == 1
    assert L.orc_policy_is_sync(C.byref(c), o.Dim3(0, 0, 0), grid) == 0


def test_gemm_f16_against_numpy_float64():
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (70, 200)).astype(np.float16)
    b = rng.uniform(-1, 1, (200, 333)).astype(np.float16)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    got = o.gemm_f16(a, b).astype(np.float64)
    assert np.abs(got - ref).max() <= 2e-3 * np.abs(ref).max()
    g = o.gemm_f16(a, b, o.EPI_GELU_ERF).astype(np.float64)
    erf = np.vectorize(math.erf)
    gref = 0.5 * ref * (1 + erf(ref / math.sqrt(2)))
    assert np.abs(g - gref).max() <= 2e-3 * np.abs(gref).max()
    r = o.gemm_f16(a, b, o.EPI_RELU).astype(np.float64)
    assert np.abs(r - np.maximum(ref, 0)).max() <= 2e-3 * np.abs(ref).max()


def test_gemm_f16_accumulates_in_k_order_like_ref_cpumatmul():
    # common.h:89-102: accum += float(a)*float(b) for k = 0..K-1, then one cast to half.
    rng = np.random.default_rng(2)
    a = rng.uniform(-1, 1, (3, 97)).astype(np.float16)
    b = rng.uniform(-1, 1, (97, 5)).astype(np.float16)
    exp = np.empty((3, 5), np.float16)
    for i in range(3):
        for j in range(5):
            acc = np.float32(0)
            for k in range(97):
                acc = np.float32(acc + np.float32(a[i, k]) * np.float32(b[k, j]))
            exp[i, j] = np.float16(acc)
    assert (o.gemm_f16(a, b).view(np.uint16) == exp.view(np.uint16)).all()


def test_dual_silu_mul():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((9, 64)).astype(np.float16)
    b1 = (rng.standard_normal((64, 40)) * 0.2).astype(np.float16)
    b2 = (rng.standard_normal((64, 40)) * 0.2).astype(np.float16)
    x = a.astype(np.float64) @ b1.astype(np.float64)
    y = a.astype(np.float64) @ b2.astype(np.float64)
    ref = x / (1 + np.exp(-x)) * y
    got = o.gemm_dual_silu_mul_f16(a, b1, b2).astype(np.float64)
    assert np.abs(got - ref).max() <= 3e-3 * np.abs(ref).max()


def test_conv3x3_against_direct_numpy():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 6, 5, 8)).astype(np.float16)
    w = (rng.standard_normal((4, 3, 3, 8)) * 0.1).astype(np.float16)
    xp = np.zeros((2, 8, 7, 8), np.float64); xp[:, 1:-1, 1:-1] = x
    ref = np.zeros((2, 6, 5, 4))
    for r in range(3):
        for s in range(3):
            ref += np.einsum("nhwc,kc->nhwk", xp[:, r:r + 6, s:s + 5], w[:, r, s].astype(np.float64))
    got = o.conv2d_3x3_nhwc_f16(x, w, relu=False).astype(np.float64)
    assert np.abs(got - ref).max() <= 3e-3 * np.abs(ref).max()
    got = o.conv2d_3x3_nhwc_f16(x, w, relu=True).astype(np.float64)
    assert np.abs(got - np.maximum(ref, 0)).max() <= 3e-3 * np.abs(ref).max()


def test_attention_decode_against_numpy():
    rng = np.random.default_rng(5)
    B, S, Hh, d = 2, 37, 3, 16
    q = rng.standard_normal((B, Hh, d)).astype(np.float16)
    k = rng.standard_normal((B, S, Hh, d)).astype(np.float16)
    v = rng.standard_normal((B, S, Hh, d)).astype(np.float16)
    s = np.einsum("bhd,bshd->bhs", q.astype(np.float64), k.astype(np.float64)) / math.sqrt(d)
    p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
    ref = np.einsum("bhs,bshd->bhd", p, v.astype(np.float64))
    got = o.attention_decode_f16(q, k, v).astype(np.float64)
    assert np.abs(got - ref).max() <= 3e-3 * np.abs(ref).max()


def test_max_rel_err_floor():
    ref = np.array([1.0, 0.001, -2.0], np.float16)
    got = np.array([1.0, 0.003, -2.0], np.float16)
    # 0.001 is under the floor 1e-2 * 2.0 = 0.02, so its error is 0.002 / 0.02 = 0.1
    assert abs(o.max_rel_err(got, ref, 1e-2) - 0.1) < 2e-2
    assert o.max_rel_err(ref, ref) == 0.0
