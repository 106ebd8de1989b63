"""CPU tests of the boundary: the C ABI library loads and exports every symbol
include/cusync_b200.h declares; the product's policy evaluator agrees with the
golden vectors taken from the reference's policy code; host-side argument
checks that need no device."""
import ctypes as C
import json
import os
import re

import build_helpers as bh
import oracle_lib as o
from cusync_b200 import _lib as L

ROOT = bh.ROOT
KIND = {"row": L.POLICY_ROWSYNC, "tile": L.POLICY_TILESYNC, "conv2d": L.POLICY_CONV2DTILESYNC}


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "cusync_b200.h")).read()
    return re.findall(r"CUSYNC_API\s+[\w\s\*]+?\b(cusync_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    bh.build_library()
    lib = C.CDLL(L.LIB_PATH)
    names = _declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
    # and the ctypes table covers exactly the declared set
    assert set(names) == set(L.SIGNATURES)


def test_version_string_needs_no_device():
    bh.build_library()
    assert b"sm_100a" in L.lib().cusync_b200_version()


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        L.lib()
        raised = False
    except L.CuSyncLibraryError as e:
        raised = "no fallback" in str(e)
    assert raised


def test_error_enum_values_follow_the_reference():
    # src/include/cusync/cusync.h:46-53: success is the LAST of six enumerators
    assert (L.ERROR_NOT_PRODUCER, L.ERROR_NOT_CONSUMER, L.ERROR_NOT_INITIALIZED,
            L.ERROR_INVALID_LINEAR_BLOCK_INDEX, L.ERROR_CUDA, L.SUCCESS) == (0, 1, 2, 3, 4, 5)
    text = open(os.path.join(ROOT, "include", "cusync_b200.h")).read()
    assert re.search(r"CUSYNC_SUCCESS\s*=\s*5", text)
    for name, val in (("NO_ATOMIC_ADD", 1), ("AVOID_WAIT_KERNEL", 2), ("AVOID_CUSTOM_ORDER", 4),
                      ("REORDER_TILE_LOADS", 8)):
        assert re.search(r"CUSYNC_OPT_%s\s*=\s*%d" % (name, val), text)


def test_product_policy_evaluator_matches_reference_golden():
    so = C.CDLL(bh.build_policy_eval_host())
    so.pe_eval.argtypes = [C.POINTER(L.Policy)] + [C.c_uint32] * 5 + [C.POINTER(C.c_uint32)]
    so.pe_block_index.restype = C.c_uint32
    so.pe_block_index.argtypes = [C.c_uint32] * 5
    so.pe_order_tile_index.restype = C.c_uint32
    so.pe_order_tile_index.argtypes = [C.c_int] + [C.c_uint32] * 4
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "policies.json")))
    n = 0
    for pol in gold["policies"]:
        for wv, pv, tx, ty, tz, gx, gy, gz, e_wait, e_post, e_idx, e_sync in pol["rows"]:
            p = L.Policy(KIND[pol["kind"]], pol["order"], pol["tile_m"], pol["tile_n"], wv, pv, pol["p0"], 0)
            out = (C.c_uint32 * 4)()
            so.pe_eval(C.byref(p), tx, ty, tz, gx, gy, out)
            assert list(out) == [e_wait, e_post, e_idx, e_sync], (pol["name"], tx, ty, tz, gx, gy)
            n += 1
    assert n > 1000
    for rec in gold["orders"]:
        gx, gy, gz = rec["grid"]
        for x, y, z, e_block, e_tile, bx, by, bz in rec["rows"]:
            assert so.pe_block_index(gx, gy, x, y, z) == e_block
            if z == 0:
                assert so.pe_order_tile_index(rec["order"], x, y, gx, gy) == e_tile


def test_product_policy_evaluator_matches_oracle_for_driver_policies():
    # StridedSync (mlp.cu:76-101) and ConsecutiveSync (attention.cu:51-70) have no golden rows (their source
    # cannot be compiled without CUTLASS); the product evaluator and the oracle restatement must agree.
    so = C.CDLL(bh.build_policy_eval_host())
    so.pe_eval.argtypes = [C.POINTER(L.Policy)] + [C.c_uint32] * 5 + [C.POINTER(C.c_uint32)]
    OL = o.lib()
    cases = [(L.POLICY_STRIDEDTILESYNC, o.STRIDEDSYNC, 2816, 2, (44, 4)),
             (L.POLICY_STRIDEDTILESYNC, o.STRIDEDSYNC, 2752 + 64, 2, (44, 3)),
             (L.POLICY_CONSECUTIVETILESYNC, o.CONSECUTIVESYNC, 12288, 0, (36, 2)),
             (L.POLICY_CONSECUTIVETILESYNC, o.CONSECUTIVESYNC, 8192, 0, (24, 5))]
    for kind, okind, p0, p1, (gx, gy) in cases:
        for order in (0, 1):
            p = L.Policy(kind, order, 128, 128, 0, 0, p0, p1)
            op = o.policy(okind, order, 128, 128, 0, 0, p0, p1)
            for m in range(gy):
                for j in range(gx):
                    for z in (0, 1):
                        out = (C.c_uint32 * 4)()
                        so.pe_eval(C.byref(p), m * 128, j * 128 + (64 if z == 0 and j % 3 == 0 else 0), z, gx, gy, out)
                        t = o.Dim3(m * 128, j * 128 + (64 if z == 0 and j % 3 == 0 else 0), z)
                        g = o.Dim3(gx, gy, 1)
                        exp = [OL.orc_policy_wait_value(C.byref(op), t, g), OL.orc_policy_post_value(C.byref(op), t, g),
                               OL.orc_policy_tile_index(C.byref(op), t, g), OL.orc_policy_is_sync(C.byref(op), t, g)]
                        assert list(out) == exp


def test_default_tile_n_table():
    bh.build_library()
    f = L.lib().cusync_gemm_default_tile_n
    assert f(2048, 6144, 12288, L.EPILOGUE_GELU_ERF) == 256
    assert f(64, 6144, 12288, L.EPILOGUE_GELU_ERF) == 256   # wide tiles + split-K for a single row of tiles
    assert f(2048, 2752, 8192, L.EPILOGUE_SILU_MUL_DUAL) == 128
    assert f(256, 1000, 512, L.EPILOGUE_NONE) == 128


def test_plan_create_rejects_bad_arguments_without_a_device():
    bh.build_library()
    plan = C.c_void_p()
    d = L.GemmDesc(0, 16, 16, 16, 16, 16, 16, None, 16, 16, 0, 0, 0, 0, 0, 0, 0, None)
    assert L.lib().cusync_gemm_plan_create(C.byref(plan), C.byref(d)) == L.ERROR_INVALID_ARGUMENT
    d = L.GemmDesc(128, 128, 128, 0x1000, 100, 0x2000, 128, None, 0x3000, 128, 0, 0, 0, 0, 0, 0, 0, None)   # lda % 8 != 0
    assert L.lib().cusync_gemm_plan_create(C.byref(plan), C.byref(d)) == L.ERROR_UNSUPPORTED
    d = L.GemmDesc(128, 128, 128, 0x1008, 128, 0x2000, 128, None, 0x3000, 128, 0, 0, 0, 0, 0, 0, 0, None)   # misaligned A
    assert L.lib().cusync_gemm_plan_create(C.byref(plan), C.byref(d)) == L.ERROR_UNSUPPORTED
    d = L.GemmDesc(128, 128, 128, 0x1000, 128, 0x2000, 128, None, 0x3000, 128, 0, 3, 0, 0, 0, 0, 0, None)   # dual without b2
    assert L.lib().cusync_gemm_plan_create(C.byref(plan), C.byref(d)) == L.ERROR_INVALID_ARGUMENT
    assert L.lib().cusync_stage_link(None, None) == L.ERROR_NOT_INITIALIZED
    assert L.lib().cusync_stage_increment_iter(None) == L.ERROR_NOT_INITIALIZED


def test_grouped_rows_order_is_a_bijection_with_rows_fastest():
    so = C.CDLL(bh.build_policy_eval_host())
    so.pe_grouped_block_index.restype = C.c_uint32
    so.pe_grouped_block_index.argtypes = [C.c_uint32] * 6
    for rows, gx, gy, gz in ((6, 48, 16, 1), (4, 5, 7, 2), (16, 3, 16, 1), (1, 4, 3, 1), (5, 2, 3, 1)):
        seen = {}
        for z in range(gz):
            for y in range(gy):
                for x in range(gx):
                    seen[so.pe_grouped_block_index(rows, gx, gy, x, y, z)] = (x, y, z)
        assert sorted(seen) == list(range(gx * gy * gz))
        # consecutive slots inside a group walk down the rows of one column
        first_group = [seen[i] for i in range(min(rows, gy))]
        assert first_group == [(0, y, 0) for y in range(min(rows, gy))]
        if gx > 1:
            assert seen[min(rows, gy)] == (1, 0, 0)


def test_mlp_config_table_is_total_and_consistent():
    # cusync_mlp_choose_config is a pure host function (the role of the reference's tile_sizes_db.py): every batch
    # from 1 to 4096 of both models gets a row, with a policy the drivers implement, a launch form, tile orders
    # that divide into the row tiles they cover, and tile shapes / K slices the kernels instantiate.
    from cusync_b200 import mlp as M
    from cusync_b200 import _lib as L
    for model in ("gpt3", "llama"):
        prev = None
        changes = 0
        for batch in range(1, 4097):
            c = M.choose_config(model, batch)
            assert c["policy"] in (L.POLICY_ROWSYNC, L.POLICY_TILESYNC)
            assert c["single_grid"] in (1, 2)
            assert c["group_rows1"] >= 1 and c["group_rows2"] >= 1
            assert c["tile_n1"] in (64, 128, 192, 256) and c["tile_n2"] in (64, 128, 192, 256)
            assert 1 <= c["split_k1"] <= 16 and 1 <= c["split_k2"] <= 16
            if c["single_grid"] == 2:      # one grid needs both GEMMs on CTA pairs: more than two row tiles, 256-wide
                # tiles (128-wide output tiles for the fused SwiGLU GEMM, whose pair MMA is [X W1 | X V])
                assert batch > 256 and c["tile_n1"] == (256 if model == "gpt3" else 128) and c["tile_n2"] == 256
            assert c["stream_wait"] == (1 if (batch + 127) // 128 <= 4 else 0)
            # K slices for the first GEMM's last partial round: only in the one-grid form, and only at seven and eight
            # row tiles of the GPT-3 shard (96 pair tiles: one round of 74 and a tail of 22, 66 units in three slices)
            assert c["tail_split1"] == (3 if (model == "gpt3" and 768 < batch <= 1024) else 0)
            assert c["tail_split1"] == 0 or c["single_grid"] == 2
            key = (c["policy"], c["single_grid"], c["group_rows1"], c["group_rows2"])
            if prev is not None and key != prev:
                changes += 1
            prev = key
        assert changes <= 4          # a handful of batch ranges, not a row per batch
    bad = L.MlpChoice()
    assert L.lib().cusync_mlp_choose_config(7, 64, 12288, 6144, C.byref(bad)) == L.ERROR_INVALID_ARGUMENT
    assert L.lib().cusync_mlp_choose_config(0, 0, 12288, 6144, C.byref(bad)) == L.ERROR_INVALID_ARGUMENT
