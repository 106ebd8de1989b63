"""GPU tests of the C++ template API (<cusync/cusync.h>, <cusync/gemm.h>):
the reference's own tests restated (tests/simple-test.cu, the twoMatMuls
example) plus a GEMM chain through the Gemm handle, user-written policy /
tile order, and a bounded-wait timeout.  The C++ side is tests/cpp/api_tests.cu."""
import ctypes as C

import numpy as np
import pytest

import build_helpers as bh
import oracle_lib as o
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    so = C.CDLL(bh.build_api_tests())
    so.api_simple_test.argtypes = [C.c_int, C.c_int, C.c_int]
    so.api_two_matmuls.argtypes = [C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_int]
    so.api_gemm_chain.argtypes = [C.c_int] * 4 + [C.c_void_p] * 5 + [C.c_int, C.c_void_p]
    so.api_conv_chain.argtypes = [C.c_int] * 3 + [C.c_void_p] * 5 + [C.c_int, C.c_void_p]
    so.api_custom_policy_and_order.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
    so.api_wait_times_out.argtypes = [C.POINTER(L.Status), C.POINTER(C.c_float)]
    return so


def test_error_and_optimization_enums(api):
    assert api.api_error_codes() == 0


# tests/simple-test.cu:107-138: SimpleTest_TileSync.NoOpts, _MultiIters.NoOpts, .NoAtomicAdd, .AvoidCustomOrder
@pytest.mark.parametrize("variant,iters", [(0, 1), (0, 2), (1, 1), (2, 1), (1, 3)])
def test_simple_test_cases(api, variant, iters):
    assert api.api_simple_test(variant, iters, 20) == 0


def test_two_matmuls_known_answers(api):
    # matrixMul.cu:149-152,235-272: A = 1, B = D = 0.01, 256^3 -> C = 2.56, E = 6.5536
    n = 256
    c = np.zeros((n, n), np.float32); e = np.zeros((n, n), np.float32)
    assert api.api_two_matmuls(n, 1.0, 0.01, c.ctypes.data_as(C.c_void_p), e.ctypes.data_as(C.c_void_p), 2) == 0
    assert np.abs(c - 2.56).max() / 2.56 / n < 1e-5
    assert np.abs(e - 6.5536).max() / 6.5536 / n < 1e-5
    # and bit-for-bit what the oracle's fp32 chain gives (same k-order accumulation)
    a = np.ones((n, n), np.float32); b = np.full((n, n), 0.01, np.float32)
    cref = o.gemm_f32(a, b)
    assert np.abs(c - cref).max() <= 1e-6


@pytest.mark.parametrize("policy", [0, 1])
def test_gemm_chain_through_the_cpp_handle(api, policy):
    M, N, K = 256, 1024, 1024
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float16)
    d = rng.uniform(-1, 1, (N, N)).astype(np.float16)
    c = np.zeros((M, N), np.float16); e = np.zeros((M, N), np.float16)
    sems = np.zeros(16, np.uint32)
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    iters = 3
    assert api.api_gemm_chain(policy, M, N, K, p(a), p(b), p(d), p(c), p(e), iters, p(sems)) == 0
    cref = o.gemm_f16(a, b)
    eref = o.gemm_f16(cref, d)
    assert o.max_rel_err(c, cref) <= 1e-2
    assert o.max_rel_err(e, eref) <= 1e-2
    if policy == 0:   # RowSync: 2 row panels, 8 column tiles each
        assert list(sems[:2]) == [8 * iters] * 2 and (sems[2:] == 0).all()
    else:             # TileSync + NoAtomicAdd: every semaphore holds postValue * iter
        assert (sems == iters).all()


def test_conv_chain_through_the_cpp_handle(api):
    # resnet.cu's call pattern on <cusync/conv.h>: Conv2dFprop<CuStage<..., TileSync>> -> Conv2dFprop<CuStage<Conv2DTileSync, ...>>
    N, H, W, Cc = 2, 56, 56, 64
    rng = np.random.default_rng(1)
    x = rng.standard_normal((N, H, W, Cc)).astype(np.float16)
    f1 = (rng.standard_normal((Cc, 3, 3, Cc)) * (2.0 / 576) ** 0.5).astype(np.float16)
    f2 = (rng.standard_normal((Cc, 3, 3, Cc)) * (2.0 / 576) ** 0.5).astype(np.float16)
    y1 = np.zeros_like(x); y2 = np.zeros_like(x)
    tiles = N * H // 2
    sems = np.zeros(tiles, np.uint32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    iters = 2
    assert api.api_conv_chain(N, H, W, p(x), p(f1), p(f2), p(y1), p(y2), iters, p(sems)) == 0
    r1 = o.conv2d_3x3_nhwc_f16(x, f1, True)
    assert o.max_rel_err(y1, r1) <= 1e-2
    assert o.max_rel_err(y2, o.conv2d_3x3_nhwc_f16(y1, f2, True)) <= 1e-2
    assert (sems == iters).all()


def test_user_written_policy_and_tile_order(api):
    blocks = 64
    order = np.zeros(blocks, np.uint32); sems = np.zeros(blocks, np.uint32)
    assert api.api_custom_policy_and_order(blocks, order.ctypes.data_as(C.c_void_p),
                                           sems.ctypes.data_as(C.c_void_p)) == 0
    assert (order == np.arange(blocks)[::-1]).all()          # slot i holds block grid-1-i
    assert (sems[:blocks // 2] == 2).all() and (sems[blocks // 2:] == 0).all()


def test_invalid_tile_order_is_reported(api):
    assert api.api_broken_order_status() == L.ERROR_INVALID_LINEAR_BLOCK_INDEX


def test_wait_runs_out_and_reports(api):
    st = L.Status(); ms = C.c_float()
    assert api.api_wait_times_out(C.byref(st), C.byref(ms)) == 0
    assert st.code == L.ERROR_TIMEOUT and st.where == 1 and st.expected == 1 and st.seen == 0
    assert 15.0 <= ms.value < 2000.0
