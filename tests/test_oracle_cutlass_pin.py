"""Pins the ARITHMETIC side of the CPU oracle to NVIDIA CUTLASS's host reference kernels, the code the
reference's own drivers check their GPU kernels against (cutlass::reference::host::Conv2dFprop at
src/ml-bench/volta_conv2d/resnet.cu:706-720; the CUTLASS host GEMM for the GEMM chains, whose arithmetic
referenceMLP restates, src/ml-bench/transformer/mlp.cu:333-379) and to CUTLASS's activation functors (GELU as
LinearCombinationGELU applies it, mlp.cu:140-163; SiLu; ReLu).

CUTLASS is an external dependency of the reference (an empty, un-pinned submodule in its tree): oracle/Makefile
target `_cutlass` compiles oracle/cutlass_host_ref.cpp against whatever CUTLASS header tree it finds and writes
oracle/_ref/libcutlass_host_ref.so.  Without such a tree these tests skip, saying so.

Measured agreement on this image (CUTLASS 4.5 headers): GEMM and GELU / ReLU bit-exact, the convolution
bit-exact, SiLU * mul within one half-precision ulp (CUTLASS divides 1 by 1 + exp(-x) and multiplies, the
oracle divides x by it).
"""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as o

SO = os.path.join(o.ORACLE_DIR, "_ref", "libcutlass_host_ref.so")


def _cutlass():
    src = os.path.join(o.ORACLE_DIR, "cutlass_host_ref.cpp")
    if not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(src):
        r = subprocess.run(["make", "-C", o.ORACLE_DIR, "_cutlass"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if r.returncode != 0 and not os.path.exists(SO):
            pytest.skip("no CUTLASS header tree to build the host reference from (make -C oracle _cutlass failed)")
    L = C.CDLL(SO)
    i, vp = C.c_int, C.c_void_p
    L.cutlass_ref_gemm_f16.restype = None
    L.cutlass_ref_gemm_f16.argtypes = [i, i, i, vp, i, vp, i, vp, i]
    L.cutlass_ref_conv2d_fprop_f16.restype = None
    L.cutlass_ref_conv2d_fprop_f16.argtypes = [i] * 8 + [vp, vp, vp]
    L.cutlass_ref_activation_f32.restype = None
    L.cutlass_ref_activation_f32.argtypes = [i, C.c_longlong, vp, vp]
    return L


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def cutlass_gemm(a, b):
    L = _cutlass()
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    m, k = a.shape; _, n = b.shape
    c = np.zeros((m, n), np.float16)       # beta = 0 still multiplies C: it must hold finite values
    L.cutlass_ref_gemm_f16(m, n, k, _p(a), k, _p(b), n, _p(c), n)
    return c


def cutlass_conv(x, w):
    L = _cutlass()
    x = np.ascontiguousarray(x); w = np.ascontiguousarray(w)
    n, h, wd, c = x.shape; k = w.shape[0]
    y = np.zeros((n, h, wd, k), np.float16)
    L.cutlass_ref_conv2d_fprop_f16(n, h, wd, c, k, 3, 3, 1, _p(x), _p(w), _p(y))
    return y


def cutlass_act(kind, x):
    L = _cutlass()
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    L.cutlass_ref_activation_f32(kind, x.size, _p(x), _p(y))
    return y


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def ulp_distance(a, b):
    """Distance in units of the last place between two float16 arrays (sign-magnitude to ordered integers)."""
    def ordered(x):
        u = bits(x).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    return np.abs(ordered(a) - ordered(b))


def test_gemm_config1_shape_is_bit_exact_with_cutlass_host_gemm():
    # BASELINE config 1: M = 256, K = N = 1024, operands uniform[-1, 1], seeded.
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (256, 1024)).astype(np.float16)
    b = rng.uniform(-1, 1, (1024, 1024)).astype(np.float16)
    d = rng.uniform(-1, 1, (1024, 1024)).astype(np.float16)
    c_ref = cutlass_gemm(a, b)
    assert (bits(o.gemm_f16(a, b)) == bits(c_ref)).all()
    # the chain: the intermediate is rounded to half once, then feeds the second GEMM
    e_ref = cutlass_gemm(c_ref, d)
    assert (bits(o.gemm_f16(o.gemm_f16(a, b), d)) == bits(e_ref)).all()


def test_gemm_at_gpt3_width_is_bit_exact_with_cutlass_host_gemm():
    # GPT-3 shard: K = 12288 (first GEMM) and K = 6144 (second), X ~ N(0,1), weights ~ N(0, 0.02); a sample of
    # rows and columns keeps CUTLASS's scalar host loop to a few seconds.
    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 12288)).astype(np.float16)
    w1 = (rng.standard_normal((12288, 512)) * 0.02).astype(np.float16)
    assert (bits(o.gemm_f16(x, w1)) == bits(cutlass_gemm(x, w1))).all()
    h = rng.standard_normal((8, 6144)).astype(np.float16)
    w2 = (rng.standard_normal((6144, 768)) * 0.02).astype(np.float16)
    assert (bits(o.gemm_f16(h, w2)) == bits(cutlass_gemm(h, w2))).all()


def test_conv3x3_config5_is_bit_exact_with_cutlass_host_conv2dfprop():
    # BASELINE config 5, N = 1: X[1,56,56,64] ~ N(0,1), filters [64,3,3,64] He-normal; two convolutions in a row.
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 56, 56, 64)).astype(np.float16)
    w1 = (rng.standard_normal((64, 3, 3, 64)) * (2.0 / 576) ** 0.5).astype(np.float16)
    w2 = (rng.standard_normal((64, 3, 3, 64)) * (2.0 / 576) ** 0.5).astype(np.float16)
    y1_ref = cutlass_conv(x, w1)
    y1 = o.conv2d_3x3_nhwc_f16(x, w1, relu=False)
    assert ulp_distance(y1, y1_ref).max() == 0
    y2_ref = cutlass_conv(y1_ref, w2)
    assert ulp_distance(o.conv2d_3x3_nhwc_f16(y1, w2, relu=False), y2_ref).max() == 0
    # the fused ReLU of config 5 against CUTLASS's ReLu functor applied to its own convolution
    relu_ref = cutlass_act(2, y1_ref.astype(np.float32)).astype(np.float16)
    assert (bits(o.conv2d_3x3_nhwc_f16(x, w1, relu=True)) == bits(relu_ref)).all()


def test_ragged_conv_shape_matches_cutlass():
    rng = np.random.default_rng(6)
    x = rng.standard_normal((2, 7, 5, 16)).astype(np.float16)
    w = (rng.standard_normal((24, 3, 3, 16)) * 0.1).astype(np.float16)
    assert ulp_distance(o.conv2d_3x3_nhwc_f16(x, w, relu=False), cutlass_conv(x, w)).max() == 0


def _epilogue_through_oracle(x, epi):
    """The oracle's epilogue applied to the fp32 values x (exact in half): a K = 1 GEMM x[:,None] * [1]."""
    a = x.astype(np.float16).reshape(-1, 1)
    one = np.ones((1, 1), np.float16)
    return o.gemm_f16(a, one, epi).reshape(-1)


def test_gelu_erf_and_relu_are_bit_exact_with_cutlass_functors():
    x = np.arange(-0x7bff, 0x7c00, dtype=np.int32)            # every finite half, by bit pattern
    x = np.where(x < 0, (-x) | 0x8000, x).astype(np.uint16).view(np.float16)
    xf = x.astype(np.float32)
    gelu_ref = cutlass_act(1, xf).astype(np.float16)
    assert (bits(_epilogue_through_oracle(xf, o.EPI_GELU_ERF)) == bits(gelu_ref)).all()
    relu_ref = cutlass_act(2, xf).astype(np.float16)
    assert (bits(_epilogue_through_oracle(xf, o.EPI_RELU)) == bits(relu_ref)).all()


def test_silu_mul_is_within_one_half_ulp_of_cutlass_silu():
    rng = np.random.default_rng(7)
    a = np.concatenate([np.linspace(-12, 12, 4001), rng.standard_normal(4000) * 3]).astype(np.float16)
    b = rng.standard_normal(a.size).astype(np.float16)
    # A dual GEMM with K = 2 whose operands pick the two columns apart: row i has the accumulators (a_i, b_i) exactly.
    got = np.empty(a.size, np.float16)
    pick_a, pick_b = np.array([[1.0], [0.0]], np.float16), np.array([[0.0], [1.0]], np.float16)
    for lo in range(0, a.size, 2000):
        g = o.gemm_dual_silu_mul_f16(np.stack([a[lo:lo + 2000], b[lo:lo + 2000]], 1), pick_a, pick_b)
        got[lo:lo + 2000] = g.reshape(-1)
    ref = (cutlass_act(3, a.astype(np.float32)) * b.astype(np.float32)).astype(np.float16)
    d = ulp_distance(got, ref)
    assert d.max() <= 1, int(d.max())
