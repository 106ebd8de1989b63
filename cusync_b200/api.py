"""Host-side mirror of the reference's C++ API over the C ABI.

Names and argument meaning follow microsoft/cusync:
  CuStage, CuSync.setProducerConsumerPair          src/include/cusync/cusync.h:87-299
  NoSync, RowSync, TileSync, Conv2DTileSync        src/include/cusync/policies.h:18-210
  StridedTileSync (StridedSync)                    src/ml-bench/transformer/mlp.cu:76-101
  ConsecutiveTileSync (ConsecutiveSync)            src/ml-bench/transformer/attention.cu:51-70
  IdentityOrder, TransposeXYOrder                  src/include/cusync/tile-orders.h:50-76
  Gemm: Arguments -> can_implement -> initialize -> run -> incrementIter
                                                   gemm/device/cusyncgemm.h:293-563, mlp.cu:653-712
Tensors are passed as raw device pointers (e.g. torch.Tensor.data_ptr()).
"""
import ctypes as C

import numpy as np

from . import _lib as L


class Optimizations:
    NoOptimization = L.OPT_NONE
    NoAtomicAdd = L.OPT_NO_ATOMIC_ADD
    AvoidWaitKernel = L.OPT_AVOID_WAIT_KERNEL
    AvoidCustomOrder = L.OPT_AVOID_CUSTOM_ORDER
    ReorderTileLoads = L.OPT_REORDER_TILE_LOADS
    StreamWait = L.OPT_STREAM_WAIT          # addition: the wait before a dependent launch without a kernel


class IdentityOrder:
    kind = L.ORDER_IDENTITY


class TransposeXYOrder:
    kind = L.ORDER_TRANSPOSE_XY


class GroupedRowsOrder:
    """Addition: blocks taken in groups of `rows` grid rows, row index fastest inside a group."""

    def __init__(self, rows):
        self.kind = L.order_grouped(rows)


def _order(o):
    return o if isinstance(o, int) else o.kind


class NoSync:
    def desc(self):
        return L.Policy(L.POLICY_NOSYNC, 0, 1, 1, 0, 0, 0, 0)


class RowSync:
    """RowSync<TileM>(waitValue[, postValue]): one semaphore per row panel."""

    def __init__(self, tile_m, wait_value=0, post_value=None):
        self.tile_m, self.wait_value = tile_m, wait_value
        self.post_value = (1 if wait_value else 0) if post_value is None else post_value

    def desc(self):
        return L.Policy(L.POLICY_ROWSYNC, L.ORDER_TRANSPOSE_XY, self.tile_m, 1, self.wait_value, self.post_value, 0, 0)


class TileSync:
    """TileSync<TileOrder, TileM, TileN>(waitValue=1, postValue=1): one semaphore per tile."""

    def __init__(self, order, tile_m, tile_n, wait_value=1, post_value=1):
        self.order, self.tile_m, self.tile_n = _order(order), tile_m, tile_n
        self.wait_value, self.post_value = wait_value, post_value

    def desc(self):
        return L.Policy(L.POLICY_TILESYNC, self.order, self.tile_m, self.tile_n, self.wait_value, self.post_value, 0, 0)


class StridedTileSync:
    """StridedSync<TileOrder, GridN, TileM, TileN, stride>: N-tiles j and j + GridN/TileN share a semaphore."""

    def __init__(self, order, grid_n, tile_m, tile_n, stride):
        self.order, self.grid_n, self.tile_m, self.tile_n, self.stride = _order(order), grid_n, tile_m, tile_n, stride

    def desc(self):
        return L.Policy(L.POLICY_STRIDEDTILESYNC, self.order, self.tile_m, self.tile_n, 0, 0, self.grid_n, self.stride)


class ConsecutiveTileSync:
    """ConsecutiveSync<TileOrder, H, TileM, TileN>: the (H/8)/TileN adjacent N-tiles of one third share a semaphore."""

    def __init__(self, order, h, tile_m, tile_n):
        self.order, self.h, self.tile_m, self.tile_n = _order(order), h, tile_m, tile_n

    def desc(self):
        return L.Policy(L.POLICY_CONSECUTIVETILESYNC, self.order, self.tile_m, self.tile_n, 0, 0, self.h, 0)


class Conv2DTileSync:
    """Conv2DTileSync<TileOrder, R, S, TileM, TileN>(waitValue=1, postValue=1)."""

    def __init__(self, order, r, s, tile_m, tile_n, wait_value=1, post_value=1):
        self.order, self.rs, self.tile_m, self.tile_n = _order(order), r * s, tile_m, tile_n
        self.wait_value, self.post_value = wait_value, post_value

    def desc(self):
        return L.Policy(L.POLICY_CONV2DTILESYNC, self.order, self.tile_m, self.tile_n, self.wait_value,
                        self.post_value, self.rs, 0)


def _stream_ptr(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream   # torch.cuda.Stream


class CuStage:
    """CuStage<TileOrder, InputSyncPolicy, OutputSyncPolicy, Opts>(grid, tileSize, inputPolicy, outputPolicy)."""

    def __init__(self, order, grid, tile_size, input_policy, output_policy, opts=Optimizations.NoOptimization):
        self._h = C.c_void_p()
        self.input_policy, self.output_policy, self.opts = input_policy, output_policy, opts
        self._grid = tuple(grid)
        ip, op = input_policy.desc(), output_policy.desc()
        rc = L.lib().cusync_stage_create(C.byref(self._h), L.Dim3(*grid), L.Dim3(*tile_size), _order(order),
                                         C.byref(ip), C.byref(op), opts)
        self.create_status = rc
        if rc not in (L.SUCCESS, L.ERROR_INVALID_LINEAR_BLOCK_INDEX):
            raise L.CuSyncError(rc, "CuStage")

    # -- reference API ---------------------------------------------------
    def grid(self):
        return self._grid

    def numTiles(self):
        return L.lib().cusync_stage_num_tiles(self._h)

    def isProducer(self):
        return not isinstance(self.output_policy, NoSync)

    def isConsumer(self):
        return not isinstance(self.input_policy, NoSync)

    def incrementIter(self):
        L.check(L.lib().cusync_stage_increment_iter(self._h), "incrementIter")

    def invokeWaitKernel(self, stream):
        return L.lib().cusync_stage_invoke_wait_kernel(self._h, _stream_ptr(stream))

    def getNoAtomicAdd(self):
        return bool(self.opts & Optimizations.NoAtomicAdd)

    def getAvoidWaitKernel(self):
        return bool(self.opts & Optimizations.AvoidWaitKernel)

    def getReorderTileLoads(self):
        return bool(self.opts & Optimizations.ReorderTileLoads)

    def getAvoidCustomOrder(self):
        return bool(self.opts & Optimizations.AvoidCustomOrder)

    # -- additions ---------------------------------------------------------
    @property
    def iter(self):
        return L.lib().cusync_stage_iter(self._h)

    def reset(self, stream=None):
        L.check(L.lib().cusync_stage_reset(self._h, _stream_ptr(stream)), "reset")

    def set_timeout_ns(self, ns):
        L.check(L.lib().cusync_stage_set_timeout_ns(self._h, int(ns)), "set_timeout_ns")

    def view(self):
        v = L.StageView()
        L.check(L.lib().cusync_stage_get_view(self._h, C.byref(v)), "get_view")
        return v

    def tile_order(self):
        n = self.numTiles()
        out = np.zeros((n, 3), dtype=np.uint32)
        L.check(L.lib().cusync_stage_read_tile_order(self._h, out.ctypes.data_as(C.c_void_p), n), "read_tile_order")
        return out

    def semaphores(self):
        n = self.numTiles()
        out = np.zeros(n, dtype=np.uint32)
        L.check(L.lib().cusync_stage_read_semaphores(self._h, out.ctypes.data_as(C.c_void_p), n), "read_semaphores")
        return out

    def status(self):
        s = L.Status()
        L.check(L.lib().cusync_stage_read_status(self._h, C.byref(s)), "read_status")
        return s

    def destroy(self):
        if self._h:
            L.lib().cusync_stage_destroy(self._h)
            self._h = C.c_void_p()


class CuSync:
    @staticmethod
    def setProducerConsumerPair(prod, cons):
        return L.lib().cusync_stage_link(prod._h, cons._h)

    setProducerConsumer = setProducerConsumerPair


def gemm_tiled_shape(m, n, tile_m, tile_n, split_k=1):  # noqa: D401
    """CuSyncGemmHorizontalThreadblockSwizzle::get_tiled_shape + get_grid_shape
    (gemm/threadblock/cusync_threadblock_swizzle.h:12-54): the launch grid is (tilesN, tilesM, splitK)."""
    return ((n + tile_n - 1) // tile_n, (m + tile_m - 1) // tile_m, split_k)


class GemmArguments:
    """Arguments{custage, problem_size, ref_A, ref_B, ref_C, ref_D, {alpha, beta}, split_k_slices}
    (gemm/device/cusyncgemm.h:293-350).  ref_C is unused (beta = 0 in every reference driver)."""

    def __init__(self, custage, problem_size, ref_a, ref_b, ref_d, epilogue=L.EPILOGUE_NONE, ref_b2=None,
                 b_layout=L.B_ROW_MAJOR_KN, tile_n=0, max_ctas=0, split_k_slices=0, cta_pair=0, tail_split=0):
        self.custage, self.problem_size = custage, problem_size
        self.ref_a, self.ref_b, self.ref_b2, self.ref_d = ref_a, ref_b, ref_b2, ref_d
        self.epilogue, self.b_layout, self.tile_n, self.max_ctas = epilogue, b_layout, tile_n, max_ctas
        self.cta_pair = cta_pair
        self.split_k_slices = split_k_slices
        self.tail_split = tail_split   # K slices for the tiles of the last partial wave: 0 = choose, 1 = none


def _ref(t):
    """(pointer, leading dimension) of a 2-D row-major tensor-like (torch.Tensor) or a (ptr, ld) pair."""
    if isinstance(t, tuple):
        return t
    assert t.dim() == 2 and t.stride(1) == 1
    return t.data_ptr(), t.stride(0)


class Gemm:
    """cutlass::gemm::device::CuSyncGemm's call pattern on the sm_100a kernels."""

    TILE_M = 128

    def __init__(self):
        self._plan = C.c_void_p()
        self.args = None

    @staticmethod
    def default_tile_n(m, n, k, epilogue=L.EPILOGUE_NONE):
        return L.lib().cusync_gemm_default_tile_n(m, n, k, epilogue)

    def _desc(self, args):
        m, n, k = args.problem_size
        a, lda = _ref(args.ref_a)
        b, ldb = _ref(args.ref_b)
        d, ldd = _ref(args.ref_d)
        b2 = _ref(args.ref_b2)[0] if args.ref_b2 is not None else None
        return L.GemmDesc(m, n, k, a, lda, b, ldb, b2, d, ldd, args.b_layout, args.epilogue, args.tile_n,
                          args.max_ctas, args.split_k_slices, args.cta_pair, args.tail_split, args.custage._h if args.custage is not None else None)

    def can_implement(self, args):
        if args.split_k_slices < 0 or (args.split_k_slices > 1 and args.epilogue == L.EPILOGUE_SILU_MUL_DUAL):
            return L.ERROR_UNSUPPORTED
        return L.SUCCESS

    @staticmethod
    def default_split_k(m, n, k, epilogue=L.EPILOGUE_NONE, tile_n=0, cta_pair=0):
        return L.lib().cusync_gemm_default_split_k(m, n, k, epilogue, tile_n, cta_pair)

    def initialize(self, args, workspace=None):
        if self.can_implement(args) != L.SUCCESS:
            return L.ERROR_UNSUPPORTED
        self.destroy()
        self.args = args
        d = self._desc(args)
        return L.lib().cusync_gemm_plan_create(C.byref(self._plan), C.byref(d))

    def run(self, overlap=True, unused=None, stream=None):
        return L.lib().cusync_gemm_run(self._plan, _stream_ptr(stream))

    def run_dependent(self, stream=None):
        """The launch as a programmatic dependent of the kernel ahead of it in `stream` (consumers only): resident
        once every block of that kernel is, with no wait kernel or second stream."""
        return L.lib().cusync_gemm_run_dependent(self._plan, _stream_ptr(stream))

    @staticmethod
    def run_chain(first, second, stream=None):
        """Both GEMMs as one persistent grid (cusync_gemm_run_chain): `second` consumes what `first` produces."""
        return L.lib().cusync_gemm_run_chain(first._plan, second._plan, _stream_ptr(stream))

    def num_ctas(self):
        return L.lib().cusync_gemm_plan_num_ctas(self._plan)

    def tail_split(self):
        return L.lib().cusync_gemm_plan_tail_split(self._plan)

    def destroy(self):
        if self._plan:
            L.lib().cusync_gemm_plan_destroy(self._plan)
            self._plan = C.c_void_p()


class Conv2dProblemSize:
    """cutlass::conv::Conv2dProblemSize as resnet.cu builds it: input NHWC, filter KRSC, stride 1, pad 1."""

    def __init__(self, n, h, w, c, k, r=3, s=3, pad=1, stride=1):
        self.n, self.h, self.w, self.c, self.k, self.r, self.s, self.pad, self.stride = n, h, w, c, k, r, s, pad, stride

    def tile_rows(self):
        return L.lib().cusync_conv2d_tile_rows_hw(self.h, self.w)

    def tile_n(self):
        """Output channels per N tile: the TileN argument of the sync policies."""
        return L.lib().cusync_conv2d_default_tile_n(self.n, self.h, self.w, self.c, self.k)

    def grid(self):
        """Stage grid (N tiles, M tiles, 1) of the implicit GEMM."""
        return (self.k // max(self.tile_n(), 1), self.n * self.h // max(self.tile_rows(), 1), 1)

    def tile_m(self):
        """Output pixels per M tile: the TileM argument of the sync policies."""
        return self.tile_rows() * self.w


class Conv2dFprop:
    """cutlass::conv::device::CuSyncImplicitGemmConvolution's call pattern (Arguments -> can_implement ->
    initialize -> run) on the sm_100a implicit-GEMM kernel."""

    def __init__(self):
        self._plan = C.c_void_p()

    GENERAL, SLAB = 1, 2      # cusync_conv2d_desc_t.kernel

    def initialize(self, custage, problem, x, filt, y, epilogue=L.EPILOGUE_NONE, max_ctas=0, kernel=0):
        self.destroy()
        d = L.Conv2dDesc(problem.n, problem.h, problem.w, problem.c, problem.k, problem.r, problem.s, problem.stride,
                         problem.pad, x.data_ptr(), filt.data_ptr(), y.data_ptr(), epilogue, max_ctas, kernel,
                         custage._h if custage is not None else None)
        return L.lib().cusync_conv2d_plan_create(C.byref(self._plan), C.byref(d))

    def run(self, stream=None):
        return L.lib().cusync_conv2d_run(self._plan, _stream_ptr(stream))

    def run_dependent(self, stream=None):
        return L.lib().cusync_conv2d_run_dependent(self._plan, _stream_ptr(stream))

    def num_ctas(self):
        return L.lib().cusync_conv2d_plan_num_ctas(self._plan)

    def destroy(self):
        if self._plan:
            L.lib().cusync_conv2d_plan_destroy(self._plan)
            self._plan = C.c_void_p()
