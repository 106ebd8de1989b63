"""ctypes binding of libcusync_b200.so (the C ABI declared in include/cusync_b200.h).

The library is hand-written sm_100a CUDA; there is no fallback.  If the shared
object is missing this module raises at import of the symbol table, and every
compute call needs a CUDA device.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcusync_b200.so")

# status codes (include/cusync_b200.h)
ERROR_NOT_PRODUCER, ERROR_NOT_CONSUMER, ERROR_NOT_INITIALIZED, ERROR_INVALID_LINEAR_BLOCK_INDEX, \
    ERROR_CUDA, SUCCESS, ERROR_TIMEOUT, ERROR_INVALID_ARGUMENT, ERROR_UNSUPPORTED, ERROR_EXCEEDS_STATIC_SCRATCH = range(10)
ERROR_NAMES = ["CuSyncErrorNotProducer", "CuSyncErrorNotConsumer", "CuSyncErrorNotInitialized",
               "CuSyncErrorInvalidLinearBlockIndex", "CuSyncErrorCUDAError", "CuSyncSuccess",
               "CuSyncErrorTimeout", "CuSyncErrorInvalidArgument", "CuSyncErrorUnsupported",
               "CuSyncErrorExceedsStaticScratch"]

OPT_NONE, OPT_NO_ATOMIC_ADD, OPT_AVOID_WAIT_KERNEL, OPT_AVOID_CUSTOM_ORDER, OPT_REORDER_TILE_LOADS = 0, 1, 2, 4, 8
OPT_STREAM_WAIT = 16
ORDER_IDENTITY, ORDER_TRANSPOSE_XY, ORDER_GROUPED_ROWS = 0, 1, 2


def order_grouped(rows):
    return ORDER_GROUPED_ROWS | (rows << 8)

POLICY_NOSYNC, POLICY_ROWSYNC, POLICY_TILESYNC, POLICY_STRIDEDTILESYNC, POLICY_CONV2DTILESYNC, \
    POLICY_CONSECUTIVETILESYNC = range(6)
EPILOGUE_NONE, EPILOGUE_GELU_ERF, EPILOGUE_RELU, EPILOGUE_SILU_MUL_DUAL = range(4)
B_ROW_MAJOR_KN, B_ROW_MAJOR_NK = 0, 1


class Dim3(C.Structure):
    _fields_ = [("x", C.c_uint32), ("y", C.c_uint32), ("z", C.c_uint32)]


class Policy(C.Structure):
    _fields_ = [("kind", C.c_int32), ("order", C.c_int32), ("tile_m", C.c_uint32), ("tile_n", C.c_uint32),
                ("wait_value", C.c_uint32), ("post_value", C.c_uint32), ("p0", C.c_uint32), ("p1", C.c_uint32)]


class Status(C.Structure):
    _fields_ = [("code", C.c_uint32), ("where", C.c_uint32), ("tile_x", C.c_uint32), ("tile_y", C.c_uint32),
                ("tile_z", C.c_uint32), ("sem_index", C.c_uint32), ("seen", C.c_uint32), ("expected", C.c_uint32)]


class StageView(C.Structure):
    _fields_ = [("grid", Dim3), ("prod_grid", Dim3), ("tile_size", Dim3), ("iter", C.c_uint32),
                ("opts", C.c_int32), ("order", C.c_int32), ("reserved", C.c_int32),
                ("in_policy", Policy), ("out_policy", Policy),
                ("tile_order", C.c_void_p), ("tile_counter", C.c_void_p), ("started", C.c_void_p),
                ("sems_post", C.c_void_p), ("sems_wait", C.c_void_p), ("status", C.c_void_p),
                ("timeout_ns", C.c_uint64),
                ("prod_finished", C.c_void_p), ("prod_finish_target", C.c_uint32), ("reserved2", C.c_uint32)]


class GemmDesc(C.Structure):
    _fields_ = [("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("a", C.c_void_p), ("lda", C.c_int64),
                ("b", C.c_void_p), ("ldb", C.c_int64),
                ("b2", C.c_void_p),
                ("d", C.c_void_p), ("ldd", C.c_int64),
                ("b_layout", C.c_int32), ("epilogue", C.c_int32), ("tile_n", C.c_int32), ("max_ctas", C.c_int32),
                ("split_k", C.c_int32), ("cta_pair", C.c_int32), ("tail_split", C.c_int32), ("stage", C.c_void_p),
                ("b_stage", C.c_void_p), ("b_sem_first", C.c_uint32), ("b_sem_stride", C.c_uint32),
                ("b_sem_value", C.c_uint32)]


class Conv2dDesc(C.Structure):
    _fields_ = [("n", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("c", C.c_int32), ("k", C.c_int32),
                ("r", C.c_int32), ("s", C.c_int32), ("stride", C.c_int32), ("pad", C.c_int32),
                ("x", C.c_void_p), ("filter", C.c_void_p), ("y", C.c_void_p),
                ("epilogue", C.c_int32), ("max_ctas", C.c_int32), ("kernel", C.c_int32), ("stage", C.c_void_p)]


class ConvChainDesc(C.Structure):
    _fields_ = [("num_convs", C.c_int32), ("n", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("channels", C.c_int32),
                ("relu", C.c_int32), ("max_ctas", C.c_int32),
                ("filters", C.POINTER(C.c_void_p)), ("activations", C.POINTER(C.c_void_p))]


class AttnDesc(C.Structure):
    _fields_ = [("batch", C.c_int32), ("seq", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
                ("qkv", C.c_void_p), ("ld_qkv", C.c_int64), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("out", C.c_void_p), ("ld_out", C.c_int64), ("kv_splits", C.c_int32), ("stage", C.c_void_p)]


class AttnBlockDesc(C.Structure):
    _fields_ = [("batch", C.c_int32), ("seq", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32),
                ("out_features", C.c_int32), ("model_hidden", C.c_int32), ("kv_splits", C.c_int32),
                ("x", C.c_void_p), ("w_qkv", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("w_o", C.c_void_p), ("qkv", C.c_void_p), ("attn_out", C.c_void_p), ("y", C.c_void_p)]


class AttnPromptDesc(C.Structure):
    _fields_ = [("batch", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("out_features", C.c_int32),
                ("model_hidden", C.c_int32),
                ("x", C.c_void_p), ("w_qkv", C.c_void_p), ("w_o", C.c_void_p),
                ("qkv", C.c_void_p), ("s", C.c_void_p), ("o", C.c_void_p), ("y", C.c_void_p)]


class MlpDesc(C.Structure):
    _fields_ = [("model", C.c_int32), ("batch", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32),
                ("policy", C.c_int32), ("opts", C.c_int32), ("tile_n1", C.c_int32), ("tile_n2", C.c_int32),
                ("split_k1", C.c_int32), ("split_k2", C.c_int32), ("max_ctas", C.c_int32), ("cta_pair", C.c_int32), ("group_rows2", C.c_int32),
                ("tail_split_sync1", C.c_int32), ("tail_split_sync2", C.c_int32),
                ("tail_split_plain1", C.c_int32), ("tail_split_plain2", C.c_int32), ("group_rows1", C.c_int32),
                ("x_rows", C.c_int32), ("single_grid", C.c_int32), ("post_rows", C.c_int32),
                ("x", C.c_void_p), ("w1", C.c_void_p), ("v", C.c_void_p), ("w2", C.c_void_p),
                ("h", C.c_void_p), ("y", C.c_void_p)]


class AllReduceDesc(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("rows", C.c_int32), ("cols", C.c_int32),
                ("ld", C.c_int64), ("tile_rows", C.c_int32), ("num_ctas", C.c_int32),
                ("buffers", C.POINTER(C.c_void_p)), ("flags", C.POINTER(C.c_void_p)),
                ("multicast_buffer", C.c_void_p), ("multicast_flags", C.c_void_p), ("timeout_ns", C.c_uint64)]


class MlpChoice(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("policy", "single_grid", "stream_wait", "group_rows1", "group_rows2",
                                         "tile_n1", "tile_n2", "split_k1", "split_k2", "tail_split1")]


MLP_GPT3, MLP_LLAMA = 0, 1

# name -> (restype, argtypes); every function include/cusync_b200.h declares
_vp, _i, _u32, _u64 = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64
SIGNATURES = {
    "cusync_stage_create": (_i, [C.POINTER(_vp), Dim3, Dim3, _i, C.POINTER(Policy), C.POINTER(Policy), _i]),
    "cusync_stage_destroy": (_i, [_vp]),
    "cusync_stage_link": (_i, [_vp, _vp]),
    "cusync_stage_increment_iter": (_i, [_vp]),
    "cusync_stage_set_iter": (_i, [_vp, _u32]),
    "cusync_stage_write_tile_order": (_i, [_vp, _vp, _u32]),
    "cusync_stage_reset": (_i, [_vp, _vp]),
    "cusync_stage_get_view": (_i, [_vp, C.POINTER(StageView)]),
    "cusync_stage_set_timeout_ns": (_i, [_vp, _u64]),
    "cusync_stage_invoke_wait_kernel": (_i, [_vp, _vp]),
    "cusync_stage_note_launch": (_i, [_vp, _u32]),
    "cusync_wait_kernel": (_i, [_vp, _u32, _vp, _vp, _u64]),
    "cusync_wait_kernel_range": (_i, [_vp, _u32, _u32, _vp, _vp, _u64]),
    "cusync_stream_wait_values": (_i, [_vp, _u32, _u32, _vp]),
    "cusync_stream_write_values": (_i, [_vp, _u32, _u32, _vp]),
    "cusync_stage_read_tile_order": (_i, [_vp, _vp, _u32]),
    "cusync_stage_read_semaphores": (_i, [_vp, _vp, _u32]),
    "cusync_stage_read_status": (_i, [_vp, C.POINTER(Status)]),
    "cusync_stage_num_tiles": (_u32, [_vp]),
    "cusync_stage_iter": (_u32, [_vp]),
    "cusync_gemm_default_tile_n": (_i, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "cusync_gemm_default_split_k": (_i, [C.c_int32] * 6),
    "cusync_gemm_plan_create": (_i, [C.POINTER(_vp), C.POINTER(GemmDesc)]),
    "cusync_gemm_plan_destroy": (_i, [_vp]),
    "cusync_gemm_plan_update": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "cusync_gemm_run": (_i, [_vp, _vp]),
    "cusync_gemm_run_dependent": (_i, [_vp, _vp]),
    "cusync_gemm_plan_tail_split": (_i, [_vp]),
    "cusync_gemm_run_chain": (_i, [_vp, _vp, _vp]),
    "cusync_gemm_chain_supported": (_i, [_vp, _vp]),
    "cusync_gemm_chain_prepare": (_i, []),
    "cusync_mlp_uses_single_grid": (_i, [_vp]),
    "cusync_mlp_choose_config": (_i, [C.c_int32] * 4 + [C.POINTER(MlpChoice)]),
    "cusync_gemm_run_noalloc": (_i, [C.POINTER(GemmDesc), _vp]),
    "cusync_gemm_noalloc_read_status": (_i, [C.POINTER(Status)]),
    "cusync_gemm_plan_set_trace": (_i, [_vp, _vp, _u32]),
    "cusync_gemm_plan_num_ctas": (_u32, [_vp]),
    "cusync_conv2d_tile_rows": (_i, [C.c_int32]),
    "cusync_conv2d_tile_rows_hw": (_i, [C.c_int32, C.c_int32]),
    "cusync_conv2d_default_tile_n": (_i, [C.c_int32] * 5),
    "cusync_conv2d_plan_create": (_i, [C.POINTER(_vp), C.POINTER(Conv2dDesc)]),
    "cusync_conv2d_plan_destroy": (_i, [_vp]),
    "cusync_conv2d_run": (_i, [_vp, _vp]),
    "cusync_conv2d_run_dependent": (_i, [_vp, _vp]),
    "cusync_conv2d_plan_num_ctas": (_u32, [_vp]),
    "cusync_conv_chain_create": (_i, [C.POINTER(_vp), C.POINTER(ConvChainDesc)]),
    "cusync_conv_chain_destroy": (_i, [_vp]),
    "cusync_conv_chain_run_stream_ordered": (_i, [_vp, _vp]),
    "cusync_conv_chain_run_cusync": (_i, [_vp, C.POINTER(_vp)]),
    "cusync_conv_chain_run_dependent": (_i, [_vp, _vp]),
    "cusync_conv_chain_run_cusync_replayable": (_i, [_vp, C.POINTER(_vp)]),
    "cusync_conv_chain_stage": (_vp, [_vp, _i]),
    "cusync_conv_chain_uses_wait_kernels": (_i, [_vp]),
    "cusync_attn_default_splits": (_i, [C.c_int32] * 3),
    "cusync_attn_plan_create": (_i, [C.POINTER(_vp), C.POINTER(AttnDesc)]),
    "cusync_attn_plan_destroy": (_i, [_vp]),
    "cusync_attn_plan_splits": (_i, [_vp]),
    "cusync_attn_run": (_i, [_vp, _vp]),
    "cusync_attn_run_dependent": (_i, [_vp, _vp]),
    "cusync_attn_block_create": (_i, [C.POINTER(_vp), C.POINTER(AttnBlockDesc)]),
    "cusync_attn_block_destroy": (_i, [_vp]),
    "cusync_attn_block_run_stream_ordered": (_i, [_vp, _vp]),
    "cusync_attn_block_run_cusync": (_i, [_vp, C.POINTER(_vp)]),
    "cusync_attn_block_run_dependent": (_i, [_vp, _vp]),
    "cusync_attn_block_stage": (_vp, [_vp, _i]),
    "cusync_attn_block_config": (_i, [_vp, C.POINTER(C.c_int32)]),
    "cusync_attn_prompt_create": (_i, [C.POINTER(_vp), C.POINTER(AttnPromptDesc)]),
    "cusync_attn_prompt_destroy": (_i, [_vp]),
    "cusync_attn_prompt_run_stream_ordered": (_i, [_vp, _vp]),
    "cusync_attn_prompt_run_cusync": (_i, [_vp, C.POINTER(_vp)]),
    "cusync_attn_prompt_run_dependent": (_i, [_vp, _vp]),
    "cusync_attn_prompt_stage": (_vp, [_vp, _i]),
    "cusync_mlp_create": (_i, [C.POINTER(_vp), C.POINTER(MlpDesc)]),
    "cusync_mlp_destroy": (_i, [_vp]),
    "cusync_mlp_run_stream_ordered": (_i, [_vp, _vp]),
    "cusync_mlp_run_cusync": (_i, [_vp, _vp, _vp]),
    "cusync_mlp_run_dependent": (_i, [_vp, _vp]),
    "cusync_mlp_run_single": (_i, [_vp, _i, _vp]),
    "cusync_mlp_update_io": (_i, [_vp, _vp, _vp]),
    "cusync_mlp_stage": (_vp, [_vp, _i]),
    "cusync_mlp_set_trace": (_i, [_vp, _vp, _u32, _vp, _u32]),
    "cusync_mlp_config": (_i, [_vp, C.POINTER(C.c_int32)]),
    "cusync_mlp_tail_splits": (_i, [_vp, C.POINTER(C.c_int32)]),
    "cusync_mlp_wait_rows": (_i, [_vp, _u32, _u32, _vp]),
    "cusync_mlp_post_x_rows": (_i, [_vp, _u32, _u32, _vp]),
    "cusync_allreduce_flag_words": (_u32, [C.c_int32, C.c_int32]),
    "cusync_allreduce_plan_create": (_i, [C.POINTER(_vp), C.POINTER(AllReduceDesc)]),
    "cusync_allreduce_plan_destroy": (_i, [_vp]),
    "cusync_allreduce_run": (_i, [_vp, _vp, _u32, _vp]),
    "cusync_allreduce_read_status": (_i, [_vp, C.POINTER(Status)]),
    "cusync_allreduce_plan_num_ctas": (_u32, [_vp]),
    "cusync_mlp_run_cusync_allreduce": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "cusync_tp_unique_id": (_i, [_vp]),
    "cusync_tp_comm_create": (_i, [C.POINTER(_vp), C.c_int32, C.c_int32, _vp]),
    "cusync_tp_comm_destroy": (_i, [_vp]),
    "cusync_tp_all_reduce": (_i, [_vp, _vp, _u64, _vp]),
    "cusync_tp_layer_run": (_i, [_vp, _vp, _vp, _vp, _u64, _vp, _vp, _vp]),
    "cusync_b200_version": (C.c_char_p, []),
    "cusync_b200_sm_count": (_i, []),
}

_lib = None


class CuSyncLibraryError(RuntimeError):
    pass


def lib():
    """Loads the shared library.  There is no CPU or PyTorch fallback behind it."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise CuSyncLibraryError(
            "libcusync_b200.so is not built (%s). Run `python -m cusync_b200.build`; "
            "there is no fallback implementation." % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        f = getattr(L, name)
        f.restype = res
        f.argtypes = args
    _lib = L
    return L


class CuSyncError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        name = ERROR_NAMES[code] if 0 <= code < len(ERROR_NAMES) else str(code)
        super().__init__("%s: %s" % (what, name))


def check(code, what):
    if code != SUCCESS:
        raise CuSyncError(code, what)
