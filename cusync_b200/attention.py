"""GPT-3 attention block, one tensor-parallel shard, as a three-stage CuSync chain (host-side driver).

Stage wiring follows src/ml-bench/transformer/attention.cu (XQKVCuStage -> middle stages -> XW12CuStage,
:105-118; runAttentionCuSync :706-833): QKV projection (producer, ConsecutiveSync out) -> decode attention
(waits and posts) -> output projection (RowSync in).  Unlike the reference's chain, the middle stage is a real
attention with heads and an fp32 softmax over a K/V cache.
"""
import ctypes as C

from . import _lib as L
from .api import _stream_ptr

HEAD_DIM = 128


class DecodeAttention:
    """Plan of the attention step alone (cusync_attn_*)."""

    def __init__(self, custage, qkv, k_cache, v_cache, out, heads, kv_splits=0):
        batch, seq = qkv.shape[0], (k_cache.shape[1] if k_cache is not None else 0)
        d = L.AttnDesc(batch, seq, heads, HEAD_DIM, qkv.data_ptr(), qkv.stride(0),
                       k_cache.data_ptr() if k_cache is not None else None,
                       v_cache.data_ptr() if v_cache is not None else None,
                       out.data_ptr(), out.stride(0), kv_splits, custage._h if custage is not None else None)
        self._plan = C.c_void_p()
        self.create_status = L.lib().cusync_attn_plan_create(C.byref(self._plan), C.byref(d))

    def run(self, stream=None):
        return L.lib().cusync_attn_run(self._plan, _stream_ptr(stream))

    def run_dependent(self, stream=None):
        return L.lib().cusync_attn_run_dependent(self._plan, _stream_ptr(stream))

    def destroy(self):
        if self._plan:
            L.lib().cusync_attn_plan_destroy(self._plan)
            self._plan = C.c_void_p()


class _StageRef:
    """Read-only view of a stage the C driver owns."""

    def __init__(self, handle):
        self._h = handle

    def semaphores(self):
        import numpy as np
        n = L.lib().cusync_stage_num_tiles(self._h)
        out = np.zeros(n, dtype=np.uint32)
        L.check(L.lib().cusync_stage_read_semaphores(self._h, out.ctypes.data_as(C.c_void_p), n), "read_semaphores")
        return out

    def status(self):
        st = L.Status()
        L.lib().cusync_stage_read_status(self._h, C.byref(st))
        return st


class AttentionBlock:
    """x[B,H] -> y[B,H]: QKV projection [H, 3*heads*128], decode attention over the cache, projection [heads*128, H].
    The chain and its stream-ordered twin live in the C driver (cusync_attn_block_*); `synced` picks which one
    run() launches."""

    def __init__(self, x, w_qkv, k_cache, v_cache, w_o, heads, model_hidden=12288, synced=True, kv_splits=0):
        import torch
        self.batch, self.hidden, self.heads = x.shape[0], x.shape[1], heads
        hd = heads * HEAD_DIM
        assert w_qkv.shape == (self.hidden, 3 * hd) and w_o.shape[0] == hd
        dev = x.device
        self.qkv = torch.empty((self.batch, 3 * hd), device=dev, dtype=torch.half)
        self.o = torch.empty((self.batch, hd), device=dev, dtype=torch.half)
        self.y = torch.empty((self.batch, w_o.shape[1]), device=dev, dtype=torch.half)
        self.x, self.w_qkv, self.w_o, self.k_cache, self.v_cache = x, w_qkv, w_o, k_cache, v_cache
        seq = k_cache.shape[1] if k_cache is not None else 0
        d = L.AttnBlockDesc(self.batch, seq, self.hidden, heads, w_o.shape[1], model_hidden, kv_splits,
                            x.data_ptr(), w_qkv.data_ptr(),
                            k_cache.data_ptr() if k_cache is not None else None,
                            v_cache.data_ptr() if v_cache is not None else None,
                            w_o.data_ptr(), self.qkv.data_ptr(), self.o.data_ptr(), self.y.data_ptr())
        self._h = C.c_void_p()
        L.check(L.lib().cusync_attn_block_create(C.byref(self._h), C.byref(d)), "cusync_attn_block_create")
        cfg = (C.c_int32 * 5)()
        L.lib().cusync_attn_block_config(self._h, cfg)
        self.config = {"tile_n": (cfg[0], cfg[1]), "split_k": (cfg[2], cfg[3]), "kv_splits": cfg[4]}
        self.synced = synced
        self.s1, self.s2, self.s3 = (_StageRef(L.lib().cusync_attn_block_stage(self._h, i)) for i in range(3))

    def run(self, streams):
        """Synced: three streams, a wait kernel before each dependent stage (attention.cu:792-811).
        Not synced: everything on streams[0], in order."""
        if not self.synced:
            L.check(L.lib().cusync_attn_block_run_stream_ordered(self._h, _stream_ptr(streams[0])), "run_stream_ordered")
            return
        arr = (C.c_void_p * 3)(*[_stream_ptr(s) for s in streams])
        L.check(L.lib().cusync_attn_block_run_cusync(self._h, C.cast(arr, C.POINTER(C.c_void_p))), "run_cusync")

    def run_stream_ordered(self, stream):
        L.check(L.lib().cusync_attn_block_run_stream_ordered(self._h, _stream_ptr(stream)), "run_stream_ordered")

    def run_dependent(self, stream):
        """The synchronised stages on one stream, each dependent one a programmatic dependent launch."""
        L.check(L.lib().cusync_attn_block_run_dependent(self._h, _stream_ptr(stream)), "run_dependent")

    def status_codes(self):
        return tuple(st.status().code for st in (self.s1, self.s2, self.s3))

    def destroy(self):
        if self._h:
            L.lib().cusync_attn_block_destroy(self._h)
            self._h = C.c_void_p()


class PromptAttentionBlock:
    """The attention block in the prompt phase, as the reference runs it (attention.cu:272-276 with seqlen = 0):
    XQKV = X Wqkv; S = Q K^T; O = S V; Y = O Wo, four dependent GEMMs without softmax or heads, each on its own
    stream behind a wait kernel (cusync_attn_prompt_*).  x[B, H], w_qkv[H, 3 * heads * 128], w_o[heads * 128, out]."""

    def __init__(self, x, w_qkv, w_o, heads, model_hidden=12288):
        import torch
        self.batch, self.hidden, self.heads = x.shape[0], x.shape[1], heads
        hd = heads * HEAD_DIM
        assert w_qkv.shape == (self.hidden, 3 * hd) and w_o.shape[0] == hd
        dev = x.device
        self.qkv = torch.empty((self.batch, 3 * hd), device=dev, dtype=torch.half)
        self.s = torch.empty((self.batch, self.batch), device=dev, dtype=torch.half)
        self.o = torch.empty((self.batch, hd), device=dev, dtype=torch.half)
        self.y = torch.empty((self.batch, w_o.shape[1]), device=dev, dtype=torch.half)
        self.x, self.w_qkv, self.w_o = x, w_qkv, w_o
        d = L.AttnPromptDesc(self.batch, self.hidden, heads, w_o.shape[1], model_hidden, x.data_ptr(), w_qkv.data_ptr(),
                             w_o.data_ptr(), self.qkv.data_ptr(), self.s.data_ptr(), self.o.data_ptr(), self.y.data_ptr())
        self._h = C.c_void_p()
        L.check(L.lib().cusync_attn_prompt_create(C.byref(self._h), C.byref(d)), "cusync_attn_prompt_create")
        self.stages = [_StageRef(L.lib().cusync_attn_prompt_stage(self._h, i)) for i in range(4)]

    def flops(self):
        hd = self.heads * HEAD_DIM
        return 2.0 * self.batch * (self.hidden * 3 * hd + 2 * self.batch * hd + hd * self.y.shape[1])

    def run(self, streams):
        """Four streams, a wait kernel before each dependent GEMM (attention.cu:792-811)."""
        arr = (C.c_void_p * 4)(*[_stream_ptr(s) for s in streams])
        L.check(L.lib().cusync_attn_prompt_run_cusync(self._h, C.cast(arr, C.POINTER(C.c_void_p))), "run_cusync")

    def run_stream_ordered(self, stream):
        L.check(L.lib().cusync_attn_prompt_run_stream_ordered(self._h, _stream_ptr(stream)), "run_stream_ordered")

    def run_dependent(self, stream):
        """The four synchronised GEMMs on one stream, GEMMs 2 to 4 as programmatic dependent launches."""
        L.check(L.lib().cusync_attn_prompt_run_dependent(self._h, _stream_ptr(stream)), "run_dependent")

    def status_codes(self):
        return tuple(st.status().code for st in self.stages)

    def destroy(self):
        if self._h:
            L.lib().cusync_attn_prompt_destroy(self._h)
            self._h = C.c_void_p()
