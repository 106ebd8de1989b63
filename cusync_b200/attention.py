"""GPT-3 attention block, one tensor-parallel shard, as a three-stage CuSync chain (host-side driver).

Stage wiring follows src/ml-bench/transformer/attention.cu (XQKVCuStage -> middle stages -> XW12CuStage,
:105-118; runAttentionCuSync :706-833): QKV projection (producer, ConsecutiveSync out) -> decode attention
(waits and posts) -> output projection (RowSync in).  Unlike the reference's chain, the middle stage is a real
attention with heads and an fp32 softmax over a K/V cache.
"""
import ctypes as C

from . import _lib as L
from .api import (CuStage, CuSync, Gemm, GemmArguments, NoSync, RowSync, ConsecutiveTileSync, TransposeXYOrder,
                  IdentityOrder, _stream_ptr)

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

    def destroy(self):
        if self._plan:
            L.lib().cusync_attn_plan_destroy(self._plan)
            self._plan = C.c_void_p()


class AttentionBlock:
    """x[B,H] -> y[B,H]: QKV projection [H, 3*heads*128], decode attention over the cache, projection [heads*128, H]."""

    def __init__(self, x, w_qkv, k_cache, v_cache, w_o, heads, model_hidden=12288, synced=True):
        import torch
        self.batch, self.hidden, self.heads = x.shape[0], x.shape[1], heads
        hd = heads * HEAD_DIM
        assert w_qkv.shape == (self.hidden, 3 * hd) and w_o.shape[0] == hd
        dev = x.device
        self.qkv = torch.empty((self.batch, 3 * hd), device=dev, dtype=torch.half)
        self.o = torch.empty((self.batch, hd), device=dev, dtype=torch.half)
        self.y = torch.empty((self.batch, w_o.shape[1]), device=dev, dtype=torch.half)
        self.x, self.w_qkv, self.w_o, self.k_cache, self.v_cache = x, w_qkv, w_o, k_cache, v_cache
        B, lib = self.batch, L.lib()
        tile_n1 = Gemm.default_tile_n(B, 3 * hd, self.hidden)
        split1 = Gemm.default_split_k(B, 3 * hd, self.hidden, L.EPILOGUE_NONE, tile_n1)
        tile_n3 = Gemm.default_tile_n(B, w_o.shape[1], hd)
        split3 = Gemm.default_split_k(B, w_o.shape[1], hd, L.EPILOGUE_NONE, tile_n3)
        seq = k_cache.shape[1]
        kv_splits = lib.cusync_attn_default_splits(B, seq, heads)
        tiles_m = (B + 127) // 128
        grid1 = ((3 * hd + tile_n1 - 1) // tile_n1, tiles_m, split1)
        grid2 = (heads, B, kv_splits)
        grid3 = ((w_o.shape[1] + tile_n3 - 1) // tile_n3, tiles_m, split3)
        self.config = {"tile_n": (tile_n1, tile_n3), "split_k": (split1, split3), "kv_splits": kv_splits}
        if synced:
            sync12 = ConsecutiveTileSync(TransposeXYOrder, model_hidden, 128, tile_n1)   # StridedSyncImpl, attention.cu:105-110
            sync23 = RowSync(128, 1, 1)
            self.s1 = CuStage(TransposeXYOrder, grid1, (1, 1, 1), NoSync(), sync12)
            self.s2 = CuStage(IdentityOrder, grid2, (1, 1, 1), sync12, sync23)
            self.s3 = CuStage(TransposeXYOrder, grid3, (1, 1, 1), sync23, NoSync())
            L.check(CuSync.setProducerConsumerPair(self.s1, self.s2), "link qkv -> attention")
            L.check(CuSync.setProducerConsumerPair(self.s2, self.s3), "link attention -> projection")
        else:
            self.s1 = CuStage(TransposeXYOrder, grid1, (1, 1, 1), NoSync(), NoSync())
            self.s2 = CuStage(IdentityOrder, grid2, (1, 1, 1), NoSync(), NoSync())
            self.s3 = CuStage(TransposeXYOrder, grid3, (1, 1, 1), NoSync(), NoSync())
        self.synced = synced
        self.g1, self.g3 = Gemm(), Gemm()
        L.check(self.g1.initialize(GemmArguments(self.s1, (B, 3 * hd, self.hidden), x, w_qkv, self.qkv, tile_n=tile_n1,
                                                 split_k_slices=split1)), "qkv gemm")
        self.attn = DecodeAttention(self.s2, self.qkv, k_cache, v_cache, self.o, heads, kv_splits)
        L.check(self.attn.create_status, "attention")
        L.check(self.g3.initialize(GemmArguments(self.s3, (B, w_o.shape[1], hd), self.o, w_o, self.y, tile_n=tile_n3,
                                                 split_k_slices=split3)), "projection gemm")

    def run(self, streams):
        """Synced: three streams, a wait kernel before each dependent stage (attention.cu:792-811).
        Not synced: everything on streams[0], in order."""
        if not self.synced:
            self.g1.run(stream=streams[0]); self.attn.run(streams[0]); self.g3.run(stream=streams[0])
            return
        s1, s2, s3 = streams
        self.g1.run(stream=s1)
        self.s1.invokeWaitKernel(s2)
        self.attn.run(s2)
        self.s2.invokeWaitKernel(s3)
        self.g3.run(stream=s3)
        for st in (self.s1, self.s2, self.s3):
            st.incrementIter()

    def status_codes(self):
        return tuple(st.status().code for st in (self.s1, self.s2, self.s3))

    def destroy(self):
        self.g1.destroy(); self.attn.destroy(); self.g3.destroy()
        for st in (self.s1, self.s2, self.s3):
            st.destroy()
