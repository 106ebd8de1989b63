"""Tensor-parallel MLP shard on the CuSync GEMM chain (host-side driver).

Mirrors the flow of the reference driver src/ml-bench/transformer/mlp.cu:
MLPParameters (:209-330) -> stages + setProducerConsumerPair (:1026-1062) ->
runBaseline* (:411-491) / runCuSync* (:645-716).  The work is done by
cusync_mlp_* of the C ABI; torch only owns device memory, streams and, for
N > 1 GPUs, the NCCL all-reduce of the row-parallel output.
"""
import ctypes as C

from . import _lib as L
from .api import _stream_ptr

# (hidden, ffn-per-shard) of the models the reference benchmarks, one 8-way tensor-parallel shard
GPT3_HIDDEN, GPT3_FFN = 12288, 4 * 12288 // 8          # mlp.cu:243-245
LLAMA_HIDDEN = 8192
LLAMA_FFN_REFERENCE = ((8192 // 3 + 127) // 128) * 128  # 2816, mlp.cu:247-250
LLAMA_FFN = 2752                                        # 65.2B model: 22016 / 8

POLICIES = {"rowsync": L.POLICY_ROWSYNC, "tilesync": L.POLICY_TILESYNC, "auto": 0}


def choose_config(model, batch, hidden=None, ffn=None):
    """What the library picks for a layer left to its choice (cusync_mlp_choose_config), as a dict."""
    gpt3 = model == "gpt3"
    hidden = hidden or (GPT3_HIDDEN if gpt3 else LLAMA_HIDDEN)
    ffn = ffn or (GPT3_FFN if gpt3 else LLAMA_FFN)
    c = L.MlpChoice()
    L.check(L.lib().cusync_mlp_choose_config(L.MLP_GPT3 if gpt3 else L.MLP_LLAMA, batch, hidden, ffn, C.byref(c)),
            "cusync_mlp_choose_config")
    return {n: getattr(c, n) for n, _ in L.MlpChoice._fields_}


class MLPShard:
    """x[B,H] -> y[B,H] through W1 (and V) [H,F] and W2 [F,H]; fp16, fp32 accumulate."""

    def __init__(self, model, batch, x, w1, w2, v=None, policy="rowsync", opts=0, tile_n1=0, tile_n2=0, max_ctas=0,
                 group_rows2=0, cta_pair=0, split_k1=0, split_k2=0, tail_split=(0, 0, 0, 0), post_rows=False, group_rows1=0, x_rows=False, single_grid=0, y=None):
        import torch
        self.model = L.MLP_GPT3 if model == "gpt3" else L.MLP_LLAMA
        self.batch, self.hidden, self.ffn = batch, w1.shape[0], w1.shape[1]
        assert x.shape == (batch, self.hidden) and w2.shape == (self.ffn, self.hidden)
        self.x, self.w1, self.w2, self.v = x, w1, w2, v
        self.h = torch.empty((batch, self.ffn), device=x.device, dtype=torch.half)
        # y may be the caller's (e.g. symmetric memory that an all-reduce kernel of another rank can reach)
        self.y = y if y is not None else torch.empty((batch, self.hidden), device=x.device, dtype=torch.half)
        assert self.y.shape == (batch, self.hidden) and self.y.is_contiguous()
        d = L.MlpDesc(self.model, batch, self.hidden, self.ffn, POLICIES[policy], opts, tile_n1, tile_n2, split_k1,
                      split_k2, max_ctas, cta_pair, group_rows2, tail_split[0], tail_split[1], tail_split[2], tail_split[3], group_rows1, 1 if x_rows else 0, single_grid, 1 if post_rows else 0,
                      x.data_ptr(), w1.data_ptr(), v.data_ptr() if v is not None else None, w2.data_ptr(),
                      self.h.data_ptr(), self.y.data_ptr())
        self._h = C.c_void_p()
        L.check(L.lib().cusync_mlp_create(C.byref(self._h), C.byref(d)), "cusync_mlp_create")
        cfg = (C.c_int32 * 6)()
        L.lib().cusync_mlp_config(self._h, cfg)
        self.tile_n1, self.tile_n2, self.ctas1, self.ctas2, self.split_k1, self.split_k2 = list(cfg)
        ts = (C.c_int32 * 4)()
        L.lib().cusync_mlp_tail_splits(self._h, ts)
        self.tail_splits = tuple(ts)   # (synchronised GEMM 1, 2, stream-ordered GEMM 1, 2)
        self.single_grid = bool(L.lib().cusync_mlp_uses_single_grid(self._h))

    def run_stream_ordered(self, stream):
        L.check(L.lib().cusync_mlp_run_stream_ordered(self._h, _stream_ptr(stream)), "run_stream_ordered")

    def run_cusync(self, producer_stream, consumer_stream):
        L.check(L.lib().cusync_mlp_run_cusync(self._h, _stream_ptr(producer_stream), _stream_ptr(consumer_stream)),
                "run_cusync")

    def run_dependent(self, stream):
        """The two synchronised GEMMs on one stream, the second a programmatic dependent launch of the first."""
        L.check(L.lib().cusync_mlp_run_dependent(self._h, _stream_ptr(stream)), "run_dependent")

    def run_cusync_allreduce(self, reducer, producer_stream, consumer_stream, reduce_stream):
        """One layer with its all-reduce overlapped (post_rows=True): `reducer` is a tp.RowAllReduce over self.y."""
        L.check(L.lib().cusync_mlp_run_cusync_allreduce(self._h, reducer._plan, _stream_ptr(producer_stream),
                                                        _stream_ptr(consumer_stream), _stream_ptr(reduce_stream)),
                "run_cusync_allreduce")

    def post_x_rows(self, first_tile, num_tiles, stream):
        """x_rows=True: the 128-row tiles [first_tile, first_tile + num_tiles) of x are complete once what `stream`
        holds so far has run; call once per tile and run_cusync (the j-th post of a tile feeds the j-th run),
        before or after that run's launch."""
        L.check(L.lib().cusync_mlp_post_x_rows(self._h, first_tile, num_tiles, _stream_ptr(stream)), "post_x_rows")

    def wait_rows(self, first_tile, num_tiles, stream):
        """After run_cusync (post_rows=True): work enqueued on `stream` afterwards sees the 128-row tiles
        [first_tile, first_tile + num_tiles) of y complete."""
        L.check(L.lib().cusync_mlp_wait_rows(self._h, first_tile, num_tiles, _stream_ptr(stream)), "wait_rows")

    def run_single(self, which, stream):
        L.check(L.lib().cusync_mlp_run_single(self._h, which, _stream_ptr(stream)), "run_single")

    def update_io(self, x=None, y=None):
        L.check(L.lib().cusync_mlp_update_io(self._h, x.data_ptr() if x is not None else None,
                                             y.data_ptr() if y is not None else None), "update_io")
        if x is not None:
            self.x = x
        if y is not None:
            self.y = y

    def traced_run(self, producer_stream, consumer_stream):
        """One run_cusync with the per-tile timeline switched on (cusync_mlp_set_trace).  Returns two int64 arrays
        [records, 8], one per GEMM; the CTA-pair kernels write record 2 * ticket + rank: {globaltimer at the ticket
        draw, at the end of the tile's MMAs, after its stores and post, SM id << 32 | block, cycles the MMA thread
        waited for operands, cycles the loader waited for a free ring slot, cycles of the tile in the MMA thread,
        of which waiting for a free accumulator} (the cycle counts in the leader's records only)."""
        import torch
        cap1 = 2 * ((self.batch + 255) // 256) * ((self.ffn + self.tile_n1 - 1) // self.tile_n1) * max(self.split_k1, 1)
        cap2 = 2 * ((self.batch + 255) // 256) * ((self.hidden + self.tile_n2 - 1) // self.tile_n2) * max(self.split_k2, 1)
        cap1, cap2 = max(cap1, 2 * self.ctas1), max(cap2, 2 * self.ctas2)
        t1 = torch.zeros((cap1, 8), dtype=torch.int64, device=self.x.device)
        t2 = torch.zeros((cap2, 8), dtype=torch.int64, device=self.x.device)
        torch.cuda.synchronize()
        L.check(L.lib().cusync_mlp_set_trace(self._h, t1.data_ptr(), cap1, t2.data_ptr(), cap2), "cusync_mlp_set_trace")
        try:
            self.run_cusync(producer_stream, consumer_stream)
            torch.cuda.synchronize()
        finally:
            L.lib().cusync_mlp_set_trace(self._h, None, 0, None, 0)
        return t1.cpu().numpy(), t2.cpu().numpy()

    def _stage_status(self, which):
        s = L.Status()
        L.lib().cusync_stage_read_status(L.lib().cusync_mlp_stage(self._h, which), C.byref(s))
        return s

    def status_codes(self):
        return self._stage_status(0).code, self._stage_status(1).code

    def producer_semaphores(self):
        import numpy as np
        st = L.lib().cusync_mlp_stage(self._h, 0)
        n = L.lib().cusync_stage_num_tiles(st)
        out = np.zeros(n, dtype=np.uint32)
        L.check(L.lib().cusync_stage_read_semaphores(st, out.ctypes.data_as(C.c_void_p), n), "read_semaphores")
        return out

    def flops(self):
        mult = 3 if self.model == L.MLP_LLAMA else 2
        return 2.0 * self.batch * self.hidden * self.ffn * mult

    def destroy(self):
        if self._h:
            L.lib().cusync_mlp_destroy(self._h)
            self._h = C.c_void_p()


def make_inputs(model, batch, device, seed=0, ffn=None):
    """Seeded synthetic inputs with the shapes and distributions of the benchmark configs:
    X ~ N(0,1), weights ~ N(0, 0.02)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    if model == "gpt3":
        hidden, f = GPT3_HIDDEN, ffn or GPT3_FFN
    else:
        hidden, f = LLAMA_HIDDEN, ffn or LLAMA_FFN
    x = torch.randn((batch, hidden), generator=g, device=device, dtype=torch.float32).half()
    w1 = (torch.randn((hidden, f), generator=g, device=device, dtype=torch.float32) * 0.02).half()
    w2 = (torch.randn((f, hidden), generator=g, device=device, dtype=torch.float32) * 0.02).half()
    v = None
    if model != "gpt3":
        v = (torch.randn((hidden, f), generator=g, device=device, dtype=torch.float32) * 0.02).half()
    return x, w1, w2, v
