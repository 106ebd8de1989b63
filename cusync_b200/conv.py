"""Chain of 3x3 convolutions on CuSync stages (host-side driver).

Mirrors the flow of the reference drivers src/ml-bench/volta_conv2d/resnet.cu and vgg.cu: stages typed
TileSync -> Conv2DTileSync (resnet.cu:107-116), runBaseline (:461-520), the CuSync loop with a wait kernel
before each dependent convolution (:560-590).  The work is done by cusync_conv_chain_* of the C ABI; torch only
owns device memory and streams.
"""
import ctypes as C

from . import _lib as L
from .api import _stream_ptr


class ConvChain:
    """activations[0] -> conv(filters[0]) -> ... ; NHWC fp16 tensors, filters [K, 3, 3, C] with K == C."""

    def __init__(self, x, filters, relu=True, max_ctas=0):
        import torch
        n, h, w, c = x.shape
        self.x, self.filters = x, list(filters)
        self.outputs = [torch.empty_like(x) for _ in self.filters]
        acts = [x] + self.outputs
        self._filters = (C.c_void_p * len(self.filters))(*[f.data_ptr() for f in self.filters])
        self._acts = (C.c_void_p * len(acts))(*[a.data_ptr() for a in acts])
        d = L.ConvChainDesc(len(self.filters), n, h, w, c, 1 if relu else 0, max_ctas,
                            C.cast(self._filters, C.POINTER(C.c_void_p)), C.cast(self._acts, C.POINTER(C.c_void_p)))
        self._h = C.c_void_p()
        L.check(L.lib().cusync_conv_chain_create(C.byref(self._h), C.byref(d)), "cusync_conv_chain_create")
        self.uses_wait_kernels = bool(L.lib().cusync_conv_chain_uses_wait_kernels(self._h))

    @property
    def y(self):
        return self.outputs[-1]

    def run_stream_ordered(self, stream):
        L.check(L.lib().cusync_conv_chain_run_stream_ordered(self._h, _stream_ptr(stream)), "run_stream_ordered")

    def run_cusync(self, streams):
        """streams: one per convolution (producer first)."""
        arr = (C.c_void_p * len(streams))(*[_stream_ptr(s) for s in streams])
        L.check(L.lib().cusync_conv_chain_run_cusync(self._h, C.cast(arr, C.POINTER(C.c_void_p))), "run_cusync")

    def run_dependent(self, stream):
        """The synchronised convolutions on one stream, each dependent one a programmatic dependent launch."""
        L.check(L.lib().cusync_conv_chain_run_dependent(self._h, _stream_ptr(stream)), "run_dependent")

    def run_cusync_replayable(self, streams):
        """Reset + run, for recording into a CUDA graph captured on streams[0]; the caller joins the streams."""
        arr = (C.c_void_p * len(streams))(*[_stream_ptr(s) for s in streams])
        L.check(L.lib().cusync_conv_chain_run_cusync_replayable(self._h, C.cast(arr, C.POINTER(C.c_void_p))),
                "run_cusync_replayable")

    def status_codes(self):
        out = []
        for i in range(len(self.filters)):
            s = L.Status()
            L.lib().cusync_stage_read_status(L.lib().cusync_conv_chain_stage(self._h, i), C.byref(s))
            out.append(s.code)
        return tuple(out)

    def semaphores(self, which):
        import numpy as np
        st = L.lib().cusync_conv_chain_stage(self._h, which)
        n = L.lib().cusync_stage_num_tiles(st)
        out = np.zeros(n, dtype=np.uint32)
        L.check(L.lib().cusync_stage_read_semaphores(st, out.ctypes.data_as(C.c_void_p), n), "read_semaphores")
        return out

    def destroy(self):
        if self._h:
            L.lib().cusync_conv_chain_destroy(self._h)
            self._h = C.c_void_p()
