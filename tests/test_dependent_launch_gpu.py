"""GPU tests of the one-stream launch form: each dependent stage is a programmatic dependent launch of the stage
ahead of it (cusync_*_run_dependent), resident once every block of that stage is, in place of the reference's second
stream and wait kernel (cusync.h:277-283, cusync_device_defs.h:78-83).  Same stages, semaphore counts and results
as the stream form; the outputs are poisoned before every run, so a stage that ran ahead of its tiles shows as NaN."""
import numpy as np
import pytest

import oracle_lib as o
import cusync_b200 as cs
from cusync_b200 import _lib as L
from cusync_b200 import mlp as M
from cusync_b200.attention import AttentionBlock, PromptAttentionBlock

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-2


def _randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).half().cuda()


def _close(a, b):
    # Two runs of the same chain whose kernels sum K slices (or key blocks) in arrival order: an intermediate differs
    # by one half ulp here and there, and the next GEMM spreads that as absolute noise of about 1e-4 * max|Y| over
    # every output; elements under 5 % of the largest are therefore compared absolutely.
    return o.max_rel_err(a.cpu().numpy(), b.cpu().numpy(), 5e-2) <= 5e-3


def _same(a, b, exact):
    return torch.equal(a, b) if exact else _close(a, b)


@pytest.mark.parametrize("model,batch", [("gpt3", 1), ("gpt3", 64), ("gpt3", 600), ("gpt3", 1024), ("gpt3", 2048),
                                         ("llama", 512), ("llama", 2048)])
def test_mlp_layer_on_one_stream_equals_the_two_stream_layer(model, batch):
    dev = torch.device("cuda")
    x, w1, w2, v = M.make_inputs(model, batch, dev, seed=31)
    s = M.MLPShard(model, batch, x, w1, w2, v, policy="rowsync", single_grid=1)
    exact = s.split_k1 == 1 and s.split_k2 == 1 and s.tail_splits[:2] == (1, 1)
    ps, cs_, one = torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream()
    s.run_cusync(ps, cs_)
    torch.cuda.synchronize()
    h_ref, y_ref = s.h.clone(), s.y.clone()
    # the forms alternate on the same stages: iteration counts and the order of runs carry over between them
    for it in range(2, 8):
        s.h.fill_(float("nan")); s.y.fill_(float("nan"))
        torch.cuda.synchronize()
        if it % 3 == 0:
            s.run_cusync(ps, cs_)
        else:
            s.run_dependent(one)
        torch.cuda.synchronize()
        assert s.status_codes() == (0, 0)
        assert not torch.isnan(s.y.float()).any()
        assert _same(s.h, h_ref, exact) and _same(s.y, y_ref, exact)
        sems = s.producer_semaphores()
        assert (sems[: (batch + 127) // 128] == it * ((w1.shape[1] + s.tile_n1 - 1) // s.tile_n1)).all()
    # back to back without a host synchronisation: run r + 1 of one stream starts after run r has finished
    for _ in range(5):
        s.run_dependent(one)
    torch.cuda.synchronize()
    assert s.status_codes() == (0, 0)
    assert _same(s.y, y_ref, exact)
    s.destroy()


@pytest.mark.parametrize("n,h,w,c,convs,max_ctas", [
    (1, 56, 56, 64, 2, 0),     # both grids resident at once
    (8, 56, 56, 64, 2, 0),     # the consumer becomes resident as the producer's blocks retire
    (32, 56, 56, 64, 2, 0),
    (2, 28, 28, 64, 4, 6),     # chain of four, few blocks per stage
    (8, 56, 56, 64, 4, 0),     # chain of four sharing the SMs
    (4, 14, 14, 256, 2, 0),
    (32, 28, 28, 128, 2, 0),
])
def test_conv_chain_on_one_stream_equals_the_stream_form(n, h, w, c, convs, max_ctas):
    g = torch.Generator().manual_seed(70 + n)
    x = torch.randn((n, h, w, c), generator=g).half().cuda()
    filters = [(torch.randn((c, 3, 3, c), generator=g) * (2.0 / (9 * c)) ** 0.5).half().cuda() for _ in range(convs)]
    chain = cs.ConvChain(x, filters, relu=True, max_ctas=max_ctas)
    streams = [torch.cuda.Stream(priority=-1)] + [torch.cuda.Stream() for _ in range(convs - 1)]
    one = torch.cuda.Stream()
    chain.run_cusync(streams)
    torch.cuda.synchronize()
    refs = [t.clone() for t in chain.outputs]
    ref = o.conv2d_3x3_nhwc_f16(refs[-2].cpu().numpy(), filters[-1].cpu().numpy(), True)
    assert o.max_rel_err(refs[-1].cpu().numpy(), ref) <= TOL
    for it in range(2, 6):
        for out in chain.outputs:
            out.fill_(float("nan"))
        torch.cuda.synchronize()
        if it == 4:
            chain.run_cusync(streams)
        else:
            chain.run_dependent(one)
        torch.cuda.synchronize()
        assert chain.status_codes() == (0,) * convs
        for got, want in zip(chain.outputs, refs):
            assert torch.equal(got, want)
        for i in range(convs - 1):
            assert (chain.semaphores(i) == it).all()
    chain.destroy()


@pytest.mark.parametrize("B,S", [(1, 512), (4, 2048), (160, 128)])
def test_attention_block_on_one_stream_equals_the_stream_form(B, S):
    heads, H = 12, 12288
    x = _randn((B, H), 10)
    w_qkv = _randn((H, 3 * heads * 128), 11, 0.02)
    w_o = _randn((heads * 128, H), 12, 0.02)
    kc = _randn((B, S, heads, 128), 13)
    vc = _randn((B, S, heads, 128), 14)
    blk = AttentionBlock(x, w_qkv, kc, vc, w_o, heads)
    streams = (torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream())
    one = torch.cuda.Stream()
    blk.run(streams)
    torch.cuda.synchronize()
    y_ref = blk.y.clone()
    tiles_m = (B + 127) // 128
    for it in range(2, 5):
        blk.qkv.fill_(float("nan")); blk.o.fill_(float("nan")); blk.y.fill_(float("nan"))
        torch.cuda.synchronize()
        blk.run_dependent(one)
        torch.cuda.synchronize()
        assert blk.status_codes() == (0, 0, 0)
        assert not torch.isnan(blk.y.float()).any()
        assert _close(blk.y, y_ref)     # the QKV GEMM splits K and the attention kernel splits the keys
        assert (blk.s2.semaphores()[:tiles_m] == it).all()
    blk.destroy()


@pytest.mark.parametrize("B", [512, 1024])
def test_prompt_attention_chain_on_one_stream_equals_the_stream_form(B):
    heads, H = 12, 12288
    hd = heads * 128
    x = _randn((B, H), 20, 0.1)
    w_qkv = _randn((H, 3 * hd), 21, 0.02)
    w_o = _randn((hd, H), 22, 0.02)
    blk = PromptAttentionBlock(x, w_qkv, w_o, heads)
    streams = [torch.cuda.Stream(priority=-1)] + [torch.cuda.Stream() for _ in range(3)]
    one = torch.cuda.Stream()
    blk.run(streams)
    torch.cuda.synchronize()
    refs = [t.clone() for t in (blk.qkv, blk.s, blk.o, blk.y)]
    tiles_m = B // 128
    for it in range(2, 5):
        for t in (blk.qkv, blk.s, blk.o, blk.y):
            t.fill_(float("nan"))
        torch.cuda.synchronize()
        blk.run_dependent(one)
        torch.cuda.synchronize()
        assert blk.status_codes() == (0, 0, 0, 0)
        for got, want in zip((blk.qkv, blk.s, blk.o, blk.y), refs):
            assert not torch.isnan(got.float()).any()
            assert _close(got, want)
        assert (blk.stages[0].semaphores()[:3 * tiles_m] == 6 * it).all()
        assert (blk.stages[2].semaphores()[:tiles_m] == 6 * it).all()
    blk.destroy()


def test_a_plan_that_waits_for_nothing_is_refused():
    # a dependent launch is ordered against the kernel ahead of it by semaphore waits alone
    a = _randn((256, 512), 1)
    b = _randn((512, 512), 2)
    d = torch.empty((256, 512), dtype=torch.float16, device="cuda")
    desc = L.GemmDesc()
    desc.m, desc.n, desc.k = 256, 512, 512
    desc.a, desc.lda = a.data_ptr(), 512
    desc.b, desc.ldb = b.data_ptr(), 512
    desc.d, desc.ldd = d.data_ptr(), 512
    desc.b_layout = L.B_ROW_MAJOR_KN
    import ctypes as C
    plan = C.c_void_p()
    assert L.lib().cusync_gemm_plan_create(C.byref(plan), C.byref(desc)) == L.SUCCESS
    assert L.lib().cusync_gemm_run_dependent(plan, None) == L.ERROR_NOT_CONSUMER
    assert L.lib().cusync_gemm_run(plan, None) == L.SUCCESS
    torch.cuda.synchronize()
    assert o.max_rel_err(d.cpu().numpy(), o.gemm_f16(a.cpu().numpy(), b.cpu().numpy())) <= TOL
    L.lib().cusync_gemm_plan_destroy(plan)
