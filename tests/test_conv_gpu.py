"""GPU parity tests of the 3x3 convolution (implicit GEMM on the sm_100a kernel) and of the two-convolution
chain of BASELINE config 5, against the CPU oracle (orc_conv2d_3x3_nhwc_f16, which follows
cutlass::reference::host::Conv2dFprop as called at volta_conv2d/resnet.cu:708-720).
Tolerance: max relative error <= 1e-2 (resnet.cu:724), small elements compared absolutely."""
import numpy as np
import pytest

import oracle_lib as o
import cusync_b200 as cs
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-2


def _inputs(n, h, w, c, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((n, h, w, c), generator=g).half().cuda()
    # He-normal filters: sigma = sqrt(2 / fan_in), fan_in = 9 c
    f = (torch.randn((k, 3, 3, c), generator=g) * (2.0 / (9 * c)) ** 0.5).half().cuda()
    return x, f


@pytest.mark.parametrize("n,h,w,c,k", [
    (1, 56, 56, 64, 64),      # config 5, N = 1
    (2, 4, 56, 64, 64),       # two tiles per image: every tile touches a border
    (3, 28, 28, 64, 128),     # four image rows per tile, two N tiles
    (1, 8, 32, 128, 64),      # two channel chunks: 18 K blocks
    (2, 2, 128, 64, 64),      # one image row per tile
    (2, 14, 14, 256, 256),    # 14 x 14 layer (eval_resnet.py:12-17): 7 of the 9 rows that would fit, so tiles end with the image
    (3, 7, 7, 512, 128),      # 7 x 7 layer: one image (49 pixels) per tile, 72 K blocks
    (1, 5, 56, 64, 64),       # odd height: one image row per tile although two would fit
    (32, 14, 14, 256, 256),   # 64 M tiles: the library takes 128-channel N tiles (two rounds of 64-wide ones otherwise)
    (32, 28, 28, 128, 256),   # 224 M tiles: 256-channel N tiles
])
@pytest.mark.parametrize("relu", [False, True])
def test_conv3x3_matches_oracle(n, h, w, c, k, relu):
    x, f = _inputs(n, h, w, c, k, 1)
    y = torch.full((n, h, w, k), float("nan"), device="cuda", dtype=torch.half)
    conv = cs.Conv2dFprop()
    prob = cs.Conv2dProblemSize(n, h, w, c, k)
    if n == 32:
        assert prob.tile_n() == (128 if h == 14 else 256) and prob.grid()[0] == k // prob.tile_n()
    assert conv.initialize(None, prob, x, f, y, L.EPILOGUE_RELU if relu else L.EPILOGUE_NONE) == L.SUCCESS
    assert conv.run(torch.cuda.current_stream()) == L.SUCCESS
    torch.cuda.synchronize()
    ref = o.conv2d_3x3_nhwc_f16(x.cpu().numpy(), f.cpu().numpy(), relu)
    assert o.max_rel_err(y.cpu().numpy(), ref) <= TOL
    conv.destroy()


@pytest.mark.parametrize("kernel", [cs.Conv2dFprop.GENERAL, cs.Conv2dFprop.SLAB])
@pytest.mark.parametrize("n,h,w", [(1, 56, 56), (2, 4, 56), (3, 28, 28), (2, 6, 62)])
def test_both_conv_kernels_on_the_64_channel_layer(kernel, n, h, w):
    # the 64 -> 64 channel layer runs on the slab kernel by default; the general implicit-GEMM kernel must give the
    # same answer up to the oracle's tolerance (the two accumulate the taps in different orders)
    x, f = _inputs(n, h, w, 64, 64, 3)
    prob = cs.Conv2dProblemSize(n, h, w, 64, 64)
    y = torch.full((n, h, w, 64), float("nan"), device="cuda", dtype=torch.half)
    conv = cs.Conv2dFprop()
    assert conv.initialize(None, prob, x, f, y, L.EPILOGUE_RELU, kernel=kernel) == L.SUCCESS
    for _ in range(2):
        y.fill_(float("nan"))
        assert conv.run(torch.cuda.current_stream()) == L.SUCCESS
        torch.cuda.synchronize()
        ref = o.conv2d_3x3_nhwc_f16(x.cpu().numpy(), f.cpu().numpy(), True)
        assert o.max_rel_err(y.cpu().numpy(), ref) <= TOL
    conv.destroy()


def test_slab_kernel_is_refused_where_it_does_not_apply():
    x, f = _inputs(1, 8, 32, 128, 64, 4)
    y = torch.empty((1, 8, 32, 64), device="cuda", dtype=torch.half)
    conv = cs.Conv2dFprop()
    prob = cs.Conv2dProblemSize(1, 8, 32, 128, 64)          # two channel chunks
    assert conv.initialize(None, prob, x, f, y, kernel=cs.Conv2dFprop.SLAB) == L.ERROR_UNSUPPORTED
    assert conv.initialize(None, prob, x, f, y, kernel=7) == L.ERROR_INVALID_ARGUMENT
    assert conv.initialize(None, prob, x, f, y) == L.SUCCESS
    conv.destroy()


def test_conv_refuses_unsupported_shapes():
    x, f = _inputs(1, 56, 56, 64, 64, 2)
    y = torch.empty((1, 56, 56, 64), device="cuda", dtype=torch.half)
    conv = cs.Conv2dFprop()
    assert conv.initialize(None, cs.Conv2dProblemSize(1, 56, 56, 64, 64, r=5, s=5), x, f, y) == L.ERROR_UNSUPPORTED
    assert conv.initialize(None, cs.Conv2dProblemSize(1, 56, 56, 48, 64), x, f, y) == L.ERROR_UNSUPPORTED
    assert conv.initialize(None, cs.Conv2dProblemSize(1, 8, 200, 64, 64), x, f, y) == L.ERROR_UNSUPPORTED   # w > 128


@pytest.mark.parametrize("n", [1, 8, 32])
@pytest.mark.parametrize("max_ctas", [0, 5])
def test_config5_conv_chain_with_conv2dtilesync(n, max_ctas):
    # BASELINE config 5: X [N,56,56,64] ~ N(0,1), both filters [64,3,3,64] He-normal, ReLU after each conv,
    # producer TileSync / consumer Conv2DTileSync (resnet.cu:107-116, 773-782).
    h = w = 56
    c = k = 64
    x, f1 = _inputs(n, h, w, c, k, 10)
    _, f2 = _inputs(1, 2, 56, c, k, 11)
    y1 = torch.empty((n, h, w, k), device="cuda", dtype=torch.half)
    y2 = torch.empty((n, h, w, k), device="cuda", dtype=torch.half)
    prob = cs.Conv2dProblemSize(n, h, w, c, k)
    grid, tile_m = prob.grid(), prob.tile_m()
    assert grid == (1, 28 * n, 1) and tile_m == 112
    sync1 = cs.TileSync(cs.TransposeXYOrder, tile_m, 64)
    sync2 = cs.Conv2DTileSync(cs.TransposeXYOrder, 3, 3, tile_m, 64)
    prod = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), cs.NoSync(), sync1)
    cons = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), sync2, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    c1, c2 = cs.Conv2dFprop(), cs.Conv2dFprop()
    assert c1.initialize(prod, prob, x, f1, y1, L.EPILOGUE_RELU, max_ctas) == L.SUCCESS
    assert c2.initialize(cons, prob, y1, f2, y2, L.EPILOGUE_RELU, max_ctas) == L.SUCCESS
    ps, cst = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    r1 = o.conv2d_3x3_nhwc_f16(x.cpu().numpy(), f1.cpu().numpy(), True)
    r2 = o.conv2d_3x3_nhwc_f16(r1, f2.cpu().numpy(), True)
    opol = o.policy(o.TILESYNC, 1, tile_m, 64, 1, 1)
    torch.cuda.synchronize()
    for it in range(1, 4):
        y1.fill_(float("nan")); y2.fill_(float("nan")); torch.cuda.synchronize()   # poison
        assert c1.run(ps) == L.SUCCESS
        assert prod.invokeWaitKernel(cst) == L.SUCCESS
        assert c2.run(cst) == L.SUCCESS
        torch.cuda.synchronize()
        assert prod.status().code == 0 and cons.status().code == 0
        assert o.max_rel_err(y1.cpu().numpy(), r1) <= TOL
        assert o.max_rel_err(y2.cpu().numpy(), r2) <= TOL
        exp, oob = o.producer_semaphores(opol, grid, tile_m, 64, 0, it)
        assert oob == 0 and (prod.semaphores() == exp).all()
        prod.incrementIter(); cons.incrementIter()
    c1.destroy(); c2.destroy(); prod.destroy(); cons.destroy()


@pytest.mark.parametrize("c", [64, 128])      # the slab kernel and the general kernel
def test_consumer_skips_its_probes_once_the_producer_kernel_has_finished(c):
    # The producer's blocks count themselves finished after their posts; a consumer block that finds the count of
    # this run's producer launch reached knows that every tile is there and stops probing semaphores.  Shown by
    # taking the semaphores away after the producer has finished: the consumer completes all the same.  In the next
    # run, with no producer launched, the count of run 1 must NOT be taken for run 2's: the consumer times out.
    import ctypes as C
    n, h, w = 2, 28, 28
    x, f1 = _inputs(n, h, w, c, c, 90)
    _, f2 = _inputs(1, 4, 28, c, c, 91)
    y1 = torch.empty((n, h, w, c), device="cuda", dtype=torch.half)
    y2 = torch.full((n, h, w, c), float("nan"), device="cuda", dtype=torch.half)
    prob = cs.Conv2dProblemSize(n, h, w, c, c)
    grid, tile_m, tile_n = prob.grid(), prob.tile_m(), prob.tile_n()
    prod = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), cs.NoSync(), cs.TileSync(cs.TransposeXYOrder, tile_m, tile_n))
    cons = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), cs.Conv2DTileSync(cs.TransposeXYOrder, 3, 3, tile_m, tile_n),
                      cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    cons.set_timeout_ns(30e6)
    c1, c2 = cs.Conv2dFprop(), cs.Conv2dFprop()
    assert c1.initialize(prod, prob, x, f1, y1, L.EPILOGUE_RELU, 0) == L.SUCCESS
    assert c2.initialize(cons, prob, y1, f2, y2, L.EPILOGUE_RELU, 0) == L.SUCCESS
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    view = L.StageView()
    # before any producer launch the consumer has no count to look at
    assert L.lib().cusync_stage_get_view(cons._h, C.byref(view)) == L.SUCCESS and not view.prod_finished
    assert c1.run(stream) == L.SUCCESS
    torch.cuda.synchronize()
    assert L.lib().cusync_stage_get_view(cons._h, C.byref(view)) == L.SUCCESS
    assert view.prod_finished and view.prod_finish_target == c1.num_ctas()
    count = grid[0] * grid[1]
    assert (prod.semaphores() == 1).all()
    assert L.lib().cusync_stage_get_view(prod._h, C.byref(view)) == L.SUCCESS
    assert L.lib().cusync_stream_write_values(C.c_void_p(view.sems_post), count, 0, sp) == L.SUCCESS   # take them away
    assert c2.run(stream) == L.SUCCESS
    torch.cuda.synchronize()
    assert cons.status().code == 0
    r1 = o.conv2d_3x3_nhwc_f16(x.cpu().numpy(), f1.cpu().numpy(), True)
    assert o.max_rel_err(y1.cpu().numpy(), r1) <= TOL
    assert o.max_rel_err(y2.cpu().numpy(), o.conv2d_3x3_nhwc_f16(y1.cpu().numpy(), f2.cpu().numpy(), True)) <= TOL
    # run 2 without its producer: nothing to go by but the semaphores, which stay below 2
    assert L.lib().cusync_stream_write_values(C.c_void_p(view.sems_post), count, 1, sp) == L.SUCCESS
    prod.incrementIter(); cons.incrementIter()
    assert L.lib().cusync_stage_get_view(cons._h, C.byref(view)) == L.SUCCESS and not view.prod_finished
    y2.fill_(float("nan"))
    assert c2.run(stream) == L.SUCCESS
    torch.cuda.synchronize()
    st = cons.status()
    assert st.code == L.ERROR_TIMEOUT and st.expected == 2 and st.seen == 1
    assert torch.isnan(y2.float()).all()
    c1.destroy(); c2.destroy(); prod.destroy(); cons.destroy()


def test_a_consumer_tile_waits_for_its_halo_neighbours_at_every_channel_chunk():
    # 128 channels in producer tiles of 64: two channel chunks along the consumer's K walk.  The host stands in for
    # the producer and posts every semaphore but ONE, the second chunk of row tile 3.  The consumer tiles of rows
    # 2, 3 and 4 all read image rows of that producer tile (own rows or halo), so all three must give up (bounded
    # wait) without writing; the other rows complete.  A consumer that only looked at its neighbours' first chunk
    # would write rows 2 and 4 from unfinished input.
    import ctypes as C
    n, h, w, c = 1, 28, 28, 128
    x, f = _inputs(n, h, w, c, c, 77)
    y = torch.full((n, h, w, c), float("nan"), device="cuda", dtype=torch.half)
    prob = cs.Conv2dProblemSize(n, h, w, c, c)
    grid, tile_m, tile_n = prob.grid(), prob.tile_m(), prob.tile_n()
    assert grid == (2, 7, 1) and tile_m == 112 and tile_n == 64
    prod = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), cs.NoSync(), cs.TileSync(cs.TransposeXYOrder, tile_m, tile_n))
    cons = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), cs.Conv2DTileSync(cs.TransposeXYOrder, 3, 3, tile_m, tile_n),
                      cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    cons.set_timeout_ns(30e6)
    conv = cs.Conv2dFprop()
    assert conv.initialize(cons, prob, x, f, y, L.EPILOGUE_RELU, 0) == L.SUCCESS
    # which semaphore the producer tile (row tile 3, chunk 1) posts: row offset 3 * tile_m, column offset tile_n
    opol = o.policy(o.TILESYNC, o.ORDER_TRANSPOSE_XY, tile_m, tile_n, 1, 1)
    missing = int(o.consumer_tile_waits(opol, grid, 3 * tile_m, 2 * tile_n, tile_n, 1)[0][1])
    view = L.StageView()
    assert L.lib().cusync_stage_get_view(prod._h, C.byref(view)) == L.SUCCESS
    count = grid[0] * grid[1]
    stream = torch.cuda.current_stream()
    for i in range(count):
        if i != missing:
            assert L.lib().cusync_stream_write_values(C.c_void_p(view.sems_post + 4 * i), 1, 1,
                                                      C.c_void_p(stream.cuda_stream)) == L.SUCCESS
    assert conv.run(stream) == L.SUCCESS
    torch.cuda.synchronize()
    st = cons.status()
    assert st.code == L.ERROR_TIMEOUT and st.sem_index == missing and st.expected == 1 and st.seen == 0
    ref = o.conv2d_3x3_nhwc_f16(x.cpu().numpy(), f.cpu().numpy(), True)
    got = y.float().cpu().numpy()
    rows = h // 7                                   # image rows per tile
    for t in range(7):
        part = got[0, t * rows:(t + 1) * rows]
        if t in (2, 3, 4):
            assert np.isnan(part).all(), "row tile %d was written although its input was not complete" % t
        else:
            assert not np.isnan(part).any()
            assert o.max_rel_err(part.astype(np.float16), ref[0, t * rows:(t + 1) * rows]) <= TOL
    conv.destroy(); prod.destroy(); cons.destroy()


@pytest.mark.parametrize("n,h,w,c,convs,max_ctas", [
    (1, 56, 56, 64, 2, 0),     # config 5, N = 1: both grids resident at once, no wait kernel
    (8, 56, 56, 64, 2, 0),     # config 5, N = 8: wait kernel before the consumer
    (2, 28, 28, 64, 4, 6),     # vgg.cu-style chain of four, few blocks per stage, general-shape kernel rows
    (1, 8, 32, 128, 3, 0),     # two channel chunks: the implicit-GEMM path between the stages
    (4, 28, 28, 128, 2, 0),    # the reference's other layer sizes (eval_resnet.py:12-17, 497-498): 128 channels, 28 x 28
    (4, 14, 14, 256, 2, 0),    # 256 channels, 14 x 14
    (8, 7, 7, 512, 2, 0),      # 512 channels, 7 x 7
    (2, 14, 14, 256, 4, 0),    # vgg.cu-style chain of four at 256 channels (vgg.cu:104-119)
    (32, 14, 14, 256, 2, 0),   # N tiles of 128 channels: Conv2DTileSync over producer tiles two channel chunks wide
    (40, 14, 14, 256, 2, 0),   # N tiles of 256 channels (80 M tiles: one round instead of two)
])
def test_conv_chain_driver(n, h, w, c, convs, max_ctas):
    # cusync_conv_chain_*: the library's own driver for the chain (resnet.cu / vgg.cu flow)
    g = torch.Generator().manual_seed(40 + n)
    x = torch.randn((n, h, w, c), generator=g).half().cuda()
    filters = [(torch.randn((c, 3, 3, c), generator=g) * (2.0 / (9 * c)) ** 0.5).half().cuda() for _ in range(convs)]
    chain = cs.ConvChain(x, filters, relu=True, max_ctas=max_ctas)
    tile_n = L.lib().cusync_conv2d_default_tile_n(n, h, w, c, c)
    assert tile_n == {32: 128, 40: 256}.get(n, 64)
    blocks = n * (h // L.lib().cusync_conv2d_tile_rows_hw(h, w)) * (c // tile_n)
    sms = L.lib().cusync_b200_sm_count()
    # left to choose: half of the device per stage in chains of three or more 64-channel convolutions, else all of it
    per_stage = min(blocks, max_ctas if max_ctas else (sms // 2 if (c == 64 and convs >= 3) else sms))
    assert chain.uses_wait_kernels == (per_stage * convs > sms)
    streams = [torch.cuda.Stream(priority=-1)] + [torch.cuda.Stream() for _ in range(convs - 1)]
    for it in range(1, 4):
        for out in chain.outputs:
            out.fill_(float("nan"))                    # a consumer that reads ahead of its producer sees NaN
        torch.cuda.synchronize()
        chain.run_cusync(streams)
        torch.cuda.synchronize()
        assert chain.status_codes() == (0,) * convs
        # every convolution against the oracle fed with the activation the GPU itself produced before it
        # (an end-to-end reference would also compare the stages' different fp16 roundings)
        acts = [x] + chain.outputs
        for i, f in enumerate(filters):
            ref = o.conv2d_3x3_nhwc_f16(acts[i].cpu().numpy(), f.cpu().numpy(), True)
            assert not np.isnan(acts[i + 1].float().cpu().numpy()).any()
            assert o.max_rel_err(acts[i + 1].cpu().numpy(), ref) <= TOL
        for i in range(convs - 1):
            assert (chain.semaphores(i) == it).all()   # every tile posted once per run
    for out in chain.outputs:
        out.fill_(float("nan"))
    chain.run_stream_ordered(torch.cuda.current_stream())
    torch.cuda.synchronize()
    ref = o.conv2d_3x3_nhwc_f16(chain.outputs[-2].cpu().numpy(), filters[-1].cpu().numpy(), True)
    assert o.max_rel_err(chain.y.cpu().numpy(), ref) <= TOL
    chain.destroy()


@pytest.mark.parametrize("n", [1, 8])
def test_conv_chain_replayed_from_a_cuda_graph(n):
    # run_cusync_replayable recorded once (capture on the producer stream, the consumer stream forked by the
    # driver's event and joined here), then replayed: every replay starts from reset stages.
    h = w = 56
    c = 64
    g = torch.Generator().manual_seed(50 + n)
    x = torch.randn((n, h, w, c), generator=g).half().cuda()
    filters = [(torch.randn((c, 3, 3, c), generator=g) * (2.0 / (9 * c)) ** 0.5).half().cuda() for _ in range(2)]
    chain = cs.ConvChain(x, filters, relu=True)
    cap, side = torch.cuda.Stream(), torch.cuda.Stream()
    chain.run_cusync([cap, side])          # warm-up outside the capture (module load, attribute calls)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=cap):
        chain.run_cusync_replayable([cap, side])
        cap.wait_stream(side)
    r1 = o.conv2d_3x3_nhwc_f16(x.cpu().numpy(), filters[0].cpu().numpy(), True)
    for _ in range(3):
        for out in chain.outputs:
            out.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert chain.status_codes() == (0, 0)
        assert o.max_rel_err(chain.outputs[0].cpu().numpy(), r1) <= TOL
        r2 = o.conv2d_3x3_nhwc_f16(chain.outputs[0].cpu().numpy(), filters[1].cpu().numpy(), True)
        assert not np.isnan(chain.y.float().cpu().numpy()).any()
        assert o.max_rel_err(chain.y.cpu().numpy(), r2) <= TOL
        assert (chain.semaphores(0) == 1).all()
    del graph
    chain.destroy()
