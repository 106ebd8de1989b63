"""GPU parity tests of the MLP shard driver (cusync_mlp_*): GPT-3 (GELU) and LLaMA (fused SwiGLU dual GEMM)
layers, overlapped and stream-ordered, against the CPU oracle chain with the intermediate rounded to fp16
(mlp.cu:334-341).  Large batches are checked on 64 sampled rows carried through the whole chain."""
import numpy as np
import pytest

import oracle_lib as o
from cusync_b200 import mlp as M
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-2


def _reference(model, x, w1, w2, v, rows):
    xs = x[rows].cpu().numpy()
    if model == "gpt3":
        h = o.gemm_f16(xs, w1.cpu().numpy(), o.EPI_GELU_ERF)
    else:
        h = o.gemm_dual_silu_mul_f16(xs, w1.cpu().numpy(), v.cpu().numpy())
    return h, o.gemm_f16(h, w2.cpu().numpy())


def _exact_chain(model, x, w1, w2, v, rows):
    """The same layer in float64 without any intermediate rounding: what both the GPU chain and the oracle's
    chain approximate."""
    import math
    xs = x[rows].cpu().numpy().astype(np.float64)
    a = xs @ w1.cpu().numpy().astype(np.float64)
    if model == "gpt3":
        h = 0.5 * a * (1.0 + np.vectorize(math.erf)(a / math.sqrt(2.0)))
    else:
        h = a / (1.0 + np.exp(-a)) * (xs @ v.cpu().numpy().astype(np.float64))
    return (h @ w2.cpu().numpy().astype(np.float64)).astype(np.float16)


def _check_final_output(y_gpu, y_oracle, y_exact, what):
    o.check_final_output(y_gpu, y_oracle, y_exact, what, TOL)


@pytest.mark.parametrize("model,batch,ffn", [
    ("gpt3", 1, None), ("gpt3", 64, None), ("gpt3", 256, None), ("gpt3", 512, None), ("gpt3", 1024, None),
    ("gpt3", 2048, None),
    ("llama", 1, None), ("llama", 64, None), ("llama", 512, None), ("llama", 2048, None),
    ("llama", 256, M.LLAMA_FFN_REFERENCE),     # the reference's d = 2816 (mlp.cu:247-250)
])
@pytest.mark.parametrize("policy", ["rowsync", "tilesync"])
def test_mlp_layer_matches_oracle_on_up_to_64_sampled_rows(model, batch, ffn, policy):
    dev = torch.device("cuda")
    x, w1, w2, v = M.make_inputs(model, batch, dev, seed=3, ffn=ffn)
    s = M.MLPShard(model, batch, x, w1, w2, v, policy=policy)
    rows = torch.arange(0, batch, max(batch // 64, 1))[:64]
    href, yref = _reference(model, x, w1, w2, v, rows)
    yexact = _exact_chain(model, x, w1, w2, v, rows)
    ps, cs_ = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    torch.cuda.synchronize()
    for it in range(1, 3):
        s.h.fill_(float("nan")); s.y.fill_(float("nan")); torch.cuda.synchronize()
        s.run_cusync(ps, cs_)
        torch.cuda.synchronize()
        assert s.status_codes() == (0, 0)
        hg = s.h[rows].cpu().numpy()
        assert o.max_rel_err(hg, href) <= TOL
        # second GEMM on its own: the oracle fed with the intermediate the GPU actually produced
        assert o.max_rel_err(s.y[rows].cpu().numpy(), o.gemm_f16(hg, w2.cpu().numpy())) <= TOL
        # end to end: the final output against the oracle's own chain and against the exact chain
        _check_final_output(s.y[rows].cpu().numpy(), yref, yexact, "%s B=%d %s run %d" % (model, batch, policy, it))
        assert not torch.isnan(s.y).any()
        sems = s.producer_semaphores()
        tiles_n = (s.ffn + s.tile_n1 - 1) // s.tile_n1
        tiles_m = (batch + 127) // 128
        if policy == "rowsync":
            assert (sems[:tiles_m] == tiles_n * it).all()
        else:
            assert (sems[:tiles_n * tiles_m] == it).all()
    # the stream-ordered arm computes the same thing: sampled rows against the oracle, and EVERY element of H and
    # Y against the synchronised arm, bit for bit (without split-K the accumulation order is fixed)
    h_sync, y_sync = s.h.clone(), s.y.clone()
    s.h.fill_(float("nan")); s.y.fill_(float("nan"))
    s.run_stream_ordered(cs_)
    torch.cuda.synchronize()
    _check_final_output(s.y[rows].cpu().numpy(), yref, yexact, "%s B=%d stream-ordered" % (model, batch))
    # (... and with the same K slices, if any, for the tiles of a last partial round in both arms)
    if s.split_k1 == 1 and s.split_k2 == 1 and s.tail_splits[:2] == s.tail_splits[2:]:
        assert torch.equal(s.h, h_sync) and torch.equal(s.y, y_sync)
    else:
        assert torch.allclose(s.y.float(), y_sync.float(), rtol=1e-2, atol=1e-3)
    s.destroy()


@pytest.mark.parametrize("batch,max_ctas", [(1024, 128), (600, 0), (64, 0)])
def test_output_rows_can_be_consumed_block_by_block(batch, max_ctas):
    # post_rows: the second GEMM posts one RowSync semaphore per 128-row tile of Y; cusync_mlp_wait_rows lets
    # another stream (in a tensor-parallel layer: the all-reduce) take row blocks as they complete.  Here the
    # other stream copies each block right behind its wait; a block taken too early would carry the NaN poison.
    from cusync_b200 import tp
    dev = torch.device("cuda")
    x, w1, w2, v = M.make_inputs("gpt3", batch, dev, seed=5)
    s = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync", post_rows=True, max_ctas=max_ctas)
    ps, cs_, side = torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream()
    tiles = (batch + 127) // 128
    snap = torch.empty_like(s.y)
    for it in range(1, 4):
        s.h.fill_(float("nan")); s.y.fill_(float("nan")); snap.fill_(float("nan")); torch.cuda.synchronize()
        s.run_cusync(ps, cs_)
        per = max(tiles // 3, 1)
        for first in range(0, tiles, per):
            n = min(per, tiles - first)
            s.wait_rows(first, n, side)
            with torch.cuda.stream(side):
                snap[first * 128:(first + n) * 128].copy_(s.y[first * 128:(first + n) * 128], non_blocking=True)
        torch.cuda.synchronize()
        assert s.status_codes() == (0, 0)
        assert not torch.isnan(snap.float()).any()
        assert torch.equal(snap, s.y)
        # semaphore counts: every row tile of Y was posted once per column tile and run
        st = L.lib().cusync_mlp_stage(s._h, 1)
        sems = np.zeros(tiles, dtype=np.uint32)
        import ctypes as C
        assert L.lib().cusync_stage_read_semaphores(st, sems.ctypes.data_as(C.c_void_p), tiles) == L.SUCCESS
        assert (sems == it * ((M.GPT3_HIDDEN + s.tile_n2 - 1) // s.tile_n2)).all()
    # the helper used by the multi-GPU bench, on a world of one rank: waits only
    g = tp.TensorParallelGroup("nccl", dev)
    s.y.fill_(float("nan")); torch.cuda.synchronize()
    s.run_cusync(ps, cs_)
    g.all_reduce_rows_overlapped(s, side, 4)
    side.synchronize()
    assert not torch.isnan(s.y.float()).any()
    torch.cuda.synchronize()
    # without post_rows the call is refused
    s2 = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync")
    with pytest.raises(L.CuSyncError):
        s2.wait_rows(0, 1, side)
    s2.destroy(); s.destroy()


@pytest.mark.parametrize("batch", [64, 600, 1024])
def test_input_rows_can_arrive_while_the_layer_runs(batch):
    # x_rows: the first GEMM waits per 128-row tile of X on a semaphore that the caller's stream writes behind the
    # copy that brings those rows (stream memory operations: neither needs an SM).  The rows come from pinned host
    # memory on a stream that first idles for a while, so the layer is running, on poisoned X, well before they
    # land.  A tile multiplied too early would carry NaN.
    dev = torch.device("cuda")
    x, w1, w2, v = M.make_inputs("gpt3", batch, dev, seed=6)
    x_host = x.cpu().pin_memory()
    ref = M.MLPShard("gpt3", batch, x.clone(), w1, w2, v, policy="rowsync")
    ref.run_stream_ordered(torch.cuda.current_stream()); torch.cuda.synchronize()
    s = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync", x_rows=True, post_rows=True)
    ps, cs_, feed = torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream()
    tiles = (batch + 127) // 128
    for it in range(1, 4):
        x.fill_(float("nan")); s.y.fill_(float("nan")); torch.cuda.synchronize()
        # Third run: the layer is launched BEFORE its rows are even submitted (the posts count per tile, so either
        # order feeds the same run).  No delay kernel then: it would need an SM that the waiting GEMM holds.
        launch_first = it == 3
        if launch_first:
            s.run_cusync(ps, cs_)
        else:
            with torch.cuda.stream(feed):
                torch.cuda._sleep(1_000_000)        # about half a millisecond before the first row arrives
        for first in reversed(range(tiles)) if it == 2 else range(tiles):   # any order will do
            r0, r1 = first * 128, min(batch, (first + 1) * 128)
            with torch.cuda.stream(feed):
                x[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
            s.post_x_rows(first, 1, feed)
        if not launch_first:
            s.run_cusync(ps, cs_)
        torch.cuda.synchronize()
        assert s.status_codes() == (0, 0)
        assert not torch.isnan(s.y.float()).any()
        # (split-K batches add their slices in arrival order: equal up to fp32 rounding, not bit for bit)
        assert torch.allclose(s.y.float(), ref.y.float(), rtol=1e-2, atol=1e-3)
        if s.split_k1 == 1 and s.split_k2 == 1 and s.tail_splits[:2] == ref.tail_splits[2:]:
            assert torch.equal(s.y, ref.y)
    with pytest.raises(L.CuSyncError):
        ref.post_x_rows(0, 1, feed)
    s.destroy(); ref.destroy()


def test_timeout_upstream_releases_the_stream_waits_downstream():
    # X never arrives (x_rows, no post): the first GEMM's bounded wait runs out, the second GEMM's does too, and
    # neither posts.  The stream waits behind the second GEMM's row semaphores (cusync_mlp_wait_rows, the form an
    # all-reduce or a copy of Y hangs on) have no bound of their own: the GEMM that gives up sets a bit in every
    # semaphore of its stage that satisfies them, so the stream drains and the host finds the timeout records.
    import ctypes as C
    import time
    dev = torch.device("cuda")
    batch = 512
    x, w1, w2, v = M.make_inputs("gpt3", batch, dev, seed=8)
    s = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync", x_rows=True, post_rows=True)
    lib = L.lib()
    prod, cons = lib.cusync_mlp_stage(s._h, 0), lib.cusync_mlp_stage(s._h, 1)
    assert lib.cusync_stage_set_timeout_ns(prod, int(300e6)) == L.SUCCESS    # waits for X: 0.3 s
    assert lib.cusync_stage_set_timeout_ns(cons, int(30e6)) == L.SUCCESS     # waits for H: 30 ms, gives up first
    ps, cs_, side = torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream()
    tiles = (batch + 127) // 128
    flag = torch.zeros(1, device=dev)
    torch.cuda.synchronize()
    s.run_cusync(ps, cs_)
    s.wait_rows(0, tiles, side)
    with torch.cuda.stream(side):
        flag.add_(1.0)
    deadline = time.time() + 20.0
    while not side.query() and time.time() < deadline:
        time.sleep(0.01)
    drained = side.query()
    if not drained:
        # do not leave the stream stuck for the rest of the session: release it by hand, then fail
        view = L.StageView()
        lib.cusync_stage_get_view(cons, C.byref(view))
        lib.cusync_stream_write_values(view.sems_post, tiles, 0x40000000, torch.cuda.Stream().cuda_stream)
    torch.cuda.synchronize()
    assert drained, "stream wait behind a GEMM that gave up was not released"
    assert flag.item() == 1.0
    assert s.status_codes() == (L.ERROR_TIMEOUT, L.ERROR_TIMEOUT)
    sems = np.zeros(tiles, dtype=np.uint32)
    assert lib.cusync_stage_read_semaphores(cons, sems.ctypes.data_as(C.c_void_p), tiles) == L.SUCCESS
    assert (sems & 0x40000000).all()
    s.destroy()


@pytest.mark.parametrize("batch,max_ctas", [(600, 0), (1024, 0), (2048, 0), (1024, 12)])
@pytest.mark.parametrize("policy", ["rowsync", "tilesync"])
def test_single_grid_layer_equals_the_two_launch_layer(batch, max_ctas, policy):
    # run_cusync as ONE persistent grid (the default where both GEMMs run on CTA pairs) against the reference-shaped
    # form, one launch per GEMM with a wait kernel in between: same H and Y bit for bit, same semaphore counts.
    dev = torch.device("cuda")
    x, w1, w2, v = M.make_inputs("gpt3", batch, dev, seed=9)
    one = M.MLPShard("gpt3", batch, x, w1, w2, v, policy=policy, max_ctas=max_ctas, single_grid=2)
    two = M.MLPShard("gpt3", batch, x, w1, w2, v, policy=policy, max_ctas=max_ctas, single_grid=1)
    assert one.single_grid and not two.single_grid
    with pytest.raises(L.CuSyncError):
        M.MLPShard("gpt3", 64, x[:64].contiguous(), w1, w2, v, policy=policy, single_grid=2)   # not on CTA pairs
    ps, cs_ = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    for it in range(1, 4):
        for s in (one, two):
            s.h.fill_(float("nan")); s.y.fill_(float("nan"))
        torch.cuda.synchronize()
        one.run_cusync(ps, cs_)
        cs_.synchronize()                       # the result is complete on the consumer stream
        assert not torch.isnan(one.y.float()).any()
        two.run_cusync(ps, cs_)
        torch.cuda.synchronize()
        assert one.status_codes() == (0, 0) and two.status_codes() == (0, 0)
        assert torch.equal(one.h, two.h) and torch.equal(one.y, two.y)
        assert (one.producer_semaphores() == two.producer_semaphores()).all()
    one.destroy(); two.destroy()


@pytest.mark.parametrize("batch", [640, 2048])
def test_llama_layer_as_one_grid_equals_the_two_launch_layer(batch):
    # the fused SwiGLU GEMM on CTA pairs followed by the second GEMM, as ONE persistent grid (the table's choice from
    # nine row tiles on) against one launch per GEMM: same H and Y bit for bit, same semaphore counts
    dev = torch.device("cuda")
    x, w1, w2, v = M.make_inputs("llama", batch, dev, seed=19)
    one = M.MLPShard("llama", batch, x, w1, w2, v, policy="rowsync", single_grid=2)
    two = M.MLPShard("llama", batch, x, w1, w2, v, policy="rowsync", single_grid=1)
    assert one.single_grid and not two.single_grid
    assert M.MLPShard("llama", 2048, *M.make_inputs("llama", 2048, dev, seed=1), policy="rowsync").single_grid
    ps, cs_ = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    for it in range(1, 4):
        for s in (one, two):
            s.h.fill_(float("nan")); s.y.fill_(float("nan"))
        torch.cuda.synchronize()
        one.run_cusync(ps, cs_)
        cs_.synchronize()
        assert not torch.isnan(one.y.float()).any()
        two.run_cusync(ps, cs_)
        torch.cuda.synchronize()
        assert one.status_codes() == (0, 0) and two.status_codes() == (0, 0)
        assert torch.equal(one.h, two.h) and torch.equal(one.y, two.y)
        assert (one.producer_semaphores() == two.producer_semaphores()).all()
    one.destroy(); two.destroy()
