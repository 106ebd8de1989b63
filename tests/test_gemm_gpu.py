"""GPU parity tests of the sm_100a GEMM kernels, called through the C ABI and
checked against the CPU oracle on the same seeded inputs.

Tolerance: max relative error <= 1e-2 on the final output (fp16 in, fp32
accumulate), elements below 1e-2 * max|ref| compared absolutely.  Semaphore
counts and tile order are compared bit-exactly."""
import numpy as np
import pytest

import oracle_lib as o
import cusync_b200 as cs
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-2


def _rand(shape, seed, scale=1.0, dist="uniform"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dist == "uniform":
        t = (torch.rand(shape, generator=g) * 2 - 1) * scale
    else:
        t = torch.randn(shape, generator=g) * scale
    return t.half().cuda()


def _gemm(a, b, epi=L.EPILOGUE_NONE, tile_n=0, b_layout=L.B_ROW_MAJOR_KN, max_ctas=0, b2=None, stage=None,
          cta_pair=0, split_k=1, runs=1, tail_split=0):
    M, K = a.shape
    N = b.shape[1]
    d = torch.full((M, N), float("nan"), device="cuda", dtype=torch.half)
    if b_layout == L.B_ROW_MAJOR_NK:
        bdev = b.t().contiguous()
        b2dev = b2.t().contiguous() if b2 is not None else None
    else:
        bdev, b2dev = b, b2
    g = cs.Gemm()
    rc = g.initialize(cs.GemmArguments(stage, (M, N, K), a, bdev, d, epilogue=epi, ref_b2=b2dev, b_layout=b_layout,
                                       tile_n=tile_n, max_ctas=max_ctas, cta_pair=cta_pair,
                                       split_k_slices=split_k, tail_split=tail_split))
    assert rc == L.SUCCESS, L.ERROR_NAMES[rc]
    for _ in range(runs):
        d.fill_(float("nan"))
        assert g.run(stream=torch.cuda.current_stream()) == L.SUCCESS
        torch.cuda.synchronize()
    n = g.num_ctas()
    g.destroy()
    return d, n


@pytest.mark.parametrize("M,N,K,tile_n", [
    (256, 1024, 1024, 128),    # config 1 shape
    (128, 256, 64, 256),       # single K block
    (1, 512, 256, 64),         # one row (decode batch 1)
    (64, 384, 512, 64),
    (300, 1000, 520, 128),     # ragged M, N and K tails
    (129, 72, 136, 64),        # N and K barely over one granule
    (512, 2752, 1024, 128),    # LLaMA ffn width: 21.5 tiles of 128
    (1024, 2048, 1024, 256),
    (512, 1536, 1024, 192),    # 192-wide tiles: three 64-column chunks, accumulators 384 of 512 TMEM columns
    (300, 1000, 520, 192),     # ... with ragged edges
])
@pytest.mark.parametrize("layout", [L.B_ROW_MAJOR_KN, L.B_ROW_MAJOR_NK])
def test_gemm_matches_oracle(M, N, K, tile_n, layout):
    a = _rand((M, K), 1)
    b = _rand((K, N), 2)
    d, _ = _gemm(a, b, tile_n=tile_n, b_layout=layout)
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy())
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("epi,oepi", [(L.EPILOGUE_GELU_ERF, o.EPI_GELU_ERF), (L.EPILOGUE_RELU, o.EPI_RELU)])
@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_gemm_epilogues(epi, oepi, tile_n):
    a = _rand((200, 768), 3, dist="normal")
    b = _rand((768, 512), 4, scale=0.05, dist="normal")
    d, _ = _gemm(a, b, epi=epi, tile_n=tile_n)
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy(), oepi)
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("M,N,K,tile_n", [(256, 512, 512, 128), (70, 2752, 256, 128), (33, 192, 1024, 64)])
@pytest.mark.parametrize("layout", [L.B_ROW_MAJOR_KN, L.B_ROW_MAJOR_NK])
def test_dual_gemm_silu_mul(M, N, K, tile_n, layout):
    a = _rand((M, K), 5, dist="normal")
    b1 = _rand((K, N), 6, scale=0.05, dist="normal")
    b2 = _rand((K, N), 7, scale=0.05, dist="normal")
    d, _ = _gemm(a, b1, epi=L.EPILOGUE_SILU_MUL_DUAL, tile_n=tile_n, b_layout=layout, b2=b2)
    ref = o.gemm_dual_silu_mul_f16(a.cpu().numpy(), b1.cpu().numpy(), b2.cpu().numpy())
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("M,N,K", [
    (256, 256, 64),       # one pair, one K block
    (512, 1024, 1024),
    (384, 512, 576),      # odd number of 128-row tiles: the last pair's second CTA has no rows; odd K chunks
    (1000, 960, 320),     # ragged M, N not a multiple of the tile
    (2048, 2048, 1024),
])
@pytest.mark.parametrize("layout", [L.B_ROW_MAJOR_KN, L.B_ROW_MAJOR_NK])
def test_cta_pair_gemm_matches_oracle(M, N, K, layout):
    a = _rand((M, K), 50)
    b = _rand((K, N), 51)
    d, n = _gemm(a, b, tile_n=256, b_layout=layout, cta_pair=2)
    assert n % 2 == 0
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy())
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("M,N,K,max_ctas", [(256, 256, 128, 0), (640, 2752, 256, 0), (1024, 1280, 1024, 6), (2048, 2752, 512, 0)])
@pytest.mark.parametrize("layout", [L.B_ROW_MAJOR_KN, L.B_ROW_MAJOR_NK])
def test_dual_gemm_silu_mul_on_cta_pairs(M, N, K, max_ctas, layout):
    # The fused SwiGLU GEMM on CTA pairs: the pair's 256-column MMA is [A B | A B2] of one 128-column output tile (the
    # leader CTA loads the B half, its peer the B2 half); the epilogue stores SiLU(A B) (.) (A B2).  N = 2752 (LLaMA's
    # ffn shard) ends in a ragged tile; M = 640 is an odd number of row tiles; few clusters and repeated runs.
    a = _rand((M, K), 60, dist="normal")
    b = _rand((K, N), 61, scale=0.05, dist="normal")
    b2 = _rand((K, N), 62, scale=0.05, dist="normal")
    d, n = _gemm(a, b, epi=L.EPILOGUE_SILU_MUL_DUAL, tile_n=128, b_layout=layout, b2=b2, cta_pair=2, max_ctas=max_ctas,
                 runs=2)
    assert n % 2 == 0
    ref = o.gemm_dual_silu_mul_f16(a.cpu().numpy(), b.cpu().numpy(), b2.cpu().numpy())
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL
    # the same numbers as the one-CTA kernel gives (same K walk per element)
    d1, _ = _gemm(a, b, epi=L.EPILOGUE_SILU_MUL_DUAL, tile_n=128, b_layout=layout, b2=b2, cta_pair=1)
    assert torch.equal(d, d1)
    # K slices (uniform or for the last partial round) have no finaliser for the two halves: refused
    for kw in (dict(tail_split=2), dict(split_k_slices=2)):
        g = cs.Gemm()
        assert g.initialize(cs.GemmArguments(None, (M, N, K), a, b, d, ref_b2=b2, epilogue=L.EPILOGUE_SILU_MUL_DUAL,
                                             tile_n=128, cta_pair=2, **kw)) == L.ERROR_UNSUPPORTED


def test_cta_pair_gemm_epilogue_and_few_clusters():
    a = _rand((1024, 512), 52, dist="normal")
    b = _rand((512, 2048), 53, scale=0.05, dist="normal")
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy(), o.EPI_GELU_ERF)
    # 4 pair rows x 8 column tiles = 32 pair tiles on 3 clusters, run three times (ticket counter re-arms)
    d = torch.empty((1024, 2048), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(None, (1024, 2048, 512), a, b, d, epilogue=L.EPILOGUE_GELU_ERF, tile_n=256,
                                         max_ctas=6, cta_pair=2, split_k_slices=1)) == L.SUCCESS
    assert g.num_ctas() == 6
    for _ in range(3):
        d.fill_(float("nan"))
        assert g.run(stream=torch.cuda.current_stream()) == L.SUCCESS
        torch.cuda.synchronize()
        assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL
    g.destroy()


@pytest.mark.parametrize("M,N,K,max_ctas,tail_split,expect", [
    (1024, 2048, 2048, 6, 3, 3),     # 32 pair tiles on 3 clusters: 2 left over, cut into 3 slices each
    (1024, 2048, 2048, 6, 0, 1),     # left to the library: no split (it measured slower)
    (1000, 960, 1024, 6, 2, 2),      # ragged edges; 16 pair tiles on 3 clusters: 1 left over, 2 slices forced
    (1024, 2048, 2048, 6, 1, 1),     # switched off
    (512, 1024, 1024, 4, 4, 1),      # 8 pair tiles on 2 clusters: nothing left over, nothing to split
])
@pytest.mark.parametrize("layout", [L.B_ROW_MAJOR_KN, L.B_ROW_MAJOR_NK])
def test_tail_split_gemm_matches_oracle(M, N, K, max_ctas, tail_split, expect, layout):
    a = _rand((M, K), 61, dist="normal")
    b = _rand((K, N), 62, scale=0.05, dist="normal")
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy(), o.EPI_GELU_ERF)
    bdev = b.t().contiguous() if layout == L.B_ROW_MAJOR_NK else b
    d = torch.empty((M, N), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(None, (M, N, K), a, bdev, d, epilogue=L.EPILOGUE_GELU_ERF, b_layout=layout,
                                         tile_n=256, max_ctas=max_ctas, cta_pair=2, split_k_slices=1,
                                         tail_split=tail_split)) == L.SUCCESS
    assert g.tail_split() == expect
    for _ in range(3):           # the workspace and the arrival counters re-arm themselves
        d.fill_(float("nan"))
        assert g.run(stream=torch.cuda.current_stream()) == L.SUCCESS
        torch.cuda.synchronize()
        assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL
    g.destroy()


def test_cta_pair_refuses_what_it_cannot_do():
    # K (and N of [k,n] weights) must be whole 64-element chunks for the pair kernel; left to choose, the
    # library falls back to one CTA per tile and still computes the right answer.
    a = _rand((256, 520), 56); b = _rand((520, 1000), 57)
    d = torch.empty((256, 1000), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(None, (256, 1000, 520), a, b, d, tile_n=256, cta_pair=2)) == L.ERROR_UNSUPPORTED
    d2, _ = _gemm(a, b, tile_n=256, cta_pair=0)
    assert o.max_rel_err(d2.cpu().numpy(), o.gemm_f16(a.cpu().numpy(), b.cpu().numpy())) <= TOL
    a = _rand((256, 256), 54); b = _rand((256, 256), 55)
    d = torch.empty((256, 256), device="cuda", dtype=torch.half)
    assert g.initialize(cs.GemmArguments(None, (256, 256, 256), a, b, d, tile_n=128, cta_pair=2)) == L.ERROR_UNSUPPORTED
    assert g.initialize(cs.GemmArguments(None, (256, 256, 256), a, b, d, epilogue=L.EPILOGUE_SILU_MUL_DUAL, ref_b2=b,
                                         tile_n=256, cta_pair=2)) == L.ERROR_UNSUPPORTED


@pytest.mark.parametrize("M,N,K,tile_n,split,pair", [
    (1, 1024, 4096, 256, 4, 1),       # decode batch 1: one row, four K slices per tile
    (64, 1536, 6144, 256, 0, 1),      # slices chosen by the library
    (100, 1000, 2048 + 64, 128, 3, 1),  # ragged N, K not a multiple of the slices
    (128, 512, 2048, 64, 2, 1),
    (256, 512, 4096, 256, 4, 2),      # CTA pairs with split-K
    (384, 768, 3072, 256, 3, 2),      # odd row-tile count: the last pair's second CTA only keeps the barriers going
])
@pytest.mark.parametrize("epi,oepi", [(L.EPILOGUE_NONE, o.EPI_NONE), (L.EPILOGUE_GELU_ERF, o.EPI_GELU_ERF)])
def test_split_k_gemm_matches_oracle(M, N, K, tile_n, split, pair, epi, oepi):
    a = _rand((M, K), 60, dist="normal")
    b = _rand((K, N), 61, scale=0.03, dist="normal")
    # three runs on one plan: the workspace and the slice counters must come back to zero by themselves
    d, _ = _gemm(a, b, epi=epi, tile_n=tile_n, cta_pair=pair, split_k=split, runs=3)
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy(), oepi)
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL


def test_split_k_defaults_and_limits():
    assert cs.Gemm.default_split_k(64, 6144, 12288, L.EPILOGUE_GELU_ERF) >= 2
    assert cs.Gemm.default_split_k(2048, 6144, 12288, L.EPILOGUE_GELU_ERF) == 1
    assert cs.Gemm.default_split_k(64, 2752, 8192, L.EPILOGUE_SILU_MUL_DUAL) == 1
    a = _rand((64, 4096), 62); b = _rand((4096, 256), 63)
    d = torch.empty((64, 256), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(None, (64, 256, 4096), a, b, d, epilogue=L.EPILOGUE_SILU_MUL_DUAL, ref_b2=b,
                                         tile_n=64, split_k_slices=2)) == L.ERROR_UNSUPPORTED


def test_chain_with_split_k_on_both_gemms():
    # one row of tiles (M = 96): producer 4 column tiles x 3 K slices, consumer 2 column tiles x 2 K slices.
    # Only the block that brings a tile's last slice posts, so every semaphore still counts one per run.
    M, K1, N1, N2 = 96, 3072, 1024, 512
    a = _rand((M, K1), 70, dist="normal")
    w1 = _rand((K1, N1), 71, scale=0.03, dist="normal")
    w2 = _rand((N1, N2), 72, scale=0.03, dist="normal")
    h = torch.empty((M, N1), device="cuda", dtype=torch.half)
    y = torch.empty((M, N2), device="cuda", dtype=torch.half)
    for policy in ("row", "tile"):
        grid1, grid2 = (4, 1, 3), (2, 1, 2)
        sync = cs.RowSync(128, 4) if policy == "row" else cs.TileSync(cs.TransposeXYOrder, 128, 256)
        prod = cs.CuStage(cs.TransposeXYOrder, grid1, (1, 1, 1), cs.NoSync(), sync)
        cons = cs.CuStage(cs.TransposeXYOrder, grid2, (1, 1, 1), sync, cs.NoSync())
        assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
        g1, g2 = cs.Gemm(), cs.Gemm()
        assert g1.initialize(cs.GemmArguments(prod, (M, N1, K1), a, w1, h, epilogue=L.EPILOGUE_GELU_ERF, tile_n=256,
                                              split_k_slices=3)) == L.SUCCESS
        assert g2.initialize(cs.GemmArguments(cons, (M, N2, N1), h, w2, y, tile_n=256, split_k_slices=2)) == L.SUCCESS
        ps, cst = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
        href = o.gemm_f16(a.cpu().numpy(), w1.cpu().numpy(), o.EPI_GELU_ERF)
        yref = o.gemm_f16(href, w2.cpu().numpy())
        torch.cuda.synchronize()
        for it in range(1, 4):
            h.fill_(float("nan")); y.fill_(float("nan")); torch.cuda.synchronize()
            g1.run(True, None, ps); prod.invokeWaitKernel(cst); g2.run(True, None, cst)
            torch.cuda.synchronize()
            assert prod.status().code == 0 and cons.status().code == 0
            assert o.max_rel_err(h.cpu().numpy(), href) <= TOL
            assert o.max_rel_err(y.cpu().numpy(), yref) <= TOL
            sems = prod.semaphores()
            if policy == "row":
                assert sems[0] == 4 * it and (sems[1:] == 0).all()
            else:
                assert (sems[:4] == it).all() and (sems[4:] == 0).all()
            prod.incrementIter(); cons.incrementIter()
        g1.destroy(); g2.destroy(); prod.destroy(); cons.destroy()


def test_persistent_scheduler_with_few_blocks_and_repeated_runs():
    # 64 tiles on 3 blocks: every block loops over many tickets; the ticket counter must re-arm itself.
    a = _rand((1024, 512), 8)
    b = _rand((512, 1024), 9)
    ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy())
    d = torch.empty((1024, 1024), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(None, (1024, 1024, 512), a, b, d, tile_n=128, max_ctas=3, split_k_slices=1)) == L.SUCCESS
    assert g.num_ctas() == 3
    for _ in range(3):
        d.fill_(float("nan"))
        assert g.run(stream=torch.cuda.current_stream()) == L.SUCCESS
        torch.cuda.synchronize()
        assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL
    g.destroy()


def test_linearity_at_full_gpt3_width():
    # Size-independent property at BASELINE width (K = 12288, N = 6144): scaling A by 2 (exact in fp16)
    # scales every output by exactly 2, and a row permutation of A permutes the rows of D bit-exactly.
    M, K, N = 256, 12288, 6144
    a = _rand((M, K), 10, dist="normal", scale=0.5)
    b = _rand((K, N), 11, scale=0.02, dist="normal")
    # (24 pair tiles, each cut into 3 K slices: the slices' partial sums are added in slice order whichever
    # finishes last, so the results stay bit-reproducible)
    d1, _ = _gemm(a, b, tile_n=256, tail_split=3)
    d2, _ = _gemm(a * 2, b, tile_n=256, tail_split=3)
    # exact wherever the result is a normal fp16 number (subnormal outputs round differently after doubling)
    normal = d1.abs() >= 2.0 ** -13
    assert torch.equal(d2[normal], (d1 * 2)[normal])
    assert (d2.float() - 2 * d1.float()).abs().max().item() <= 2.0 ** -23
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(0)).cuda()
    d3, _ = _gemm(a[perm].contiguous(), b, tile_n=256, tail_split=3)
    assert torch.equal(d3, d1[perm])
    # 64 sampled rows carried through the oracle
    rows = torch.arange(0, M, 4)
    ref = o.gemm_f16(a[rows].cpu().numpy(), b.cpu().numpy())
    assert o.max_rel_err(d1[rows].cpu().numpy(), ref) <= TOL


def _chain(policy_name, M, N1, K1, N2, tile_n1, tile_n2, iters, opts=0, epi1=L.EPILOGUE_NONE, max_ctas=0,
           wait_kernel=True, seed=20, cta_pair=0, tail_split=0, single_grid=False):
    a = _rand((M, K1), seed, dist="normal")
    w1 = _rand((K1, N1), seed + 1, scale=0.03, dist="normal")
    w2 = _rand((N1, N2), seed + 2, scale=0.03, dist="normal")
    h = torch.empty((M, N1), device="cuda", dtype=torch.half)
    y = torch.empty((M, N2), device="cuda", dtype=torch.half)
    grid1 = cs.gemm_tiled_shape(M, N1, 128, tile_n1)
    grid2 = cs.gemm_tiled_shape(M, N2, 128, tile_n2)
    if policy_name == "row":
        sync = cs.RowSync(128, grid1[0])
        opol = o.policy(o.ROWSYNC, 1, 128, tile_n1, grid1[0], 1)
    else:
        sync = cs.TileSync(cs.TransposeXYOrder, 128, tile_n1)
        opol = o.policy(o.TILESYNC, 1, 128, tile_n1, 1, 1)
    prod = cs.CuStage(cs.TransposeXYOrder, grid1, (1, 1, 1), cs.NoSync(), sync, opts)
    cons = cs.CuStage(cs.TransposeXYOrder, grid2, (1, 1, 1), sync, cs.NoSync(), opts)
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    g1, g2 = cs.Gemm(), cs.Gemm()
    assert g1.initialize(cs.GemmArguments(prod, (M, N1, K1), a, w1, h, epilogue=epi1, tile_n=tile_n1,
                                          max_ctas=max_ctas, cta_pair=cta_pair, split_k_slices=1,
                                          tail_split=tail_split)) == L.SUCCESS
    assert g2.initialize(cs.GemmArguments(cons, (M, N2, N1), h, w2, y, tile_n=tile_n2, max_ctas=max_ctas,
                                          cta_pair=cta_pair, split_k_slices=1, tail_split=tail_split)) == L.SUCCESS
    if tail_split > 1:
        assert g1.tail_split() == tail_split and g2.tail_split() == tail_split
    ps, cst = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    oepi = {L.EPILOGUE_NONE: o.EPI_NONE, L.EPILOGUE_GELU_ERF: o.EPI_GELU_ERF}[epi1]
    href = o.gemm_f16(a.cpu().numpy(), w1.cpu().numpy(), oepi)
    yref = o.gemm_f16(href, w2.cpu().numpy())
    torch.cuda.synchronize()
    for it in range(1, iters + 1):
        # poison: a consumer that reads ahead of its producer sees NaN
        h.fill_(float("nan")); y.fill_(float("nan"))
        torch.cuda.synchronize()
        if single_grid:
            assert cs.Gemm.run_chain(g1, g2, ps) == L.SUCCESS
        else:
            assert g1.run(True, None, ps) == L.SUCCESS
            if wait_kernel:
                assert prod.invokeWaitKernel(cst) == L.SUCCESS
            assert g2.run(True, None, cst) == L.SUCCESS
        torch.cuda.synchronize()
        assert prod.status().code == 0 and cons.status().code == 0
        assert o.max_rel_err(h.cpu().numpy(), href) <= TOL
        assert o.max_rel_err(y.cpu().numpy(), yref) <= TOL
        # bit-exact semaphore counts against the oracle's simulation of `it` runs
        exp, oob = o.producer_semaphores(opol, grid1, 128, tile_n1, opts & L.OPT_NO_ATOMIC_ADD, it)
        assert oob == 0
        assert (prod.semaphores() == exp).all()
        prod.incrementIter(); cons.incrementIter()
    # bit-exact schedule buffer
    exp_order, bad = o.tile_order(1, grid1)
    assert bad == 0 and (prod.tile_order() == exp_order).all()
    g1.destroy(); g2.destroy(); prod.destroy(); cons.destroy()


@pytest.mark.parametrize("policy", ["row", "tile"])
def test_config1_two_dependent_gemms(policy):
    # BASELINE config 1: M=256, K=N=1024, 128x128 tiles, U[-1,1] inputs
    M = 256
    a = _rand((M, 1024), 0)
    b = _rand((1024, 1024), 1)
    dd = _rand((1024, 1024), 2)
    c = torch.empty((M, 1024), device="cuda", dtype=torch.half)
    e = torch.empty((M, 1024), device="cuda", dtype=torch.half)
    grid = cs.gemm_tiled_shape(M, 1024, 128, 128)
    assert grid == (8, 2, 1)
    sync = cs.TileSync(cs.TransposeXYOrder, 128, 128) if policy == "tile" else cs.RowSync(128, grid[0])
    prod = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), cs.NoSync(), sync)
    cons = cs.CuStage(cs.TransposeXYOrder, grid, (1, 1, 1), sync, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    g1, g2 = cs.Gemm(), cs.Gemm()
    assert g1.initialize(cs.GemmArguments(prod, (M, 1024, 1024), a, b, c, tile_n=128, split_k_slices=1)) == L.SUCCESS
    assert g2.initialize(cs.GemmArguments(cons, (M, 1024, 1024), c, dd, e, tile_n=128, split_k_slices=1)) == L.SUCCESS
    ps, cst = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    cref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy())
    eref = o.gemm_f16(cref, dd.cpu().numpy())
    for it in range(1, 4):
        c.fill_(float("nan")); e.fill_(float("nan")); torch.cuda.synchronize()
        g1.run(True, None, ps); prod.invokeWaitKernel(cst); g2.run(True, None, cst)
        torch.cuda.synchronize()
        assert o.max_rel_err(c.cpu().numpy(), cref) <= TOL
        assert o.max_rel_err(e.cpu().numpy(), eref) <= TOL
        sems = prod.semaphores()
        if policy == "tile":
            assert (sems == it).all()
        else:
            assert (sems[:2] == 8 * it).all() and (sems[2:] == 0).all()
        prod.incrementIter(); cons.incrementIter()
    g1.destroy(); g2.destroy(); prod.destroy(); cons.destroy()


@pytest.mark.parametrize("policy", ["row", "tile"])
@pytest.mark.parametrize("opts", [0, L.OPT_NO_ATOMIC_ADD])
def test_chain_many_tiles_few_blocks(policy, opts):
    if policy == "row" and opts:
        pytest.skip("NoAtomicAdd needs one poster per semaphore (mlp.cu:9-14)")
    # producer 8x4 = 32 tiles, consumer 4x4 tiles of 256, only 6 blocks each: consumers really wait
    _chain(policy, 512, 1024, 512, 1024, 128, 256, iters=3, opts=opts, max_ctas=6)


def test_chain_gelu_mismatched_tile_widths():
    # GPT-3-like slice: producer tile 256 wide with fused GELU, consumer K walk crosses producer tiles
    _chain("tile", 384, 1536, 1024, 768, 256, 128, iters=2, epi1=L.EPILOGUE_GELU_ERF)
    _chain("row", 384, 1536, 1024, 768, 256, 128, iters=2, epi1=L.EPILOGUE_GELU_ERF)


@pytest.mark.parametrize("policy", ["row", "tile"])
@pytest.mark.parametrize("opts", [0, L.OPT_NO_ATOMIC_ADD])
def test_chain_with_cta_pairs(policy, opts):
    if policy == "row" and opts:
        pytest.skip("NoAtomicAdd needs one poster per semaphore (mlp.cu:9-14)")
    # both GEMMs on CTA pairs, few clusters so consumers really wait; M = 640 -> 5 row tiles (odd)
    _chain(policy, 640, 1024, 512, 1024, 256, 256, iters=3, opts=opts, max_ctas=4, cta_pair=2)
    _chain(policy, 512, 1536, 1024, 768, 256, 256, iters=2, opts=opts, epi1=L.EPILOGUE_GELU_ERF, cta_pair=2)


@pytest.mark.parametrize("policy", ["row", "tile"])
def test_chain_with_tail_split_on_both_gemms(policy):
    # 3 pair rows x 4 column tiles = 12 pair tiles on 5 clusters: the last 2 tiles of either GEMM are cut
    # into K slices; a split producer tile posts once (from the pair that adds the last slice), a split
    # consumer tile waits slice by slice.
    _chain(policy, 640, 1024, 1024, 1024, 256, 256, iters=3, max_ctas=10, cta_pair=2, tail_split=2)
    _chain(policy, 768, 1024, 2048, 1024, 256, 256, iters=2, max_ctas=10, cta_pair=2, tail_split=4,
           epi1=L.EPILOGUE_GELU_ERF)


def test_chain_without_wait_kernel_small_grids():
    # AvoidWaitKernel (cusync.h:61-62): both grids fit one wave
    _chain("tile", 256, 512, 256, 512, 128, 128, iters=2, opts=L.OPT_AVOID_WAIT_KERNEL, wait_kernel=False)


def test_consumer_times_out_instead_of_hanging():
    # Nothing ever posts: the consumer GEMM must return with a timeout record, and the stage must be
    # reusable after reset.  The bound is 30 ms.
    M, N, K = 128, 128, 256
    a = _rand((M, K), 30); b = _rand((K, N), 31)
    d = torch.zeros((M, N), device="cuda", dtype=torch.half)
    sync = cs.TileSync(cs.TransposeXYOrder, 128, 128)
    prod = cs.CuStage(cs.TransposeXYOrder, (2, 1, 1), (1, 1, 1), cs.NoSync(), sync)
    cons = cs.CuStage(cs.TransposeXYOrder, (1, 1, 1), (1, 1, 1), sync, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    cons.set_timeout_ns(30e6)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(cons, (M, N, K), a, b, d, tile_n=128, split_k_slices=1)) == L.SUCCESS
    assert g.run(stream=torch.cuda.current_stream()) == L.SUCCESS
    torch.cuda.synchronize()      # returns: no hang
    st = cons.status()
    assert st.code == L.ERROR_TIMEOUT and st.where == 1 and st.expected == 1 and st.seen == 0 and st.sem_index == 0
    cons.reset(); prod.reset(); torch.cuda.synchronize()
    assert cons.status().code == 0
    # after reset the pair works: run the producer-side post by hand via a real producer GEMM
    x = _rand((M, 64), 32); w = _rand((64, 256), 33)
    g1 = cs.Gemm()
    assert g1.initialize(cs.GemmArguments(prod, (M, 256, 64), x, w, a, tile_n=128, split_k_slices=1)) == L.SUCCESS
    s2 = torch.cuda.Stream()
    g1.run(stream=torch.cuda.current_stream()); prod.invokeWaitKernel(s2); g.run(stream=s2)
    torch.cuda.synchronize()
    assert cons.status().code == 0
    ref = o.gemm_f16(o.gemm_f16(x.cpu().numpy(), w.cpu().numpy()), b.cpu().numpy())
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL
    g.destroy(); g1.destroy(); prod.destroy(); cons.destroy()


def test_stage_grid_must_match_the_tile_grid():
    a = _rand((256, 256), 40); b = _rand((256, 256), 41)
    d = torch.empty((256, 256), device="cuda", dtype=torch.half)
    st = cs.CuStage(cs.TransposeXYOrder, (3, 2, 1), (1, 1, 1), cs.NoSync(), cs.TileSync(cs.TransposeXYOrder, 128, 128))
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(st, (256, 256, 256), a, b, d, tile_n=128, split_k_slices=1)) == L.ERROR_INVALID_ARGUMENT
    # an unlinked consumer is refused too
    c = cs.CuStage(cs.TransposeXYOrder, (2, 2, 1), (1, 1, 1), cs.TileSync(cs.TransposeXYOrder, 128, 128), cs.NoSync())
    assert g.initialize(cs.GemmArguments(c, (256, 256, 256), a, b, d, tile_n=128, split_k_slices=1)) == L.ERROR_NOT_INITIALIZED
    st.destroy(); c.destroy()


def test_link_error_codes():
    s = cs.TileSync(cs.TransposeXYOrder, 128, 128)
    prod = cs.CuStage(cs.TransposeXYOrder, (2, 2, 1), (1, 1, 1), cs.NoSync(), s)
    cons = cs.CuStage(cs.TransposeXYOrder, (2, 2, 1), (1, 1, 1), s, cs.NoSync())
    # cusync.h:289-298
    assert cs.CuSync.setProducerConsumerPair(cons, cons) == L.ERROR_NOT_PRODUCER
    assert cs.CuSync.setProducerConsumerPair(prod, prod) == L.ERROR_NOT_CONSUMER
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    assert cons.invokeWaitKernel(None) == L.ERROR_NOT_PRODUCER
    prod.destroy(); cons.destroy()


def test_stream_memory_operations_wait_and_post():
    # cusync_stream_wait_values / cusync_stream_write_values: a stream holds until semaphores reach a value, and
    # another stream's write releases it, without any kernel of the library.  The posting side is submitted
    # first (behind a delay), as a stream wait must only wait for work that is already submitted: two streams
    # may share a hardware queue, and a wait at its head would keep a later post from ever being issued.
    sems = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros(1024, device="cuda")
    a, b = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    lib = L.lib()
    with torch.cuda.stream(b):
        torch.cuda._sleep(100_000_000)                     # some tens of milliseconds
    assert lib.cusync_stream_write_values(sems.data_ptr(), 3, 3, b.cuda_stream) == L.SUCCESS
    assert lib.cusync_stream_write_values(sems.data_ptr() + 12, 1, 5, b.cuda_stream) == L.SUCCESS   # >= counts
    assert lib.cusync_stream_wait_values(sems.data_ptr(), 4, 3, a.cuda_stream) == L.SUCCESS
    with torch.cuda.stream(a):
        out.add_(1.0)
        seen = sems.clone()                                # what the stream sees once its wait lets it through
    torch.cuda.synchronize()
    assert (out == 1.0).all() and sems.tolist() == [3, 3, 3, 5]
    assert seen.tolist() == [3, 3, 3, 5]                   # held until every post had landed
    assert lib.cusync_stream_wait_values(None, 1, 1, a.cuda_stream) == L.ERROR_NOT_INITIALIZED
    # more semaphores than one batched operation carries: posted first, then waited for
    many = torch.zeros(150, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert lib.cusync_stream_write_values(many.data_ptr(), 150, 7, b.cuda_stream) == L.SUCCESS
    assert lib.cusync_stream_wait_values(many.data_ptr(), 150, 7, b.cuda_stream) == L.SUCCESS
    torch.cuda.synchronize()
    assert many.tolist() == [7] * 150


@pytest.mark.parametrize("policy", ["row", "tile"])
def test_chain_with_the_wait_as_a_stream_operation(policy):
    # Optimizations.StreamWait: invokeWaitKernel enqueues a stream wait on the producer's "blocks started" word
    _chain(policy, 640, 1024, 512, 1024, 256, 256, iters=3, opts=cs.Optimizations.StreamWait, max_ctas=4, cta_pair=2)
    _chain(policy, 256, 1024, 1024, 1024, 128, 128, iters=2, opts=cs.Optimizations.StreamWait)


def test_strided_tile_sync_chain_of_the_unfused_llama_layer():
    # The reference's LLaMA chain (mlp.cu:103-109, 762-792): the first GEMM writes [X W1 | X V] side by side
    # (N = 2 d) and posts StridedSync<TransposeXY, d, TM, TN, 2>: column tiles j and j + d / TN share semaphore j,
    # which reaches 2 per run; the second GEMM reads the first d columns through the leading dimension 2 d and
    # waits for 2.  d = 2816 as in the reference, 128-wide producer tiles: 44 column tiles, 22 semaphores per row.
    M, K1, d, N2, TN = 300, 512, 2816, 768, 128
    a = _rand((M, K1), 80, dist="normal")
    w1v = _rand((K1, 2 * d), 81, scale=0.05, dist="normal")
    w2 = _rand((d, N2), 82, scale=0.03, dist="normal")
    buf = torch.empty((M, 2 * d), device="cuda", dtype=torch.half)
    y = torch.empty((M, N2), device="cuda", dtype=torch.half)
    grid1 = cs.gemm_tiled_shape(M, 2 * d, 128, TN)
    grid2 = cs.gemm_tiled_shape(M, N2, 128, 256)
    assert grid1 == (44, 3, 1)
    sync = cs.StridedTileSync(cs.TransposeXYOrder, d, 128, TN, 2)
    prod = cs.CuStage(cs.TransposeXYOrder, grid1, (1, 1, 1), cs.NoSync(), sync)     # two posters per semaphore: atomics
    cons = cs.CuStage(cs.TransposeXYOrder, grid2, (1, 1, 1), sync, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    g1, g2 = cs.Gemm(), cs.Gemm()
    # few blocks, so that the second GEMM really waits for column tiles of both halves
    assert g1.initialize(cs.GemmArguments(prod, (M, 2 * d, K1), a, w1v, buf, tile_n=TN, max_ctas=8,
                                          split_k_slices=1)) == L.SUCCESS
    assert g2.initialize(cs.GemmArguments(cons, (M, N2, d), buf[:, :d], w2, y, tile_n=256, max_ctas=8,
                                          split_k_slices=1, cta_pair=1)) == L.SUCCESS
    ref1 = o.gemm_f16(a.cpu().numpy(), w1v.cpu().numpy())
    yref = o.gemm_f16(np.ascontiguousarray(ref1[:, :d]), w2.cpu().numpy())
    opol = o.policy(o.STRIDEDSYNC, o.ORDER_TRANSPOSE_XY, 128, TN, 0, 0, p0=d, p1=2)
    ps, cst = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    torch.cuda.synchronize()
    for it in range(1, 4):
        buf.fill_(float("nan")); y.fill_(float("nan")); torch.cuda.synchronize()
        assert g1.run(True, None, ps) == L.SUCCESS
        assert prod.invokeWaitKernel(cst) == L.SUCCESS
        assert g2.run(True, None, cst) == L.SUCCESS
        torch.cuda.synchronize()
        assert prod.status().code == 0 and cons.status().code == 0
        assert o.max_rel_err(buf.cpu().numpy(), ref1) <= TOL
        assert o.max_rel_err(y.cpu().numpy(), yref) <= TOL
        sems = prod.semaphores().reshape(3, 44)
        assert (sems[:, :22] == 2 * it).all() and (sems[:, 22:] == 0).all()
        exp, oob = o.producer_semaphores(opol, grid1, 128, TN, 0, it)
        assert oob == 0 and (prod.semaphores() == exp).all()
        prod.incrementIter(); cons.incrementIter()
    g1.destroy(); g2.destroy(); prod.destroy(); cons.destroy()


@pytest.mark.parametrize("kernel", ["split_k", "tail_split"])
def test_consumer_k_slices_that_begin_inside_a_producer_tile_wait_for_it(kernel):
    # TileSync, producer tiles 256 wide, consumer K = 1024 cut into three slices: the slices begin at K offsets
    # 0, 384 and 768, the second one in the middle of producer tile 1.  Its first K block has to wait for that
    # tile although 384 is not a multiple of the producer's tile width.  The producer is slow (long K, few
    # blocks) and H is poisoned, so a slice that read ahead would put NaN into Y.
    M, K1, N1, N2 = 512, 8192, 1024, 1024
    a = _rand((M, K1), 90, dist="normal", scale=0.5)
    w1 = _rand((K1, N1), 91, scale=0.02, dist="normal")
    w2 = _rand((N1, N2), 92, scale=0.03, dist="normal")
    h = torch.empty((M, N1), device="cuda", dtype=torch.half)
    y = torch.empty((M, N2), device="cuda", dtype=torch.half)
    split = 3 if kernel == "split_k" else 1
    grid1 = cs.gemm_tiled_shape(M, N1, 128, 256)
    grid2 = cs.gemm_tiled_shape(M, N2, 128, 256, split)
    sync = cs.TileSync(cs.TransposeXYOrder, 128, 256)
    prod = cs.CuStage(cs.TransposeXYOrder, grid1, (1, 1, 1), cs.NoSync(), sync)
    cons = cs.CuStage(cs.TransposeXYOrder, grid2, (1, 1, 1), sync, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    g1, g2 = cs.Gemm(), cs.Gemm()
    assert g1.initialize(cs.GemmArguments(prod, (M, N1, K1), a, w1, h, tile_n=256, max_ctas=4, cta_pair=1,
                                          split_k_slices=1)) == L.SUCCESS
    if kernel == "split_k":     # one CTA per tile, three K slices per tile
        assert g2.initialize(cs.GemmArguments(cons, (M, N2, N1), h, w2, y, tile_n=256, max_ctas=12, cta_pair=1,
                                              split_k_slices=3)) == L.SUCCESS
    else:                       # CTA pairs: 8 pair tiles on 3 clusters, the 2 left over cut into 3 slices each
        assert g2.initialize(cs.GemmArguments(cons, (M, N2, N1), h, w2, y, tile_n=256, max_ctas=6, cta_pair=2,
                                              split_k_slices=1, tail_split=3)) == L.SUCCESS
        assert g2.tail_split() == 3
    href = o.gemm_f16(a.cpu().numpy(), w1.cpu().numpy())
    yref = o.gemm_f16(href, w2.cpu().numpy())
    ps, cst = torch.cuda.Stream(priority=-1), torch.cuda.Stream()
    torch.cuda.synchronize()
    for it in range(1, 4):
        h.fill_(float("nan")); y.fill_(float("nan")); torch.cuda.synchronize()
        assert g1.run(True, None, ps) == L.SUCCESS
        assert prod.invokeWaitKernel(cst) == L.SUCCESS
        assert g2.run(True, None, cst) == L.SUCCESS
        torch.cuda.synchronize()
        assert prod.status().code == 0 and cons.status().code == 0
        assert not torch.isnan(y.float()).any()
        assert o.max_rel_err(y.cpu().numpy(), yref) <= TOL
        assert (prod.semaphores() == it).all()
        prod.incrementIter(); cons.incrementIter()
    g1.destroy(); g2.destroy(); prod.destroy(); cons.destroy()


def test_policies_built_for_another_tile_shape_are_refused():
    a = _rand((256, 512), 95); b = _rand((512, 512), 96)
    d = torch.empty((256, 512), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    # producer: 128-wide policy tiles on a 256-wide kernel tile would post past the end of the semaphore array
    st = cs.CuStage(cs.TransposeXYOrder, (2, 2, 1), (1, 1, 1), cs.NoSync(), cs.TileSync(cs.TransposeXYOrder, 128, 128))
    assert g.initialize(cs.GemmArguments(st, (256, 512, 512), a, b, d, tile_n=256, cta_pair=1,
                                         split_k_slices=1)) == L.ERROR_INVALID_ARGUMENT
    st.destroy()
    # consumer: a block loads 128 rows but a 64-row policy tile covers only the first half of them
    narrow = cs.TileSync(cs.TransposeXYOrder, 64, 128)
    prod = cs.CuStage(cs.TransposeXYOrder, (4, 4, 1), (1, 1, 1), cs.NoSync(), narrow)
    cons = cs.CuStage(cs.TransposeXYOrder, (2, 2, 1), (1, 1, 1), narrow, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    assert g.initialize(cs.GemmArguments(cons, (256, 512, 512), a, b, d, tile_n=256, cta_pair=1,
                                         split_k_slices=1)) == L.ERROR_INVALID_ARGUMENT
    prod.destroy(); cons.destroy()
    # consumer: policy tiles that are not whole 64-element K blocks
    odd = cs.TileSync(cs.TransposeXYOrder, 128, 96)
    prod = cs.CuStage(cs.TransposeXYOrder, (6, 2, 1), (1, 1, 1), cs.NoSync(), odd)
    cons = cs.CuStage(cs.TransposeXYOrder, (2, 2, 1), (1, 1, 1), odd, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, cons) == L.SUCCESS
    assert g.initialize(cs.GemmArguments(cons, (256, 512, 512), a, b, d, tile_n=256, cta_pair=1,
                                         split_k_slices=1)) == L.ERROR_INVALID_ARGUMENT
    prod.destroy(); cons.destroy()


@pytest.mark.parametrize("policy", ["row", "tile"])
def test_chain_as_one_persistent_grid(policy):
    # cusync_gemm_run_chain: both GEMMs in one grid of CTA pairs drawing from one ticket counter.  Few clusters,
    # so pairs go from producer units straight on to consumer units and really wait; odd row-tile count;
    # with and without tail splits; three runs (the shared counter re-arms itself).
    _chain(policy, 640, 1024, 512, 1024, 256, 256, iters=3, max_ctas=4, cta_pair=2, single_grid=True)
    _chain(policy, 512, 1536, 1024, 768, 256, 256, iters=2, epi1=L.EPILOGUE_GELU_ERF, cta_pair=2, single_grid=True)
    _chain(policy, 768, 1024, 2048, 1024, 256, 256, iters=2, max_ctas=10, cta_pair=2, tail_split=4,
           epi1=L.EPILOGUE_GELU_ERF, single_grid=True)
    _chain(policy, 1024, 2048, 1024, 2048, 256, 256, iters=2, opts=L.OPT_NO_ATOMIC_ADD if policy == "tile" else 0,
           cta_pair=2, single_grid=True)


def test_one_grid_chain_refuses_kernels_it_cannot_combine():
    a = _rand((256, 256), 97); b = _rand((256, 256), 98)
    d1 = torch.empty((256, 256), device="cuda", dtype=torch.half)
    d2 = torch.empty((256, 256), device="cuda", dtype=torch.half)
    g1, g2 = cs.Gemm(), cs.Gemm()
    assert g1.initialize(cs.GemmArguments(None, (256, 256, 256), a, b, d1, tile_n=256, cta_pair=2)) == L.SUCCESS
    assert g2.initialize(cs.GemmArguments(None, (256, 256, 256), d1, b, d2, tile_n=128, cta_pair=1)) == L.SUCCESS
    assert cs.Gemm.run_chain(g1, g2, torch.cuda.current_stream()) == L.ERROR_UNSUPPORTED
    g1.destroy(); g2.destroy()
