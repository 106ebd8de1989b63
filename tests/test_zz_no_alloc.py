"""cusync_gemm_run_noalloc: the GEMM entry point for callers that may not
allocate device memory when they call the library (a plug-in under a runtime
that owns the device through its own arena, a latency-critical loop where
cudaMalloc would serialise the device, a process at its memory limit).  Its
scratch is a fixed array inside the library instead of a cudaMalloc'd stage.

Checked here, through the C ABI: its output against the regular plan-based
entry point on the same inputs, on two calls in a row that share the scratch
(the second with a different shape, so stale contents would show), and the
refusal of a problem with more tiles than the fixed scratch holds.
This file sorts last on purpose: a run that stops at the first failure has
then already run every other test."""
import ctypes as C

import pytest

import oracle_lib as o
import cusync_b200 as cs
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-2   # same tolerance as the other GEMM parity tests


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return ((torch.rand(shape, generator=g) * 2 - 1) * scale).half().cuda()


def _desc(a, b, d, epi, tile_n, b2=None):
    M, K = a.shape
    N = b.shape[1]
    return L.GemmDesc(M, N, K, a.data_ptr(), K, b.data_ptr(), N, b2.data_ptr() if b2 is not None else None,
                      d.data_ptr(), N, L.B_ROW_MAJOR_KN, epi, tile_n, 0, 1, 1, 0, None)


def _plan_based(a, b, epi, tile_n, b2=None):
    d = torch.full((a.shape[0], b.shape[1]), float("nan"), device="cuda", dtype=torch.half)
    g = cs.Gemm()
    assert g.initialize(cs.GemmArguments(None, (a.shape[0], b.shape[1], a.shape[1]), a, b, d, epilogue=epi,
                                         ref_b2=b2, tile_n=tile_n, cta_pair=1, split_k_slices=1)) == L.SUCCESS
    assert g.run(stream=torch.cuda.current_stream()) == L.SUCCESS
    torch.cuda.synchronize()
    g.destroy()
    return d


def test_noalloc_matches_plan_based_entry_point_on_two_calls_in_a_row():
    stream = torch.cuda.current_stream().cuda_stream
    cases = [
        # (M, N, K, tile_n, epilogue): the first fills 8 x 8 = 64 schedule slots, the second only 3 x 2
        (1024, 1024, 512, 128, L.EPILOGUE_GELU_ERF),
        (300, 200, 264, 128, L.EPILOGUE_NONE),
    ]
    outs = []
    for i, (M, N, K, tile_n, epi) in enumerate(cases):
        a = _rand((M, K), 100 + i)
        b = _rand((K, N), 200 + i, scale=0.1)
        d = torch.full((M, N), float("nan"), device="cuda", dtype=torch.half)
        desc = _desc(a, b, d, epi, tile_n)
        # both calls are issued before any synchronisation: they run back to back on one stream
        assert L.lib().cusync_gemm_run_noalloc(C.byref(desc), stream) == L.SUCCESS
        outs.append((a, b, d, epi, tile_n))
    torch.cuda.synchronize()
    for a, b, d, epi, tile_n in outs:
        expect = _plan_based(a, b, epi, tile_n)
        assert not torch.isnan(d).any()
        assert o.max_rel_err(d.cpu().numpy(), expect.cpu().numpy()) <= TOL
        assert torch.equal(d, expect)          # same kernel, same schedule: bit-identical as well
        oepi = {L.EPILOGUE_NONE: o.EPI_NONE, L.EPILOGUE_GELU_ERF: o.EPI_GELU_ERF}[epi]
        ref = o.gemm_f16(a.cpu().numpy(), b.cpu().numpy(), oepi)
        assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL


def test_noalloc_dual_gemm_after_a_plain_one():
    stream = torch.cuda.current_stream().cuda_stream
    a = _rand((200, 256), 1); b1 = _rand((256, 320), 2, 0.1); b2 = _rand((256, 320), 3, 0.1)
    d = torch.full((200, 320), float("nan"), device="cuda", dtype=torch.half)
    desc = _desc(a, b1, d, L.EPILOGUE_SILU_MUL_DUAL, 64, b2)
    assert L.lib().cusync_gemm_run_noalloc(C.byref(desc), stream) == L.SUCCESS
    torch.cuda.synchronize()
    expect = _plan_based(a, b1, L.EPILOGUE_SILU_MUL_DUAL, 64, b2)
    assert o.max_rel_err(d.cpu().numpy(), expect.cpu().numpy()) <= TOL
    ref = o.gemm_dual_silu_mul_f16(a.cpu().numpy(), b1.cpu().numpy(), b2.cpu().numpy())
    assert o.max_rel_err(d.cpu().numpy(), ref) <= TOL
    # the call left no timeout record in the static array
    status = L.Status()
    assert L.lib().cusync_gemm_noalloc_read_status(C.byref(status)) == L.SUCCESS
    assert status.code == 0


def test_noalloc_refuses_the_kernel_forms_it_does_not_run():
    stream = torch.cuda.current_stream().cuda_stream
    a = _rand((512, 256), 7); b = _rand((256, 512), 8, 0.1)
    d = torch.zeros((512, 512), device="cuda", dtype=torch.half)
    for split_k, cta_pair, tail_split in ((2, 0, 0), (0, 2, 0), (0, 0, 2)):
        desc = L.GemmDesc(512, 512, 256, a.data_ptr(), 256, b.data_ptr(), 512, None, d.data_ptr(), 512,
                          L.B_ROW_MAJOR_KN, L.EPILOGUE_NONE, 256, 0, split_k, cta_pair, tail_split, None)
        assert L.lib().cusync_gemm_run_noalloc(C.byref(desc), stream) == L.ERROR_UNSUPPORTED
    torch.cuda.synchronize()
    assert (d == 0).all()


def test_noalloc_refuses_more_tiles_than_its_scratch_and_stage_handles():
    stream = torch.cuda.current_stream().cuda_stream
    a = _rand((128, 64), 5); b = _rand((64, 128), 6)
    d = torch.zeros((128, 128), device="cuda", dtype=torch.half)
    # 12800 x 6464 with 128 x 64 tiles = 100 x 101 = 10100 tiles > 8192: refused before anything is touched
    big = L.GemmDesc(12800, 6464, 64, a.data_ptr(), 64, b.data_ptr(), 6464, None, d.data_ptr(), 6464,
                     L.B_ROW_MAJOR_KN, L.EPILOGUE_NONE, 64, 0, 0, 0, 0, None)
    assert L.lib().cusync_gemm_run_noalloc(C.byref(big), stream) == L.ERROR_EXCEEDS_STATIC_SCRATCH
    torch.cuda.synchronize()
    assert (d == 0).all()
    st = cs.CuStage(cs.TransposeXYOrder, (1, 1, 1), (1, 1, 1), cs.NoSync(), cs.NoSync())
    with_stage = L.GemmDesc(128, 128, 64, a.data_ptr(), 64, b.data_ptr(), 128, None, d.data_ptr(), 128,
                            L.B_ROW_MAJOR_KN, L.EPILOGUE_NONE, 128, 0, 0, 0, 0, st._h)
    assert L.lib().cusync_gemm_run_noalloc(C.byref(with_stage), stream) == L.ERROR_INVALID_ARGUMENT
    st.destroy()
