"""GPU parity tests of the decode-attention middle stage and of the three-stage attention block of BASELINE
config 4 (QKV projection -> attention over a K/V cache -> output projection) against the CPU oracle.
The reference's attention chain has no softmax and pins only the stage wiring (attention.cu:105-118); the
arithmetic here is checked against orc_attention_decode_f16 (parity unpinned by any reference test)."""
import numpy as np
import pytest

import oracle_lib as o
import cusync_b200 as cs
from cusync_b200 import _lib as L
from cusync_b200.attention import AttentionBlock, DecodeAttention, PromptAttentionBlock

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
TOL = 1e-2


def _randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).half().cuda()


def _oracle_attention(qkv, kc, vc, heads):
    B = qkv.shape[0]
    hd = heads * 128
    q = qkv[:, :hd].reshape(B, heads, 128)
    knew = qkv[:, hd:2 * hd].reshape(B, 1, heads, 128)
    vnew = qkv[:, 2 * hd:].reshape(B, 1, heads, 128)
    k = np.concatenate([kc, knew], axis=1)
    v = np.concatenate([vc, vnew], axis=1)
    return o.attention_decode_f16(q, k, v).reshape(B, hd)


def _exact_block(x, w_qkv, kc, vc, w_o, heads):
    """The whole block in float64 without intermediate rounding."""
    f = lambda t: t.cpu().numpy().astype(np.float64)
    B, hd = x.shape[0], heads * 128
    qkv = f(x) @ f(w_qkv)
    q = qkv[:, :hd].reshape(B, heads, 128)
    k = np.concatenate([f(kc), qkv[:, hd:2 * hd].reshape(B, 1, heads, 128)], axis=1)
    v = np.concatenate([f(vc), qkv[:, 2 * hd:].reshape(B, 1, heads, 128)], axis=1)
    s = np.einsum("bhd,bshd->bhs", q, k) / np.sqrt(128.0)
    p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
    return (np.einsum("bhs,bshd->bhd", p, v).reshape(B, hd) @ f(w_o)).astype(np.float16)


@pytest.mark.parametrize("B,S,heads,splits", [(1, 512, 12, 0), (4, 2048, 12, 0), (3, 100, 2, 1), (2, 1000, 3, 7),
                                              (5, 0, 2, 1), (130, 64, 1, 2)])
def test_decode_attention_matches_oracle(B, S, heads, splits):
    qkv = _randn((B, 3 * heads * 128), 1)
    kc = _randn((B, S, heads, 128), 2)
    vc = _randn((B, S, heads, 128), 3)
    out = torch.full((B, heads * 128), float("nan"), device="cuda", dtype=torch.half)
    a = DecodeAttention(None, qkv, kc if S else None, vc if S else None, out, heads, splits)
    assert a.create_status == L.SUCCESS
    for _ in range(2):      # split counters must re-arm themselves
        out.fill_(float("nan"))
        assert a.run(torch.cuda.current_stream()) == L.SUCCESS
        torch.cuda.synchronize()
        ref = _oracle_attention(qkv.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), heads)
        assert o.max_rel_err(out.cpu().numpy(), ref) <= TOL
    a.destroy()


@pytest.mark.parametrize("B,S", [(1, 512), (4, 1024), (2, 2048), (160, 128)])
def test_config4_attention_block_chain(B, S):
    heads, H = 12, 12288
    x = _randn((B, H), 10)
    w_qkv = _randn((H, 3 * heads * 128), 11, 0.02)
    w_o = _randn((heads * 128, H), 12, 0.02)
    kc = _randn((B, S, heads, 128), 13)
    vc = _randn((B, S, heads, 128), 14)
    blk = AttentionBlock(x, w_qkv, kc, vc, w_o, heads)
    streams = (torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream())
    qkv_ref = o.gemm_f16(x.cpu().numpy(), w_qkv.cpu().numpy())
    # the oracle's own chain end to end: projection -> attention over the cache -> projection
    y_ref = o.gemm_f16(_oracle_attention(qkv_ref, kc.cpu().numpy(), vc.cpu().numpy(), heads), w_o.cpu().numpy())
    y_exact = _exact_block(x, w_qkv, kc, vc, w_o, heads)
    torch.cuda.synchronize()
    for it in range(1, 4):
        blk.qkv.fill_(float("nan")); blk.o.fill_(float("nan")); blk.y.fill_(float("nan"))   # poison
        torch.cuda.synchronize()
        blk.run(streams)
        torch.cuda.synchronize()
        assert blk.status_codes() == (0, 0, 0)
        qkv = blk.qkv.cpu().numpy()
        assert o.max_rel_err(qkv, qkv_ref) <= TOL
        o_gpu = blk.o.cpu().numpy()
        assert o.max_rel_err(o_gpu, _oracle_attention(qkv, kc.cpu().numpy(), vc.cpu().numpy(), heads)) <= TOL
        assert o.max_rel_err(blk.y.cpu().numpy(), o.gemm_f16(o_gpu, w_o.cpu().numpy())) <= TOL
        # ... and the final output against the oracle's full chain and against the exact chain
        o.check_final_output(blk.y.cpu().numpy(), y_ref, y_exact, "attention block B=%d S=%d run %d" % (B, S, it), TOL)
        # semaphores: three per row panel of the QKV stage (Q, K, V thirds), each reaching its 6 column tiles;
        # one per row panel of the attention stage
        tiles_m = (B + 127) // 128
        group = 1536 // blk.config["tile_n"][0]
        assert (blk.s1.semaphores()[:3 * tiles_m] == group * it).all()
        assert (blk.s2.semaphores()[:tiles_m] == it).all()
    blk.destroy()
    # stream-ordered arm gives the same output
    ref_blk = AttentionBlock(x, w_qkv, kc, vc, w_o, heads, synced=False)
    ref_blk.run((torch.cuda.current_stream(),))
    torch.cuda.synchronize()
    o_gpu = ref_blk.o.cpu().numpy()
    assert o.max_rel_err(ref_blk.y.cpu().numpy(), o.gemm_f16(o_gpu, w_o.cpu().numpy())) <= TOL
    ref_blk.destroy()


def test_attention_wait_times_out():
    B, S, heads = 2, 64, 2
    qkv = _randn((B, 3 * heads * 128), 20); kc = _randn((B, S, heads, 128), 21); vc = _randn((B, S, heads, 128), 22)
    out = torch.zeros((B, heads * 128), device="cuda", dtype=torch.half)
    sync = cs.RowSync(128, 1, 1)
    prod = cs.CuStage(cs.TransposeXYOrder, (1, 1, 1), (1, 1, 1), cs.NoSync(), sync)
    mid = cs.CuStage(cs.IdentityOrder, (heads, B, 1), (1, 1, 1), sync, cs.NoSync())
    assert cs.CuSync.setProducerConsumerPair(prod, mid) == L.SUCCESS
    mid.set_timeout_ns(20e6)
    a = DecodeAttention(mid, qkv, kc, vc, out, heads, 1)
    assert a.create_status == L.SUCCESS
    assert a.run(torch.cuda.current_stream()) == L.SUCCESS
    torch.cuda.synchronize()
    st = mid.status()
    assert st.code == L.ERROR_TIMEOUT and st.expected == 1 and st.seen == 0
    assert (out == 0).all()
    a.destroy(); prod.destroy(); mid.destroy()


@pytest.mark.parametrize("B", [512, 1024])
def test_prompt_phase_attention_chain_of_four_gemms(B):
    # attention.cu:272-276 with seqlen = 0: XQKV = X Wqkv; S = Q K^T; O = S V; Y = O Wo (no softmax), four stages
    # on four streams.  Every stage is compared with the oracle fed with what the GPU produced before it, and the
    # final output with the oracle's own chain.  Inputs are scaled down (X ~ N(0, 0.1^2)) so that O stays inside
    # fp16: the reference skips its check of this chain because its inputs overflow (attention.cu:512-515).
    heads, H = 12, 12288
    hd = heads * 128
    x = _randn((B, H), 20, 0.1)
    w_qkv = _randn((H, 3 * hd), 21, 0.02)
    w_o = _randn((hd, H), 22, 0.02)
    blk = PromptAttentionBlock(x, w_qkv, w_o, heads)
    streams = [torch.cuda.Stream(priority=-1)] + [torch.cuda.Stream() for _ in range(3)]
    rows = np.arange(0, B, B // 64)                # 64 sampled rows through the row-wise stages
    qkv_ref = o.gemm_f16(x.cpu().numpy(), w_qkv.cpu().numpy())
    s_ref = o.gemm_f16(qkv_ref[rows, :hd], np.ascontiguousarray(qkv_ref[:, hd:2 * hd].T))
    o_ref = o.gemm_f16(s_ref, np.ascontiguousarray(qkv_ref[:, 2 * hd:]))
    y_ref = o.gemm_f16(o_ref, w_o.cpu().numpy())
    f = lambda t: t.cpu().numpy().astype(np.float64)
    qkv64 = f(x) @ f(w_qkv)
    y_exact = (((qkv64[rows, :hd] @ qkv64[:, hd:2 * hd].T) @ qkv64[:, 2 * hd:]) @ f(w_o)).astype(np.float16)
    tiles_m = B // 128
    torch.cuda.synchronize()
    for it in range(1, 4):
        for t in (blk.qkv, blk.s, blk.o, blk.y):
            t.fill_(float("nan"))                  # a stage that reads ahead of its producer sees NaN
        torch.cuda.synchronize()
        blk.run(streams)
        torch.cuda.synchronize()
        assert blk.status_codes() == (0, 0, 0, 0)
        qkv = blk.qkv.cpu().numpy()
        assert o.max_rel_err(qkv, qkv_ref) <= TOL
        s_gpu = blk.s.cpu().numpy()
        assert not np.isnan(s_gpu.astype(np.float32)).any()
        assert o.max_rel_err(s_gpu[rows], o.gemm_f16(qkv[rows, :hd], np.ascontiguousarray(qkv[:, hd:2 * hd].T))) <= TOL
        o_gpu = blk.o.cpu().numpy()
        assert not np.isnan(o_gpu.astype(np.float32)).any()
        assert o.max_rel_err(o_gpu[rows], o.gemm_f16(s_gpu[rows], np.ascontiguousarray(qkv[:, 2 * hd:]))) <= TOL
        y_gpu = blk.y.cpu().numpy()
        assert not np.isnan(y_gpu.astype(np.float32)).any()
        assert o.max_rel_err(y_gpu[rows], o.gemm_f16(o_gpu[rows], w_o.cpu().numpy())) <= TOL
        o.check_final_output(y_gpu[rows], y_ref, y_exact, "prompt attention B=%d run %d" % (B, it), TOL)
        # semaphores: ConsecutiveSync counts the six column tiles of each third of a row panel; RowSync counts the
        # column tiles of S (B / 256) and of O (6)
        assert (blk.stages[0].semaphores()[:3 * tiles_m] == 6 * it).all()
        assert (blk.stages[1].semaphores()[:tiles_m] == (B // 256) * it).all()
        assert (blk.stages[2].semaphores()[:tiles_m] == 6 * it).all()
    y_sync = blk.y.clone()
    blk.y.fill_(float("nan"))
    blk.run_stream_ordered(torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(blk.y, y_sync)
    blk.destroy()
    with pytest.raises(L.CuSyncError):
        PromptAttentionBlock(x[:256].contiguous(), w_qkv, w_o, heads)      # needs more than two row tiles
