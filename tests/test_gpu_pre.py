"""RMS-norm and the fused pre-attention stage (deinterleave + q/k norm + RoPE + KV store in
one launch) against the golden vectors, the CPU oracle and the separate entry points."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
NH, NKV, HD = 24, 4, 256


@pytest.fixture(scope="module")
def G(cuda):
    from tests import gpu_util
    return gpu_util


def rms(G, x, w, eps, inplace=False):
    rd, lib = G.rd, G.lib
    dx = G.dev(x)
    dw = G.dev(w) if w is not None else None
    dy = dx if inplace else G.poison(x.shape)
    rows = int(np.prod(x.shape[:-1]))
    rd.check(lib.rd_rms_norm(rd.ptr(dx), rd.ptr(dw), rd.ptr(dy), rows, x.shape[-1], eps, G.st()))
    torch.cuda.synchronize()
    return G.host(dy)


def test_rms_norm_golden_bit_exact(G, oracle, golden):
    g = golden("rms_norm")
    eps = float(g["eps"])
    assert np.array_equal(rms(G, g["x"], g["w"], eps), g["y_w"])
    assert np.array_equal(rms(G, g["x"], None, eps), g["y_now"])
    assert np.array_equal(rms(G, g["xw"], g["ww"], 1e-5), g["yw"])
    assert np.array_equal(rms(G, g["x"], g["w"], eps, inplace=True), g["y_w"])   # x and y alias
    rng = np.random.default_rng(3)
    x = rng.standard_normal((64, 1000)).astype(np.float32)                       # ragged width
    assert np.array_equal(rms(G, x, None, 1e-6), oracle.rms_norm(x, None, 1e-6))
    assert G.lib.rd_rms_norm(None, None, None, 0, 256, 1e-6, G.st()) == G.rd.OK
    assert G.lib.rd_rms_norm(None, None, None, 2, 256, 1e-6, G.st()) == G.rd.ERR_NULL
    assert G.lib.rd_rms_norm(None, None, None, 2, 0, 1e-6, G.st()) == G.rd.ERR_SHAPE


def separate_calls(G, qg, ks, vs, qw, kw, eps, pos, kt, vt, n_rot):
    """The reference's sequence (graph.cuh:915-954) through this library's own entry points."""
    rd, lib = G.rd, G.lib
    n_tok = qg.shape[0]
    d_qg, d_k, d_v = G.dev(qg), G.dev(ks), G.dev(vs)
    d_qw, d_kw, d_pos = G.dev(qw), G.dev(kw), G.dev(pos)
    q, gate = G.poison((n_tok, NH, HD)), G.poison((n_tok, NH, HD))
    rd.check(lib.rd_deinterleave_q_gate(rd.ptr(d_qg), rd.ptr(q), rd.ptr(gate), n_tok, NH, HD, G.st()))
    rd.check(lib.rd_rms_norm(rd.ptr(q), rd.ptr(d_qw), rd.ptr(q), n_tok * NH, HD, eps, G.st()))
    rd.check(lib.rd_rms_norm(rd.ptr(d_k), rd.ptr(d_kw), rd.ptr(d_k), n_tok * NKV, HD, eps, G.st()))
    if n_rot:
        rd.check(lib.rd_rope(rd.ptr(q), n_tok, NH, HD, n_rot, 1e7, rd.ptr(d_pos), G.st()))
        rd.check(lib.rd_rope(rd.ptr(d_k), n_tok, NKV, HD, n_rot, 1e7, rd.ptr(d_pos), G.st()))
    kr = torch.full((n_tok * NKV * rd.row_bytes(kt),), 0xA5, dtype=torch.uint8, device="cuda")
    vr = torch.full((n_tok * NKV * rd.row_bytes(vt),), 0xA5, dtype=torch.uint8, device="cuda")
    rd.check(lib.rd_kv_store_rows(kt, rd.ptr(d_k), rd.ptr(kr), n_tok * NKV * HD, G.st()))
    rd.check(lib.rd_kv_store_rows(vt, rd.ptr(d_v), rd.ptr(vr), n_tok * NKV * HD, G.st()))
    torch.cuda.synchronize()
    return G.host(q), G.host(gate), G.host(kr), G.host(vr), G.host(d_k)


def fused_call(G, qg, ks, vs, qw, kw, eps, pos, kt, vt, n_rot):
    rd, lib = G.rd, G.lib
    n_tok = qg.shape[0]
    d_qg, d_k, d_v = G.dev(qg), G.dev(ks), G.dev(vs)
    d_qw = G.dev(qw) if qw is not None else None
    d_kw = G.dev(kw) if kw is not None else None
    d_pos = G.dev(pos)
    q, gate = G.poison((n_tok, NH, HD)), G.poison((n_tok, NH, HD))
    kr = torch.full((n_tok * NKV * rd.row_bytes(kt),), 0xA5, dtype=torch.uint8, device="cuda")
    vr = torch.full((n_tok * NKV * rd.row_bytes(vt),), 0xA5, dtype=torch.uint8, device="cuda")
    rd.check(lib.rd_pre_attn_fused(rd.ptr(d_qg), rd.ptr(d_k), rd.ptr(d_v), rd.ptr(d_qw), rd.ptr(d_kw), eps,
                                   rd.ptr(q), rd.ptr(gate), rd.ptr(kr), rd.ptr(vr), kt, vt, rd.ptr(d_pos),
                                   n_tok, NH, NKV, HD, n_rot, 1e7, G.st()))
    torch.cuda.synchronize()
    return G.host(q), G.host(gate), G.host(kr), G.host(vr)


@pytest.mark.parametrize("kt,vt", [(3, 3), (2, 1), (4, 5), (1, 0), (0, 2)])
@pytest.mark.parametrize("n_tok,n_rot", [(1, 64), (5, 64), (3, 128), (2, 0)])
def test_fused_equals_separate_calls(G, kt, vt, n_tok, n_rot):
    rng = np.random.default_rng(1000 * kt + 100 * vt + 10 * n_tok + n_rot)
    qg = rng.standard_normal((n_tok, NH, 2 * HD)).astype(np.float32)
    ks = (2.0 * rng.standard_normal((n_tok, NKV, HD))).astype(np.float32)
    vs = rng.standard_normal((n_tok, NKV, HD)).astype(np.float32)
    qw = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    kw = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    pos = np.array([130999, 0, 17, 4095, 262143][:n_tok], dtype=np.int32)
    q0, g0, k0, v0, _ = separate_calls(G, qg, ks, vs, qw, kw, 1e-6, pos, kt, vt, n_rot)
    q1, g1, k1, v1 = fused_call(G, qg, ks, vs, qw, kw, 1e-6, pos, kt, vt, n_rot)
    assert np.array_equal(q1, q0)
    assert np.array_equal(g1, g0) and np.array_equal(g1, qg[:, :, HD:])
    assert np.array_equal(k1, k0)
    assert np.array_equal(v1, v0)
    G.status_ok()


def test_fused_against_oracle_chain(G, oracle):
    """Against the CPU restatement of the reference's sequence: V bytes exact; q within f32
    rounding of the sin/cos routines; K bytes differ only where such a rounding moves a
    value across a quantization boundary."""
    rng = np.random.default_rng(8)
    n_tok = 7
    qg = rng.standard_normal((n_tok, NH, 2 * HD)).astype(np.float32)
    ks = rng.standard_normal((n_tok, NKV, HD)).astype(np.float32)
    vs = rng.standard_normal((n_tok, NKV, HD)).astype(np.float32)
    qw = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    kw = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    pos = np.arange(1000, 1000 + n_tok, dtype=np.int32)
    q_in, gate_want = oracle.deinterleave_q_gate(qg, n_tok, NH, HD)
    q_want = oracle.rope(oracle.rms_norm(q_in, qw, 1e-6), pos)
    k_want = oracle.rope(oracle.rms_norm(ks, kw, 1e-6), pos)
    for kt, vt in ((0, 3), (3, 2)):
        q1, g1, k1, v1 = fused_call(G, qg, ks, vs, qw, kw, 1e-6, pos, kt, vt, 64)
        assert np.array_equal(g1, gate_want)
        np.testing.assert_allclose(q1, q_want, rtol=0, atol=4e-6)
        assert np.array_equal(v1, oracle.kv_store_rows(vt, vs))
        want_k = oracle.kv_store_rows(kt, k_want)
        if kt == 0:
            np.testing.assert_allclose(k1.view(np.float32), want_k.view(np.float32), rtol=0, atol=4e-6)
        else:
            assert (k1 != want_k).mean() < 2e-2
    # no weights: plain normalisation
    q1, _, _, _ = fused_call(G, qg, ks, vs, None, None, 1e-6, pos, 1, 1, 64)
    np.testing.assert_allclose(q1, oracle.rope(oracle.rms_norm(q_in, None, 1e-6), pos), rtol=0, atol=4e-6)
    G.status_ok()


def test_fused_argument_errors(G):
    rd, lib = G.rd, G.lib
    p = rd.ptr(torch.zeros(64, device="cuda"))
    call = lambda hd, n_rot, kt=3, q=p: lib.rd_pre_attn_fused(q, p, p, None, None, 1e-6, p, p, p, p, kt, 3, p, 1,
                                                             NH, NKV, hd, n_rot, 1e7, G.st())
    assert call(128, 64) == rd.ERR_UNSUPPORTED
    assert call(256, 32) == rd.ERR_UNSUPPORTED
    assert call(256, 320) == rd.ERR_SHAPE
    assert call(256, 64, kt=9) == rd.ERR_TYPE
    assert call(256, 64, q=None) == rd.ERR_NULL
