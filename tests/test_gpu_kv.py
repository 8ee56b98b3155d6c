"""KV append / fill / RoPE / gate kernels on the GPU against the CPU oracle and the
golden vectors. Quantized bytes must be identical (0 differing bytes)."""
import numpy as np
import pytest

from oracle.oracle import TYPE_NAMES

pytestmark = pytest.mark.gpu
ALL_TYPES = range(6)


@pytest.fixture(scope="module")
def G(cuda):
    from tests import gpu_util
    return gpu_util


@pytest.mark.parametrize("t", ALL_TYPES, ids=[TYPE_NAMES[t] for t in ALL_TYPES])
def test_store_golden_bit_exact(G, golden, t):
    g = golden("kv_store")
    got = G.kv_store(t, g["src"])
    assert int((got != g["bytes_" + TYPE_NAMES[t]]).sum()) == 0
    G.status_ok()


@pytest.mark.parametrize("t", ALL_TYPES, ids=[TYPE_NAMES[t] for t in ALL_TYPES])
@pytest.mark.parametrize("n_tok", [1, 4, 512])
def test_store_random_rows_bit_exact(G, oracle, t, n_tok):
    rng = np.random.default_rng(100 + n_tok)
    src = rng.standard_normal((n_tok, 4, 256)).astype(np.float32)
    got = G.kv_store(t, src)
    want = oracle.kv_store_rows(t, src)
    assert got.size == want.size
    assert int((got != want).sum()) == 0


@pytest.mark.parametrize("t", [2, 3, 4, 5], ids=["q8_0", "q4_0", "q5_0", "q4_1"])
def test_store_large_and_hostile_bit_exact(G, oracle, t):
    """16M values incl. ties, tiny/huge magnitudes and sums that land on rounding
    boundaries (where a fused multiply-add would change the byte)."""
    rng = np.random.default_rng(7)
    n = 1 << 24
    src = rng.standard_normal(n).astype(np.float32)
    src[: n // 8] = np.round(src[: n // 8] * 4) / 4            # many exact ties
    src[n // 8: n // 4] *= 1e-6
    src[n // 4: n // 4 + n // 8] *= 1e4
    src[n // 2: n // 2 + 4096] = 0.0
    blk = src[n // 2 + 4096: n // 2 + 8192].reshape(-1, 32)
    blk[:, 5] = 3.0
    blk[:, 9] = -3.0                                           # +max before -max: first wins
    got = G.kv_store(t, src)
    want = oracle.kv_store_rows(t, src)
    assert int((got != want).sum()) == 0


def test_store_ragged_width_and_untouched_tail(G, oracle, rd):
    import torch
    src = np.random.default_rng(3).standard_normal(96).astype(np.float32)
    for t in ALL_TYPES:
        d_src = G.dev(src)
        nbytes = len(oracle.kv_store_rows(t, src))
        dst = torch.full((nbytes + 64,), 0xA5, dtype=torch.uint8, device="cuda")
        rd.check(rd.lib.rd_kv_store_rows(t, rd.ptr(d_src), rd.ptr(dst), 96, G.st()))
        torch.cuda.synchronize()
        got = G.host(dst)
        assert (got[:nbytes] == oracle.kv_store_rows(t, src)).all()
        assert (got[nbytes:] == 0xA5).all(), "wrote past the last block"


@pytest.mark.parametrize("t", ALL_TYPES, ids=[TYPE_NAMES[t] for t in ALL_TYPES])
def test_fill_matches_oracle(G, oracle, golden, rd, t):
    import torch
    n_rows = 1000
    buf = torch.zeros(n_rows * rd.row_bytes(t), dtype=torch.uint8, device="cuda")
    rd.check(rd.lib.rd_kv_fill(t, rd.ptr(buf), n_rows, 256, 11, G.st()))
    torch.cuda.synchronize()
    got = G.host(buf)
    assert (got == oracle.kv_fill(t, n_rows, 256, 11)).all()
    if t != 3:  # the reference's q4_0 fill is racy and is no fixture
        g = golden("kv_fill")
        assert (got[: g["fill_" + TYPE_NAMES[t]].size] == g["fill_" + TYPE_NAMES[t]]).all()


def test_rope_matches_oracle_and_golden(G, oracle, golden, rd):
    import torch
    g = golden("rope")
    x = G.dev(g["x"])
    pos = G.dev(g["pos"])
    rd.check(rd.lib.rd_rope(rd.ptr(x), 6, 4, 256, 64, 1e7, rd.ptr(pos), G.st()))
    torch.cuda.synchronize()
    got = G.host(x)
    rel = np.linalg.norm(got.astype(np.float64) - g["out"]) / np.linalg.norm(g["out"].astype(np.float64))
    assert rel < 1e-6, rel        # the reference's own gate (check_rope_gpu.hip:86)
    assert (got[:, :, 64:] == g["x"][:, :, 64:]).all()
    # Q-shaped, 24 heads, many positions
    rng = np.random.default_rng(5)
    xq = rng.standard_normal((64, 24, 256)).astype(np.float32)
    p = rng.integers(0, 262144, size=64).astype(np.int32)
    d, dp = G.dev(xq), G.dev(p)
    rd.check(rd.lib.rd_rope(rd.ptr(d), 64, 24, 256, 64, 1e7, rd.ptr(dp), G.st()))
    torch.cuda.synchronize()
    want = oracle.rope(xq, p)
    rel = np.linalg.norm(G.host(d).astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64))
    assert rel < 1e-6, rel


def test_append_two_tensors_equals_two_stores(G, oracle, rd):
    import torch
    rng = np.random.default_rng(9)
    ks = rng.standard_normal((7, 4, 256)).astype(np.float32)
    vs = rng.standard_normal((7, 4, 256)).astype(np.float32)
    for kt, vt in ((3, 3), (2, 1), (1, 3), (0, 2), (4, 5)):
        kd = torch.zeros(7 * 4 * rd.row_bytes(kt), dtype=torch.uint8, device="cuda")
        vd = torch.zeros(7 * 4 * rd.row_bytes(vt), dtype=torch.uint8, device="cuda")
        dks, dvs = G.dev(ks), G.dev(vs)   # keep the device inputs alive across the call
        rd.check(rd.lib.rd_kv_append(kt, vt, rd.ptr(dks), rd.ptr(dvs), rd.ptr(kd),
                                     rd.ptr(vd), 7, 4, 256, None, 0, 0.0, G.st()))
        torch.cuda.synchronize()
        assert (G.host(kd) == oracle.kv_store_rows(kt, ks)).all()
        assert (G.host(vd) == oracle.kv_store_rows(vt, vs)).all()


def test_append_with_fused_rope(G, oracle, rd):
    """RoPE fused into the K append. Device sin/cos differ from the host's by an ulp, so
    the gate is numeric for K (values within one quantisation step, almost all bytes
    equal) and bit-exact for V, which is not rotated."""
    import torch
    rng = np.random.default_rng(10)
    n_tok = 33
    ks = rng.standard_normal((n_tok, 4, 256)).astype(np.float32)
    vs = rng.standard_normal((n_tok, 4, 256)).astype(np.float32)
    pos = (np.arange(n_tok) * 4001 % 131072).astype(np.int32)
    kr = oracle.rope(ks, pos)
    for kt in (0, 1, 2, 3):
        kd = torch.zeros(n_tok * 4 * rd.row_bytes(kt), dtype=torch.uint8, device="cuda")
        vd = torch.zeros(n_tok * 4 * rd.row_bytes(3), dtype=torch.uint8, device="cuda")
        dks, dvs, dpos = G.dev(ks), G.dev(vs), G.dev(pos)
        rd.check(rd.lib.rd_kv_append(kt, 3, rd.ptr(dks), rd.ptr(dvs), rd.ptr(kd), rd.ptr(vd),
                                     n_tok, 4, 256, rd.ptr(dpos), 64, 1e7, G.st()))
        torch.cuda.synchronize()
        assert (G.host(dks) == ks).all(), "k_src must not be modified"
        assert (G.host(vd) == oracle.kv_store_rows(3, vs)).all()
        got = G.host(kd)
        want = oracle.kv_store_rows(kt, kr)
        if kt == 0:   # raw f32: an ulp of sin/cos shows in the low byte; compare values
            assert np.allclose(got.view(np.float32), want.view(np.float32), rtol=2e-6, atol=2e-7)
        else:
            assert (got != want).mean() < 2e-2
        a = oracle.kv_dequant_rows(kt, got, n_tok * 4)
        b = oracle.kv_dequant_rows(kt, want, n_tok * 4)
        step = np.abs(kr).reshape(-1, 32).max(axis=1).repeat(32).reshape(a.shape) / 7.0
        assert (np.abs(a - b) <= step * 1.01 + 1e-6).all()


def test_gate_and_deinterleave(G, oracle, golden, rd):
    import torch
    g = golden("gate")
    dg, dy = G.dev(g["g"]), G.dev(g["y"])
    rd.check(rd.lib.rd_sigmoid_gate(rd.ptr(dg), rd.ptr(dy), 512, G.st()))
    torch.cuda.synchronize()
    assert np.abs(G.host(dg) - g["g_out"]).max() <= 2e-7
    assert np.abs(G.host(dy) - g["y_out"]).max() <= 1e-6
    rng = np.random.default_rng(2)
    yq = rng.standard_normal((5, 24, 512)).astype(np.float32)
    q = torch.zeros((5, 24, 256), device="cuda")
    gate = torch.zeros((5, 24, 256), device="cuda")
    dyq = G.dev(yq)
    rd.check(rd.lib.rd_deinterleave_q_gate(rd.ptr(dyq), rd.ptr(q), rd.ptr(gate), 5, 24, 256, G.st()))
    torch.cuda.synchronize()
    wq, wg = oracle.deinterleave_q_gate(yq, 5, 24, 256)
    assert (G.host(q) == wq).all() and (G.host(gate) == wg).all()
    G.status_ok()
