"""Causal prefill attention (tcgen05 kernel) on the GPU against the CPU oracle and the
golden vector of the reference's own tile kernel. Gates: max-abs <= 2e-3, cosine >= 0.9999."""
import numpy as np
import pytest

from tests.conftest import check_attn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G(cuda):
    from tests import gpu_util
    return gpu_util


def run_prefill(G, rd, q, kc, vc, pos, keys_total, nkv, gate=None, n_rot=0, inplace=False):
    import torch
    n_q, nh, _ = q.shape
    dq, dk, dv, dpos = G.dev(q), G.dev(kc), G.dev(vc), G.dev(np.asarray(pos, dtype=np.int32))
    out = dq if inplace else G.poison(q.shape)
    dg = G.dev(gate) if gate is not None else None
    if gate is None and n_rot == 0:
        rc = rd.lib.rd_fa2_prefill(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), rd.ptr(dpos), n_q,
                                   int(max(pos)), keys_total, nh, nkv, 256, 1 / 16, G.st())
    else:
        rc = rd.lib.rd_attn_prefill_fused(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), rd.ptr(dg),
                                          rd.ptr(dpos), n_q, keys_total, nh, nkv, 256, 1 / 16, n_rot, 1e7,
                                          G.st())
    rd.check(rc, "prefill")
    torch.cuda.synchronize()
    assert rd.lib.rd_device_status() == rd.OK
    return G.host(out)


def test_golden_tile_kernel(G, golden, rd):
    g = golden("fa2_prefill")
    got = run_prefill(G, rd, g["q"], g["k"], g["v"], g["pos"], int(g["pos"][-1]) + 1, 1)
    check_attn(got, g["out"], what="fa2 prefill golden")


@pytest.mark.parametrize("n_q,pos0", [(512, 0), (200, 0), (128, 37), (1, 0), (512, 1536), (130, 4000)])
def test_prefill_shapes_vs_oracle(G, oracle, rd, n_q, pos0):
    rng = np.random.default_rng(n_q + pos0)
    keys_total = pos0 + n_q
    nh, nkv = (24, 4) if keys_total <= 1024 else (6, 1)   # keep the CPU oracle quick
    K = rng.standard_normal((keys_total, nkv, 256)).astype(np.float32)
    V = rng.standard_normal((keys_total, nkv, 256)).astype(np.float32)
    q = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(1, K), oracle.kv_store_rows(1, V)
    pos = np.arange(pos0, keys_total, dtype=np.int32)
    want = oracle.attn(q, kc, vc, pos, nkv, 1 / 16, 1, 1)
    got = run_prefill(G, rd, q, kc, vc, pos, keys_total, nkv)
    check_attn(got, want, what=f"prefill n_q={n_q} pos0={pos0}")
    got2 = run_prefill(G, rd, q, kc, vc, pos, keys_total, nkv, inplace=True)   # q and o alias
    check_attn(got2, want, what="prefill in place")


def test_prefill_ragged_positions_and_empty_rows(G, oracle, rd):
    rng = np.random.default_rng(5)
    keys_total, n_q = 300, 140
    K = rng.standard_normal((keys_total, 1, 256)).astype(np.float32)
    V = rng.standard_normal((keys_total, 1, 256)).astype(np.float32)
    q = rng.standard_normal((n_q, 6, 256)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(1, K), oracle.kv_store_rows(1, V)
    pos = rng.integers(0, keys_total, size=n_q).astype(np.int32)
    pos[3] = -1            # a token with no keys: zeros
    pos[77] = 0
    want = oracle.attn(q, kc, vc, pos, 1, 1 / 16, 1, 1)
    got = run_prefill(G, rd, q, kc, vc, pos, keys_total, 1)
    assert (got[3] == 0).all()
    check_attn(got, want, what="ragged pos")


def test_prefill_fused_rope_and_gate(G, oracle, rd):
    """benchmark config 3 in one piece: 512 tokens at position 0, K/V appended as f16 with the
    K RoPE fused into the append, Q RoPE and the sigmoid gate fused into the prefill."""
    import torch
    rng = np.random.default_rng(0)
    n_q, nh, nkv = 512, 24, 4
    q = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    ks = rng.standard_normal((n_q, nkv, 256)).astype(np.float32)
    vs = rng.standard_normal((n_q, nkv, 256)).astype(np.float32)
    gate = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    pos = np.arange(n_q, dtype=np.int32)
    # oracle chain: rope(q), rope(k) -> f16 cache -> attention -> gate
    qr, kr = oracle.rope(q, pos), oracle.rope(ks, pos)
    kc_o, vc_o = oracle.kv_store_rows(1, kr), oracle.kv_store_rows(1, vs)
    att = oracle.attn(qr, kc_o, vc_o, pos, nkv, 1 / 16, 1, 1)
    _, want = oracle.sigmoid_gate(gate, att)
    # device chain through the C ABI
    dks, dvs, dpos = G.dev(ks), G.dev(vs), G.dev(pos)
    kc = torch.zeros(n_q * nkv * 512, dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    rd.check(rd.lib.rd_kv_append(1, 1, rd.ptr(dks), rd.ptr(dvs), rd.ptr(kc), rd.ptr(vc), n_q, nkv, 256,
                                 rd.ptr(dpos), 64, 1e7, G.st()))
    torch.cuda.synchronize()
    assert (G.host(vc) == vc_o).all()
    got = run_prefill(G, rd, q, G.host(kc), G.host(vc), pos, n_q, nkv, gate=gate, n_rot=64)
    check_attn(got, want, what="fused rope + gate prefill-512")


@pytest.mark.parametrize("kt,vt", [(3, 3), (2, 2), (4, 5), (2, 1)])
@pytest.mark.parametrize("pos0", [0, 1536, 7680])
def test_typed_prefill_over_quantized_caches(G, oracle, rd, kt, vt, pos0):
    """512 new tokens over (q4_0,q4_0), (q8_0,q8_0), (q5_0,q4_1), (q8_0,f16) caches through
    rd_attn_prefill_typed (caches expanded once to f16, then the tensor-core kernel) against
    the oracle's attention over the same stored bytes; t = pos[qt] as in
    attn_split_batch_launch (include/rdna4/attn.cuh:958-1049)."""
    import torch
    n_q = 512
    keys_total = pos0 + n_q
    nh, nkv = (24, 4) if keys_total <= 1024 else (6, 1)   # keep the CPU oracle quick
    rng = np.random.default_rng(100 * kt + 10 * vt + pos0)
    K = rng.standard_normal((keys_total, nkv, 256)).astype(np.float32)
    V = rng.standard_normal((keys_total, nkv, 256)).astype(np.float32)
    q = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    gate = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(kt, K), oracle.kv_store_rows(vt, V)
    pos = np.arange(pos0, keys_total, dtype=np.int32)
    y = oracle.attn(q, kc, vc, pos, nkv, 1 / 16, kt, vt)
    _, want = oracle.sigmoid_gate(gate.copy(), y)
    nbytes = rd.lib.rd_attn_prefill_workspace_bytes(kt, vt, n_q, keys_total, nh, nkv, 256)
    # f16 copies of the caches that are not f16, plus the records of the key split (if any)
    assert nbytes >= sum(((keys_total * nkv * 512 + 255) // 256) * 256 for t in (kt, vt) if t != 1)
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device="cuda")
    dq, dk, dv, dg, dpos = G.dev(q), G.dev(kc), G.dev(vc), G.dev(gate), G.dev(pos)
    out = G.poison(q.shape)
    rd.check(rd.lib.rd_attn_prefill_typed(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), rd.ptr(dg), rd.ptr(dpos),
                                          n_q, keys_total, nh, nkv, 256, 1 / 16, kt, vt, 0, 0.0, rd.ptr(ws), nbytes,
                                          G.st()))
    torch.cuda.synchronize()
    assert rd.lib.rd_device_status() == rd.OK
    check_attn(G.host(out), want, what=f"typed prefill {kt}/{vt} pos0={pos0}")
    if nbytes:   # a workspace that is too small is refused before anything runs
        assert rd.lib.rd_attn_prefill_typed(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), None, rd.ptr(dpos), n_q,
                                            keys_total, nh, nkv, 256, 1 / 16, kt, vt, 0, 0.0, rd.ptr(ws), nbytes - 256,
                                            G.st()) == rd.ERR_WORKSPACE


@pytest.mark.parametrize("n_q,row0,n_rot,with_gate", [(512, 0, 64, True), (200, 300, 64, False), (130, 70, 0, True),
                                                      (1, 0, 32, False)])
def test_prefill_with_the_append_fused(G, oracle, rd, n_q, row0, n_rot, with_gate):
    """rd_attn_prefill_append_fused = rd_kv_append (rows row0.., K rotated) + rd_attn_prefill_fused:
    the caches end up with the bytes rd_kv_append writes, the output is the two-call chain's
    (same cache bytes, same query path: bit-identical) and passes the oracle gate."""
    import torch
    rng = np.random.default_rng(n_q + row0)
    nh, nkv = 24, 4
    keys_total = row0 + n_q
    q = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    ks = rng.standard_normal((n_q, nkv, 256)).astype(np.float32)
    vs = rng.standard_normal((n_q, nkv, 256)).astype(np.float32)
    gate = rng.standard_normal((n_q, nh, 256)).astype(np.float32) if with_gate else None
    pos = np.arange(row0, keys_total, dtype=np.int32)
    old = oracle.kv_store_rows(1, rng.standard_normal((max(row0, 1), nkv, 256)).astype(np.float32))[:row0 * nkv * 512]
    base_k = np.concatenate([old, np.full(n_q * nkv * 512, 0xEE, dtype=np.uint8)])
    old_v = oracle.kv_store_rows(1, rng.standard_normal((max(row0, 1), nkv, 256)).astype(np.float32))[:row0 * nkv * 512]
    base_v = np.concatenate([old_v, np.full(n_q * nkv * 512, 0xEE, dtype=np.uint8)])
    dq, dks, dvs, dpos = G.dev(q), G.dev(ks), G.dev(vs), G.dev(pos)
    dg = G.dev(gate) if with_gate else None
    # two calls
    kc1, vc1 = G.dev(base_k), G.dev(base_v)
    off = row0 * nkv * 512
    rd.check(rd.lib.rd_kv_append(1, 1, rd.ptr(dks), rd.ptr(dvs), rd.ptr(kc1) + off, rd.ptr(vc1) + off, n_q, nkv, 256,
                                 rd.ptr(dpos) if n_rot else None, n_rot, 1e7, G.st()))
    out1 = G.poison(q.shape)
    rd.check(rd.lib.rd_attn_prefill_fused(rd.ptr(dq), rd.ptr(kc1), rd.ptr(vc1), rd.ptr(out1), rd.ptr(dg), rd.ptr(dpos),
                                          n_q, keys_total, nh, nkv, 256, 1 / 16, n_rot, 1e7, G.st()))
    # one call
    kc2, vc2 = G.dev(base_k), G.dev(base_v)
    out2 = G.poison(q.shape)
    rd.check(rd.lib.rd_attn_prefill_append_fused(rd.ptr(dq), rd.ptr(dks), rd.ptr(dvs), rd.ptr(kc2), rd.ptr(vc2),
                                                 rd.ptr(out2), rd.ptr(dg), rd.ptr(dpos), n_q, row0, keys_total, nh,
                                                 nkv, 256, 1 / 16, n_rot, 1e7, G.st()))
    torch.cuda.synchronize()
    assert rd.lib.rd_device_status() == rd.OK
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert torch.equal(out1, out2)
    # and the chain against the oracle
    qr = oracle.rope(q, pos, n_rot=n_rot) if n_rot else q
    att = oracle.attn(qr, G.host(kc2), G.host(vc2), pos, nkv, 1 / 16, 1, 1)
    want = oracle.sigmoid_gate(gate.copy(), att)[1] if with_gate else att
    check_attn(G.host(out2), want, what=f"append-fused prefill n_q={n_q} row0={row0} n_rot={n_rot}")
    # argument errors
    call = lambda kn, r0, kt_: rd.lib.rd_attn_prefill_append_fused(rd.ptr(dq), kn, rd.ptr(dvs), rd.ptr(kc2),
                                                                   rd.ptr(vc2), rd.ptr(out2), None, rd.ptr(dpos), n_q,
                                                                   r0, kt_, nh, nkv, 256, 1 / 16, n_rot, 1e7, G.st())
    assert call(None, row0, keys_total) == rd.ERR_NULL
    assert call(rd.ptr(dks), row0 + 1, keys_total) == rd.ERR_SHAPE
    assert call(rd.ptr(dks), -1, keys_total) == rd.ERR_SHAPE


def test_rotating_prefill_in_place_with_a_tile_that_attends_nothing(G, oracle, rd):
    """o aliases q, the queries are rotated by the pre-pass, and the first token tile has no
    key at all (pos = -1): that tile's CTAs have nothing to wait for but must not store their
    zeros before the pre-pass has read the rows they overwrite."""
    rng = np.random.default_rng(11)
    n_q, nh, nkv, keys_total = 256, 24, 4, 128
    K = rng.standard_normal((keys_total, nkv, 256)).astype(np.float32)
    V = rng.standard_normal((keys_total, nkv, 256)).astype(np.float32)
    q = rng.standard_normal((n_q, nh, 256)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(1, K), oracle.kv_store_rows(1, V)
    pos = np.concatenate([np.full(128, -1), np.arange(128)]).astype(np.int32)
    want = oracle.attn(oracle.rope(q, np.maximum(pos, 0)), kc, vc, pos, nkv, 1 / 16, 1, 1)
    for _ in range(3):
        got = run_prefill(G, rd, q, kc, vc, pos, keys_total, nkv, n_rot=64, inplace=True)
        assert (got[:128] == 0).all()
        check_attn(got, want, what="in-place rotating prefill, key-less first tile")
