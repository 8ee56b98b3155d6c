"""Context-sharded decode with the fused record exchange, exercised on ONE GPU: the
ranks' exchange buffers all live on this device and the ranks' launches are issued one
after another on one stream -- every push before any merge, so no kernel ever waits
for a launch that has not finished. The multi-process run over NVLink is bench.py
--gpus N; the sharding arithmetic itself is covered on CPU in test_sharding.py."""
import numpy as np
import pytest
import torch

from tests.conftest import check_attn

pytestmark = pytest.mark.gpu
NH, NKV, HD = 24, 4, 256


@pytest.fixture(scope="module")
def G(cuda):
    from tests import gpu_util
    return gpu_util


def make_groups(G, world, wait_limit_us=0):
    rd, lib = G.rd, G.lib
    nbytes = lib.rd_shard_xbuf_bytes(NH, HD, world)
    assert nbytes >= 2 * world * NH * 258 * 4
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    groups = [rd.shard_group(r, [rd.ptr(b) for b in bufs], wait_limit_us) for r in range(world)]
    return bufs, groups


@pytest.mark.parametrize("world,kt,vt,n_keys", [(2, 3, 3, 5000), (4, 2, 1, 1000), (8, 3, 3, 6), (3, 1, 0, 777)])
def test_push_merge_matches_full_context(G, oracle, world, kt, vt, n_keys):
    """Records of contiguous key slices, pushed to every rank and merged there, give the
    attention over the whole context on every rank -- three calls in a row, so both
    parities of the exchange buffer and their reuse are covered."""
    import ctypes as C
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(world * 1000 + n_keys)
    K = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(kt, K), oracle.kv_store_rows(vt, V)
    rk, rv = rd.row_bytes(kt) * NKV, rd.row_bytes(vt) * NKV
    per = (n_keys + world - 1) // world          # some ranks own nothing when world > keys
    bufs, groups = make_groups(G, world)
    dk, dv = G.dev(kc), G.dev(vc)
    for call in range(3):
        q = rng.standard_normal((NH, HD)).astype(np.float32)
        gate = rng.standard_normal((NH, HD)).astype(np.float32)
        want_g, want = oracle.sigmoid_gate(gate, oracle.attn(q[None], kc, vc, [n_keys - 1], NKV, 1 / 16, kt, vt)[0])
        dq = G.dev(q)
        parts, outs, gates = [], [], []
        for r in range(world):                    # every rank: slice records, then push
            b, e = r * per, min(n_keys, (r + 1) * per)
            n_splits = 1 + r % 3
            part = G.poison((NH, n_splits, 2 + HD))
            off_k, off_v = min(b, n_keys - 1) * rk, min(b, n_keys - 1) * rv
            rd.check(lib.rd_attn_decode_split(rd.ptr(dq), rd.ptr(dk) + off_k, rd.ptr(dv) + off_v, None,
                                              rd.ptr(part), max(e - b, 0) - 1, NH, NKV, HD, 1 / 16, kt, vt,
                                              n_splits, G.st()))
            rd.check(lib.rd_attn_shard_push(rd.ptr(part), n_splits, NH, HD, C.addressof(groups[r]), G.st()))
            parts.append(part)
        for r in range(world):                    # then every rank merges
            out, dg = G.poison((NH, HD)), G.dev(gate)
            rd.check(lib.rd_attn_shard_merge(rd.ptr(out), rd.ptr(dg), NH, HD, C.addressof(groups[r]), G.st()))
            outs.append(out)
            gates.append(dg)
        torch.cuda.synchronize()
        for r in range(world):
            check_attn(G.host(outs[r]), want, what=f"rank {r} of {world}, call {call}")
            assert np.abs(G.host(gates[r]) - want_g).max() <= 1e-6
            assert torch.equal(outs[r], outs[0])   # every rank merges the same records
    G.status_ok()
    for r in range(world):                        # three calls completed on every rank
        assert int(bufs[r][:4].view(torch.int32).item()) == 3


def test_world_one_sharded_entry_equals_decode(G, oracle):
    """rd_attn_decode_sharded with a group of one is the plain decode."""
    import ctypes as C
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(3)
    n = 3000
    K = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(3, K), oracle.kv_store_rows(3, V)
    bufs, groups = make_groups(G, 1)
    dq, dk, dv = G.dev(q), G.dev(kc), G.dev(vc)
    nbytes = lib.rd_attn_workspace_bytes(1, NH, HD)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = G.poison((NH, HD))
    for _ in range(2):
        rd.check(lib.rd_attn_decode_sharded(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), n - 1, NH, NKV,
                                            HD, 1 / 16, 3, 3, None, rd.ptr(ws), nbytes,
                                            C.addressof(groups[0]), G.st()))
    torch.cuda.synchronize()
    check_attn(G.host(out), oracle.attn(q[None], kc, vc, [n - 1], NKV, 1 / 16, 3, 3)[0])
    assert np.abs(G.host(out) - G.attn_decode(q, kc, vc, n - 1, 3, 3)).max() <= 2e-5
    G.status_ok()


@pytest.mark.parametrize("kt,vt,n", [(3, 3, 3000), (2, 1, 1), (0, 0, 517), (4, 5, 2), (1, 3, 9000)])
def test_world_one_sharded_append_stores_the_row_and_attends_it(G, oracle, kt, vt, n):
    """rd_attn_decode_sharded_append = rd_kv_append of row n-1 + rd_attn_decode_sharded over
    n keys, in one launch: the stored bytes are the oracle's, the output attends the new
    key. n = 1 is the owner of an otherwise empty slice."""
    import ctypes as C
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(40 + n)
    K = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(kt, K), oracle.kv_store_rows(vt, V)
    rk, rv = rd.row_bytes(kt) * NKV, rd.row_bytes(vt) * NKV
    k0, v0 = kc.copy(), vc.copy()
    k0[(n - 1) * rk:], v0[(n - 1) * rv:] = 0xEE, 0xEE     # the newest row is not in the cache yet
    bufs, groups = make_groups(G, 1)
    dk, dv = G.dev(k0), G.dev(v0)
    nbytes = lib.rd_attn_workspace_bytes(1, NH, HD)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    for call in range(2):
        q = rng.standard_normal((NH, HD)).astype(np.float32)
        gate = rng.standard_normal((NH, HD)).astype(np.float32)
        want_g, want = oracle.sigmoid_gate(gate.copy(), oracle.attn(q[None], kc, vc, [n - 1], NKV, 1 / 16, kt, vt)[0])
        dq, dg, out = G.dev(q), G.dev(gate), G.poison((NH, HD))
        dkn, dvn = G.dev(K[n - 1]), G.dev(V[n - 1])
        rd.check(lib.rd_attn_decode_sharded_append(rd.ptr(dq), rd.ptr(dkn), rd.ptr(dvn), rd.ptr(dk), rd.ptr(dv),
                                                   rd.ptr(out), n - 1, NH, NKV, HD, 1 / 16, kt, vt, rd.ptr(dg),
                                                   rd.ptr(ws), nbytes, C.addressof(groups[0]), G.st()))
        torch.cuda.synchronize()
        assert np.array_equal(G.host(dk), kc) and np.array_equal(G.host(dv), vc)
        check_attn(G.host(out), want, what=f"call {call}")
        assert np.abs(G.host(dg) - want_g).max() <= 1e-6
    G.status_ok()
    # argument errors of the fused form
    assert lib.rd_attn_decode_sharded_append(rd.ptr(dq), None, rd.ptr(dvn), rd.ptr(dk), rd.ptr(dv), rd.ptr(out),
                                             n - 1, NH, NKV, HD, 1 / 16, kt, vt, None, rd.ptr(ws), nbytes,
                                             C.addressof(groups[0]), G.st()) == rd.ERR_NULL
    assert lib.rd_attn_decode_sharded_append(rd.ptr(dq), rd.ptr(dkn), rd.ptr(dvn), rd.ptr(dk), rd.ptr(dv),
                                             rd.ptr(out), -1, NH, NKV, HD, 1 / 16, kt, vt, None, rd.ptr(ws), nbytes,
                                             C.addressof(groups[0]), G.st()) == rd.ERR_SHAPE
    assert lib.rd_attn_decode_sharded_append(rd.ptr(dq), rd.ptr(dkn), rd.ptr(dvn), rd.ptr(dk), rd.ptr(dv),
                                             rd.ptr(dq), n - 1, NH, NKV, HD, 1 / 16, kt, vt, None, rd.ptr(ws),
                                             nbytes, C.addressof(groups[0]), G.st()) == rd.ERR_UNSUPPORTED


def test_missing_rank_times_out_and_reports(G):
    """A rank that never pushes: the merge gives up after the wait limit, stores zeros,
    and the library reports RD_ERR_DEVICE once; the context stays usable."""
    import ctypes as C
    rd, lib = G.rd, G.lib
    G.status_ok()
    bufs, groups = make_groups(G, 2, wait_limit_us=20000)
    part = torch.zeros(NH, 1, 2 + HD, device="cuda")
    part[:, :, 1] = 1.0
    part[:, :, 2:] = 5.0
    rd.check(lib.rd_attn_shard_push(rd.ptr(part), 1, NH, HD, C.addressof(groups[0]), G.st()))
    out = G.poison((NH, HD))
    rd.check(lib.rd_attn_shard_merge(rd.ptr(out), None, NH, HD, C.addressof(groups[0]), G.st()))
    torch.cuda.synchronize()
    assert lib.rd_device_status() == rd.ERR_DEVICE
    assert lib.rd_device_status() == rd.OK        # reported once, then cleared
    assert (out == 0).all()
    # the same buffers with only rank 0 in the group work right after
    bufs1, groups1 = make_groups(G, 1)
    rd.check(lib.rd_attn_shard_push(rd.ptr(part), 1, NH, HD, C.addressof(groups1[0]), G.st()))
    rd.check(lib.rd_attn_shard_merge(rd.ptr(out), None, NH, HD, C.addressof(groups1[0]), G.st()))
    torch.cuda.synchronize()
    assert torch.allclose(out, torch.full_like(out, 5.0))
    G.status_ok()


def test_group_argument_errors(G):
    import ctypes as C
    rd, lib = G.rd, G.lib
    bufs, groups = make_groups(G, 2)
    part = torch.zeros(NH, 1, 2 + HD, device="cuda")
    out = G.poison((NH, HD))
    assert lib.rd_attn_shard_push(rd.ptr(part), 1, NH, HD, None, G.st()) == rd.ERR_NULL
    assert lib.rd_attn_shard_push(None, 1, NH, HD, C.addressof(groups[0]), G.st()) == rd.ERR_NULL
    assert lib.rd_attn_shard_push(rd.ptr(part), 0, NH, HD, C.addressof(groups[0]), G.st()) == rd.ERR_SHAPE
    assert lib.rd_attn_shard_push(rd.ptr(part), 1, NH, 128, C.addressof(groups[0]), G.st()) == rd.ERR_UNSUPPORTED
    bad = rd.shard_group(2, [rd.ptr(b) for b in bufs])
    assert lib.rd_attn_shard_merge(rd.ptr(out), None, NH, HD, C.addressof(bad), G.st()) == rd.ERR_SHAPE
    bad = rd.shard_group(0, [rd.ptr(bufs[0]), rd.ptr(bufs[1]) + 4])
    assert lib.rd_attn_shard_merge(rd.ptr(out), None, NH, HD, C.addressof(bad), G.st()) == rd.ERR_ALIGN
    bad = rd.shard_group(0, [rd.ptr(bufs[0])] * 9)
    assert lib.rd_attn_shard_merge(rd.ptr(out), None, NH, HD, C.addressof(bad), G.st()) == rd.ERR_SHAPE
    assert lib.rd_shard_xbuf_bytes(NH, HD, 9) == 0
    torch.cuda.synchronize()
