"""rd_attn_decode_noalloc: the decode entry point for callers that must not allocate.

A serving process whose memory manager owns the whole device, or a decode loop that
cannot afford the device-wide synchronisation of cudaMalloc, cannot use the entry points
that grow a workspace on first use. This entry keeps its partial records in a fixed
array inside the library instead. The test drives it through the C ABI on two calls in
a row (the array keeps the first call's records, so the second call also proves that
nothing depends on its initial contents) and compares with the allocating entry point
on the same inputs, to the tolerance of the other attention tests. The file name sorts
last on purpose: a run that stops at the first failure has then already run the rest.
"""
import numpy as np
import pytest

from tests.conftest import check_attn


@pytest.mark.gpu
def test_noalloc_matches_allocating_entry_on_two_calls_in_a_row(cuda, rd, oracle):
    import torch
    from tests import gpu_util as G

    L = rd.lib
    rng = np.random.default_rng(77)
    cases = [(3, 3, 5000), (2, 1, 333)]   # (K type, V type, keys): q4_0/q4_0 and q8_0/f16
    for call, (kt, vt, n) in enumerate(cases):
        K = rng.standard_normal((n, 4, 256)).astype(np.float32)
        V = rng.standard_normal((n, 4, 256)).astype(np.float32)
        q = rng.standard_normal((24, 256)).astype(np.float32)
        gate = rng.standard_normal((24, 256)).astype(np.float32)
        kc, vc = oracle.kv_store_rows(kt, K), oracle.kv_store_rows(vt, V)
        dq, dk, dv = G.dev(q), G.dev(kc), G.dev(vc)
        # existing entry point (allocating workspace), no gate
        want = G.attn_decode(q, kc, vc, n - 1, kt, vt, n_splits=16)
        # new entry point, without and with the fused gate
        out = G.poison((24, 256))
        rd.check(L.rd_attn_decode_noalloc(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), n - 1, 24, 4,
                                          256, 1 / 16, kt, vt, None, G.st()), "rd_attn_decode_noalloc")
        torch.cuda.synchronize()
        check_attn(G.host(out), want, what=f"no-alloc call {call}")
        dg = G.dev(gate)
        out2 = G.poison((24, 256))
        rd.check(L.rd_attn_decode_noalloc(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out2), n - 1, 24, 4,
                                          256, 1 / 16, kt, vt, rd.ptr(dg), G.st()), "rd_attn_decode_noalloc+gate")
        torch.cuda.synchronize()
        sg, gated = oracle.sigmoid_gate(gate, want)
        check_attn(G.host(out2), gated, what=f"no-alloc gated call {call}")
        assert np.abs(G.host(dg) - sg).max() <= 2e-7
    assert L.rd_device_status() == rd.OK


def test_noalloc_rejects_sizes_beyond_its_fixed_maximum(rd):
    buf = np.zeros(64, dtype=np.float32)
    p = buf.ctypes.data   # never dereferenced: the limit check comes first
    # 48 query heads: beyond the stated maximum of 24, refused as a limit before anything else
    assert rd.lib.rd_attn_decode_noalloc(p, p, p, p, 3, 48, 8, 256, 0.0625, rd.F16, rd.F16, None,
                                         None) == rd.ERR_LIMIT
    assert rd.lib.rd_attn_decode_noalloc(p, p, p, p, 3, 25, 4, 256, 0.0625, rd.F16, rd.F16, None,
                                         None) == rd.ERR_LIMIT
    assert rd.lib.rd_attn_decode_noalloc(p, p, p, None, 3, 24, 4, 256, 0.0625, rd.F16, rd.F16, None,
                                         None) == rd.ERR_NULL
    assert "maximum" in rd.strerror(rd.ERR_LIMIT)



def test_noalloc_split_cap_keeps_the_records_inside_the_fixed_array(rd):
    """The entry plans with at most RD_NOALLOC_MAX_SPLITS (160) "SMs": on any part, heads x
    splits x 258 floats stays inside the 24 x 160 x 258 array. rd_attn_plan is that planner
    (host arithmetic when the SM count is given)."""
    import ctypes as C
    cap, heads = 160, 24
    for sms in (148, 160, 161, 192, 1024):
        for n_keys in (1, 500, 131001, 10 ** 7):
            n = C.c_int(0)
            assert rd.lib.rd_attn_plan(n_keys, 1, 4, rd.Q4_0, rd.Q4_0, min(sms, cap), None, None, C.byref(n)) == rd.OK
            assert 1 <= n.value <= cap
            assert heads * n.value * 258 <= heads * cap * 258
