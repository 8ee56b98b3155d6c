"""rd_attn_decode_append_ws: the newest row is stored by the first CTAs of the split-KV
launch and attended by the merge. Against rd_kv_append followed by rd_attn_decode_ws (cache
bytes equal, output within the attention tolerance) and against the oracle."""
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


@pytest.mark.parametrize("kt,vt", [(3, 3), (2, 1), (1, 0), (4, 5), (0, 2)])
@pytest.mark.parametrize("t", [0, 1, 47, 48, 1000, 20011])
def test_append_decode_equals_separate_calls(G, oracle, kt, vt, t):
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(100 * kt + 10 * vt + t)
    rk, rv = rd.row_bytes(kt) * NKV, rd.row_bytes(vt) * NKV
    st = G.st()
    kc = torch.zeros((t + 1) * rk, dtype=torch.uint8, device="cuda")
    vc = torch.zeros((t + 1) * rv, dtype=torch.uint8, device="cuda")
    if t > 0:
        rd.check(lib.rd_kv_fill(kt, rd.ptr(kc), t * NKV, HD, 7, st))
        rd.check(lib.rd_kv_fill(vt, rd.ptr(vc), t * NKV, HD, 8, st))
    kc2, vc2 = kc.clone(), vc.clone()
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    kn = (2.0 * rng.standard_normal((NKV, HD))).astype(np.float32)
    vn = rng.standard_normal((NKV, HD)).astype(np.float32)
    gate = rng.standard_normal((NH, HD)).astype(np.float32)
    dq, dkn, dvn = G.dev(q), G.dev(kn), G.dev(vn)
    nbytes = lib.rd_attn_workspace_bytes(1, NH, HD)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    # separate calls
    g0, out0 = G.dev(gate), G.poison((NH, HD))
    rd.check(lib.rd_kv_append(kt, vt, rd.ptr(dkn), rd.ptr(dvn), rd.ptr(kc) + t * rk, rd.ptr(vc) + t * rv, 1, NKV, HD,
                              None, 0, 0.0, st))
    rd.check(lib.rd_attn_decode_ws(rd.ptr(dq), rd.ptr(kc), rd.ptr(vc), rd.ptr(out0), None, 0, t, NH, NKV, HD, 1 / 16,
                                   kt, vt, 1, rd.ptr(g0), rd.ptr(ws), nbytes, st))
    # fused
    g1, out1 = G.dev(gate), G.poison((NH, HD))
    rd.check(lib.rd_attn_decode_append_ws(rd.ptr(dq), rd.ptr(dkn), rd.ptr(dvn), rd.ptr(kc2), rd.ptr(vc2), rd.ptr(out1),
                                          t, NH, NKV, HD, 1 / 16, kt, vt, rd.ptr(g1), rd.ptr(ws), nbytes, st))
    torch.cuda.synchronize()
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert torch.equal(g0, g1)
    check_attn(G.host(out1), G.host(out0), what="fused vs separate")
    _, want = oracle.sigmoid_gate(gate, oracle.attn(q[None], G.host(kc), G.host(vc), [t], NKV, 1 / 16, kt, vt)[0])
    check_attn(G.host(out1), want, what="fused vs oracle")
    G.status_ok()


def test_append_decode_argument_errors(G):
    rd, lib = G.rd, G.lib
    keep = [torch.zeros(NH * HD, device="cuda"), torch.zeros(NH * HD, device="cuda"),
            torch.zeros(4096, dtype=torch.uint8, device="cuda")]     # stay alive for the whole test
    p, p2, c = rd.ptr(keep[0]), rd.ptr(keep[1]), rd.ptr(keep[2])
    ws = torch.empty(lib.rd_attn_workspace_bytes(1, NH, HD), dtype=torch.uint8, device="cuda")
    call = lambda q, out, t=0, w=rd.ptr(ws), wb=ws.numel(): lib.rd_attn_decode_append_ws(
        q, p, p, c, c, out, t, NH, NKV, HD, 1 / 16, 3, 3, None, w, wb, G.st())
    assert call(p, p) == rd.ERR_UNSUPPORTED          # q aliases out
    assert call(p, p2, t=-1) == rd.ERR_SHAPE
    assert call(None, p2) == rd.ERR_NULL
    assert call(p, p2, w=None) == rd.ERR_WORKSPACE
    assert call(p, p2, wb=16) == rd.ERR_WORKSPACE
    assert call(p, p2) == rd.OK
    torch.cuda.synchronize()
