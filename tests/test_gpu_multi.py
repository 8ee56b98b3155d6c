"""Many sequences in one launch (rd_attn_decode_multi) against the CPU oracle and against
the per-sequence entry points. Same gates as the single-sequence tests: max-abs error
<= 2e-3 and cosine >= 0.9999 against the oracle's f32 attention over the same bytes."""
import ctypes as C

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


def run_multi(G, qs, kcs, vcs, ts, q_len, kt, vt, gates=None, nkv=NKV):
    """qs[i] device [q_len][n_head][256]; kcs / vcs device uint8 caches; ts[i] last key.
    Returns the list of device outputs (and keeps every buffer alive until the sync)."""
    rd, lib = G.rd, G.lib
    n = len(qs)
    n_head = qs[0].shape[1]
    outs = [G.poison(tuple(q.shape)) for q in qs]
    arr = (rd.AttnSeq * n)()
    for i in range(n):
        arr[i].q, arr[i].k, arr[i].v = rd.ptr(qs[i]), rd.ptr(kcs[i]), rd.ptr(vcs[i])
        arr[i].out = rd.ptr(outs[i])
        arr[i].gate = rd.ptr(gates[i]) if gates is not None else None
        arr[i].t = int(ts[i])
    nbytes = lib.rd_attn_multi_workspace_bytes(n, q_len, n_head, HD)
    assert nbytes > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.rd_attn_decode_multi(C.addressof(arr), n, q_len, n_head, nkv, HD, 1 / 16, kt, vt,
                                  rd.ptr(ws), nbytes, G.st())
    rd.check(rc, "rd_attn_decode_multi")
    torch.cuda.synchronize()
    return outs


@pytest.mark.parametrize("kt,vt", [(2, 1), (3, 3), (1, 0), (0, 2)])
@pytest.mark.parametrize("q_len", [1, 4])
def test_ragged_sequences_against_oracle(G, oracle, kt, vt, q_len):
    rng = np.random.default_rng(100 * kt + 10 * vt + q_len)
    lens = [q_len, q_len + 1, 17, 33, 300, 1025, 4097]
    qs, kcs, vcs, want = [], [], [], []
    for n in lens:
        K = rng.standard_normal((n, NKV, HD)).astype(np.float32)
        V = rng.standard_normal((n, NKV, HD)).astype(np.float32)
        q = rng.standard_normal((q_len, NH, HD)).astype(np.float32)
        kc, vc = oracle.kv_store_rows(kt, K), oracle.kv_store_rows(vt, V)
        pos = np.arange(n - q_len, n, dtype=np.int32)
        want.append(oracle.attn(q, kc, vc, pos, NKV, 1 / 16, kt, vt))
        qs.append(G.dev(q))
        kcs.append(G.dev(kc))
        vcs.append(G.dev(vc))
    outs = run_multi(G, qs, kcs, vcs, [n - 1 for n in lens], q_len, kt, vt)
    for n, o, w in zip(lens, outs, want):
        check_attn(G.host(o), w, what=f"{n} keys, q_len {q_len}")
    G.status_ok()


def test_fused_gate_and_small_head_counts(G, oracle):
    rng = np.random.default_rng(5)
    for nkv in (1, 2):
        nh = 6 * nkv
        lens = [40, 700, 64]
        qs, kcs, vcs, gates, want = [], [], [], [], []
        for n in lens:
            K = rng.standard_normal((n, nkv, HD)).astype(np.float32)
            V = rng.standard_normal((n, nkv, HD)).astype(np.float32)
            q = rng.standard_normal((2, nh, HD)).astype(np.float32)
            g = rng.standard_normal((2, nh, HD)).astype(np.float32)
            kc, vc = oracle.kv_store_rows(2, K), oracle.kv_store_rows(3, V)
            y = oracle.attn(q, kc, vc, np.array([n - 2, n - 1], dtype=np.int32), nkv, 1 / 16, 2, 3)
            want.append(oracle.sigmoid_gate(g, y))
            qs.append(G.dev(q))
            kcs.append(G.dev(kc))
            vcs.append(G.dev(vc))
            gates.append(G.dev(g))
        outs = run_multi(G, qs, kcs, vcs, [n - 1 for n in lens], 2, 2, 3, gates=gates, nkv=nkv)
        for o, g, (wg, wy) in zip(outs, gates, want):
            check_attn(G.host(o), wy, what="gated output")
            assert np.abs(G.host(g) - wg).max() <= 1e-6
    G.status_ok()


def test_argument_errors(G):
    rd, lib = G.rd, G.lib
    q = G.poison((1, NH, HD))
    kc = torch.zeros(4 * 1088, dtype=torch.uint8, device="cuda")
    arr = (rd.AttnSeq * 1)()
    arr[0].q, arr[0].k, arr[0].v, arr[0].out, arr[0].t = rd.ptr(q), rd.ptr(kc), rd.ptr(kc), rd.ptr(q), 3
    nbytes = lib.rd_attn_multi_workspace_bytes(1, 1, NH, HD)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    call = lambda a, n, ql, w, wb: lib.rd_attn_decode_multi(a, n, ql, NH, NKV, HD, 1 / 16, 2, 2, w, wb,
                                                            G.st())
    assert call(C.addressof(arr), 0, 1, rd.ptr(ws), nbytes) == rd.OK          # nothing to do
    assert call(None, 1, 1, rd.ptr(ws), nbytes) == rd.ERR_NULL
    assert call(C.addressof(arr), 1, 0, rd.ptr(ws), nbytes) == rd.ERR_SHAPE
    assert call(C.addressof(arr), 1, 1, None, nbytes) == rd.ERR_WORKSPACE
    assert call(C.addressof(arr), 1, 1, rd.ptr(ws), 1024) == rd.ERR_WORKSPACE
    assert call(C.addressof(arr), 1, 1, rd.ptr(ws) + 8, nbytes) == rd.ERR_ALIGN
    assert call(C.addressof(arr), 1, 5, rd.ptr(ws), nbytes) == rd.ERR_SHAPE   # t < q_len - 1
    arr[0].out = None
    assert call(C.addressof(arr), 1, 1, rd.ptr(ws), nbytes) == rd.ERR_NULL
    assert lib.rd_attn_multi_workspace_bytes(0, 1, NH, HD) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("q_len", [1, 4])
def test_batched_decode_64_sequences(G, oracle, q_len):
    """64 sequences, context lengths uniform in [1024, 32768] from seed 7, K q8_0 / V f16
    (caches filled on the device): the one-launch result equals the per-sequence entry
    point on every sequence, and the oracle on eight sequences spread over the lengths."""
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(7)
    lens = rng.integers(1024, 32769, size=64)
    qs, kcs, vcs = [], [], []
    for i, n in enumerate(lens):
        n = int(n)
        kc = torch.empty(n * NKV * 272, dtype=torch.uint8, device="cuda")
        vc = torch.empty(n * NKV * 512, dtype=torch.uint8, device="cuda")
        rd.check(lib.rd_kv_fill(2, rd.ptr(kc), n * NKV, HD, 1000 + i, G.st()))
        rd.check(lib.rd_kv_fill(1, rd.ptr(vc), n * NKV, HD, 2000 + i, G.st()))
        qs.append(G.dev(oracle.kv_fill_values(q_len * NH, HD, 3000 + i).reshape(q_len, NH, HD)))
        kcs.append(kc)
        vcs.append(vc)
    outs = run_multi(G, qs, kcs, vcs, [int(n) - 1 for n in lens], q_len, 2, 1)
    worst = 0.0
    for i, n in enumerate(lens):
        n = int(n)
        pos = G.dev(np.arange(n - q_len, n, dtype=np.int32))
        ref = G.poison(tuple(qs[i].shape))
        rd.check(lib.rd_attn_batch(rd.ptr(qs[i]), rd.ptr(kcs[i]), rd.ptr(vcs[i]), rd.ptr(ref),
                                   rd.ptr(pos), q_len, NH, NKV, HD, 1 / 16, 2, 1, G.st()))
        torch.cuda.synchronize()
        worst = max(worst, float((outs[i] - ref).abs().max()))
    # the same kernel with a different key split: only the merge order differs
    assert worst <= 2e-5, worst
    for i in np.argsort(lens)[::8]:   # eight sequences spread over the whole length range
        n = int(lens[i])
        pos = np.arange(n - q_len, n, dtype=np.int32)
        want = oracle.attn(G.host(qs[i]), G.host(kcs[i]), G.host(vcs[i]), pos, NKV, 1 / 16, 2, 1)
        check_attn(G.host(outs[i]), want, what=f"sequence {i} ({n} keys)")
    G.status_ok()


def test_plan_and_launch_captured_with_a_growing_context(G, oracle):
    """rd_attn_multi_plan into pinned memory + rd_attn_multi_launch captured ONCE: every
    replay reads the plan as rewritten for that step (contexts one key longer each time,
    item count padded to a fixed number), and matches the oracle."""
    rd, lib = G.rd, G.lib
    kt = vt = 3
    rng = np.random.default_rng(77)
    caps, t0 = [40, 700, 3000], [20, 650, 2900]
    n = len(caps)
    Ks = [rng.standard_normal((c, NKV, HD)).astype(np.float32) for c in caps]
    Vs = [rng.standard_normal((c, NKV, HD)).astype(np.float32) for c in caps]
    kcs = [oracle.kv_store_rows(kt, K) for K in Ks]
    vcs = [oracle.kv_store_rows(vt, V) for V in Vs]
    dks, dvs = [G.dev(k) for k in kcs], [G.dev(v) for v in vcs]
    qs = [G.dev(rng.standard_normal((1, NH, HD)).astype(np.float32)) for _ in range(n)]
    outs = [G.poison((1, NH, HD)) for _ in range(n)]
    arr = (rd.AttnSeq * n)()
    for i in range(n):
        arr[i].q, arr[i].k, arr[i].v, arr[i].out = rd.ptr(qs[i]), rd.ptr(dks[i]), rd.ptr(dvs[i]), rd.ptr(outs[i])
    pbytes = lib.rd_attn_multi_plan_bytes(n, 1)
    assert pbytes > 256
    plan = torch.empty(pbytes, dtype=torch.uint8).pin_memory()
    wbytes = lib.rd_attn_multi_workspace_bytes(n, 1, NH, HD)
    ws = torch.empty(wbytes, dtype=torch.uint8, device="cuda")
    pad = 64

    def replan(step):
        for i in range(n):
            arr[i].t = t0[i] + step
        rd.check(lib.rd_attn_multi_plan(C.addressof(arr), n, 1, NH, NKV, HD, kt, vt, pad, plan.data_ptr(), pbytes),
                 "rd_attn_multi_plan")

    replan(0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rd.check(lib.rd_attn_multi_launch(plan.data_ptr(), 1 / 16, rd.ptr(ws), wbytes, rd.stream_ptr()))   # warm-up
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        rd.check(lib.rd_attn_multi_launch(plan.data_ptr(), 1 / 16, rd.ptr(ws), wbytes, rd.stream_ptr()))
    for step in (0, 1, 7, 19):
        replan(step)
        for o in outs:
            o.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        for i in range(n):
            t = t0[i] + step
            q = G.host(qs[i])
            want = oracle.attn(q, kcs[i], vcs[i], np.asarray([t], dtype=np.int32), NKV, 1 / 16, kt, vt)
            check_attn(G.host(outs[i]), want, what=f"step {step}, sequence {i}")
    G.status_ok()
    # a plan that needs more items than the padding allows is refused, not truncated
    assert lib.rd_attn_multi_plan(C.addressof(arr), n, 1, NH, NKV, HD, kt, vt, 2, plan.data_ptr(), pbytes) == rd.ERR_LIMIT
    assert lib.rd_attn_multi_plan(C.addressof(arr), n, 1, NH, NKV, HD, kt, vt, pad, plan.data_ptr(), 128) == rd.ERR_WORKSPACE
    assert lib.rd_attn_multi_launch(None, 1 / 16, rd.ptr(ws), wbytes, G.st()) == rd.ERR_NULL
    bad = torch.zeros(pbytes, dtype=torch.uint8)
    assert lib.rd_attn_multi_launch(bad.data_ptr(), 1 / 16, rd.ptr(ws), wbytes, G.st()) == rd.ERR_SHAPE
