"""benchmark configs 1 and 2 as named parity cases (config 3 is test_gpu_prefill.py::
test_prefill_fused_rope_and_gate, config 4 test_gpu_attn.py::test_long_context_q4_0_full_size,
config 5 test_gpu_multi.py::test_batched_decode_64_sequences). Inputs are seeded synthetic
N(0,1) tensors of the stated shapes; gates: KV bytes as the oracle's quantizer writes them,
attention max-abs <= 2e-3 and cosine >= 0.9999 against the f32 CPU oracle."""
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


def test_config1_decode_4096_f16_rope_gate(G, oracle):
    """1 sequence, q_len 1, context 4096, K and V f16, rotary on the first 64 dims
    (theta 1e7), sigmoid output gate: append kernel (fused K RoPE) -> rd_rope on Q ->
    decode with the gate fused into the merge."""
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(0)
    n = 4096
    K = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    q = rng.standard_normal((1, NH, HD)).astype(np.float32)
    gate = rng.standard_normal((NH, HD)).astype(np.float32)
    pos = np.arange(n, dtype=np.int32)
    # oracle: rotate K rows by their position and Q by the last one, store f16, attend, gate
    kc_want = oracle.kv_store_rows(1, oracle.rope(K, pos))
    vc_want = oracle.kv_store_rows(1, V)
    q_rot = oracle.rope(q, pos[-1:])
    g_want, y_want = oracle.sigmoid_gate(gate, oracle.attn(q_rot, kc_want, vc_want, [n - 1], NKV, 1 / 16, 1, 1)[0])
    # GPU
    dK, dV, dpos = G.dev(K), G.dev(V), G.dev(pos)
    kc = torch.empty(n * NKV * 512, dtype=torch.uint8, device="cuda")
    vc = torch.empty_like(kc)
    rd.check(lib.rd_kv_append(1, 1, rd.ptr(dK), rd.ptr(dV), rd.ptr(kc), rd.ptr(vc), n, NKV, HD, rd.ptr(dpos), 64,
                              1e7, G.st()))
    dq, dg = G.dev(q), G.dev(gate)
    rd.check(lib.rd_rope(rd.ptr(dq), 1, NH, HD, 64, 1e7, rd.ptr(dpos) + 4 * (n - 1), G.st()))
    nbytes = lib.rd_attn_workspace_bytes(1, NH, HD)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = G.poison((NH, HD))
    rd.check(lib.rd_attn_decode_ws(rd.ptr(dq), rd.ptr(kc), rd.ptr(vc), rd.ptr(out), None, 0, n - 1, NH, NKV, HD,
                                   1 / 16, 1, 1, 4, rd.ptr(dg), rd.ptr(ws), nbytes, G.st()))
    torch.cuda.synchronize()
    assert np.array_equal(G.host(vc), vc_want)
    assert (G.host(kc) != kc_want).mean() < 2e-2       # sin/cos rounding moves the odd f16 ulp
    check_attn(G.host(out), y_want, what="config 1")
    assert np.abs(G.host(dg) - g_want).max() <= 1e-6
    G.status_ok()


def test_config2_decode_32768_q8_0_split_merge(G, oracle):
    """1 sequence, q_len 1, context 32768, K and V q8_0 produced by quantizing N(0,1) rows
    with the append kernel; split-KV with LSE merge, both through the one-call entry and as
    16 caller-visible partial records merged by rd_attn_merge."""
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(2)
    n = 32768
    K = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    kc_want, vc_want = oracle.kv_store_rows(2, K), oracle.kv_store_rows(2, V)
    want = oracle.attn(q[None], kc_want, vc_want, [n - 1], NKV, 1 / 16, 2, 2)[0]
    kc = torch.empty(n * NKV * 272, dtype=torch.uint8, device="cuda")
    vc = torch.empty_like(kc)
    dK, dV = G.dev(K), G.dev(V)
    rd.check(lib.rd_kv_append(2, 2, rd.ptr(dK), rd.ptr(dV), rd.ptr(kc), rd.ptr(vc), n, NKV, HD, None, 0, 0.0,
                              G.st()))
    torch.cuda.synchronize()
    assert np.array_equal(G.host(kc), kc_want) and np.array_equal(G.host(vc), vc_want)   # bit-exact
    check_attn(G.attn_decode(q, kc_want, vc_want, n - 1, 2, 2, n_splits=16), want, what="config 2, one call")
    part = G.attn_partials(q, kc_want, vc_want, n - 1, 2, 2, 16)
    assert part.shape == (NH, 16, 2 + HD)
    check_attn(G.merge(part), want, what="config 2, 16 records + rd_attn_merge")
    check_attn(oracle.attn_merge(part), want, what="config 2, 16 records + oracle merge")
    G.status_ok()
