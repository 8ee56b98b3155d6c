"""The CPU oracle against the golden vectors.

The vectors in tests/golden were produced by the reference project's own kernels
executed on the CPU (tests/golden/gen_golden.py), so these tests pin the plain-C
restatement to the reference: bit-exact for bytes, a few ulp for f32 attention
(the reference accumulates with an online softmax in a different order).
"""
import numpy as np
import pytest

from oracle.oracle import F16, F32, Q4_0, Q4_1, Q5_0, Q8_0, TYPE_NAMES

ALL_TYPES = (F32, F16, Q8_0, Q4_0, Q5_0, Q4_1)


def test_fp16_conversions_bit_exact(oracle, golden):
    g = golden("fp16")
    got = np.array([oracle.float_to_fp16(x) for x in g["f32_in"]], dtype=np.uint16)
    assert (got == g["f16_out"]).all()
    back = np.array([oracle.fp16_to_float(h) for h in g["f16_in"]], dtype=np.float32)
    assert (back.view(np.uint32) == g["f32_out"].view(np.uint32)).all()


@pytest.mark.parametrize("t", ALL_TYPES, ids=[TYPE_NAMES[t] for t in ALL_TYPES])
def test_kv_store_bytes_bit_exact(oracle, golden, t):
    g = golden("kv_store")
    got = oracle.kv_store_rows(t, g["src"])
    want = g["bytes_" + TYPE_NAMES[t]]
    assert got.size == want.size == g["src"].shape[0] * int(g["row_bytes_" + TYPE_NAMES[t]])
    assert int((got != want).sum()) == 0


def test_tables(oracle, golden):
    g = golden("tables")
    assert [oracle.row_bytes(t, 256) for t in range(6)] == list(g["row_bytes"])
    assert list(g["row_bytes"]) == [1024, 512, 272, 144, 176, 160]
    # exact cache budgets at 131072 tokens, 16 layers x 4 kv heads (tests/check_kvtype.hip:157-163)
    per_tok = lambda k, v: 16 * 4 * (oracle.row_bytes(k) + oracle.row_bytes(v))
    assert 131072 * per_tok(F16, F16) == 8589934592
    assert 131072 * per_tok(Q8_0, Q8_0) == 4563402752
    assert 131072 * per_tok(Q4_0, Q4_0) == 2415919104
    assert 131072 * per_tok(Q5_0, Q4_1) == 2818572288


def test_kv_rand_and_fill(oracle, golden):
    g = golden("kv_fill")
    for si, s in enumerate(g["seeds"]):
        for ii, i in enumerate(g["idx"]):
            assert np.float32(oracle.kv_rand(int(i), int(s))) == g["vals"][si, ii]
    for t in (F32, F16, Q8_0, Q5_0, Q4_1):
        assert (oracle.kv_fill(t, 6, 256, 11) == g["fill_" + TYPE_NAMES[t]]).all()
    # q4_0: the contract is "hash values through the real quantizer"
    vals = oracle.kv_fill_values(6, 256, 11)
    assert (oracle.kv_fill(Q4_0, 6, 256, 11) == oracle.kv_store_rows(Q4_0, vals)).all()


def test_rope_matches_reference(oracle, golden):
    g = golden("rope")
    got = oracle.rope(g["x"], g["pos"])
    # same libm on the same host: identical; allow the reference's own gate otherwise
    num = np.linalg.norm(got.astype(np.float64) - g["out"])
    assert num / np.linalg.norm(g["out"].astype(np.float64)) < 1e-6


def test_gate_matches_reference(oracle, golden):
    g = golden("gate")
    g2, y2 = oracle.sigmoid_gate(g["g"], g["y"])
    assert np.abs(g2 - g["g_out"]).max() <= 1e-7
    assert np.abs(y2 - g["y_out"]).max() <= 1e-6


@pytest.mark.parametrize("mode", ["finite", "tail_empty", "all_empty", "extremal"])
def test_merge_matches_reference(oracle, golden, mode):
    g = golden("merge")
    p, want = g["partial_" + mode], g["out_" + mode]
    got = oracle.attn_merge(p)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-6
    got64 = oracle.attn_merge(p, f64=True)
    assert np.abs(got64 - want).max() <= 2e-6
    if mode == "all_empty":
        assert (got == 0).all()


def test_attn_decode_matches_reference(oracle, golden):
    g = golden("attn_decode")
    for i in range(int(g["n_cases"])):
        kt, vt, n = int(g[f"c{i}_kt"]), int(g[f"c{i}_vt"]), int(g[f"c{i}_n"])
        q, k, v, want = g[f"c{i}_q"], g[f"c{i}_k"], g[f"c{i}_v"], g[f"c{i}_out"]
        nkv = q.shape[0] // 6
        got = oracle.attn(q[None], k, v, [n - 1], nkv, 1 / 16, kt, vt)[0]
        assert np.abs(got - want).max() <= 5e-6, (i, kt, vt, n)
        got64 = oracle.attn(q[None], k, v, [n - 1], nkv, 1 / 16, kt, vt, f64=True)[0]
        assert np.abs(got64 - want).max() <= 5e-6
        # reference split path == reference unsplit path to its own gate
        assert np.abs(g[f"c{i}_out_split4"] - want).max() <= 5e-6
        # merging the oracle's own partial records reproduces the output
        for ns in (1, 3, 4, n + 2):
            part = oracle.attn_partials(q, k, v, 0, n, nkv, 1 / 16, kt, vt, ns)
            assert np.abs(oracle.attn_merge(part) - want).max() <= 5e-6
        if n == 1:
            # one key: the output is exactly the dequantized stored V row (check_rope_gpu.hip:340-393)
            vrow = oracle.kv_dequant_rows(vt, v, nkv, 256)
            for h in range(q.shape[0]):
                assert np.abs(got[h] - vrow[h // 6]).max() < 1e-4


def test_reference_partials_merge_with_oracle_merge(oracle, golden):
    g = golden("attn_decode")
    for i in range(3):
        got = oracle.attn_merge(g[f"c{i}_partial4"])
        assert np.abs(got - g[f"c{i}_out_split4"]).max() <= 1e-6


def test_attn_batch_matches_reference(oracle, golden):
    g = golden("attn_batch")
    got = oracle.attn(g["p_q"], g["p_k"], g["p_v"], g["p_pos"], 1, 1 / 16, F16, F16)
    assert np.abs(got - g["p_out"]).max() <= 5e-6
    got = oracle.attn(g["v_q"], g["v_k"], g["v_v"], g["v_pos"], 1, 1 / 16, Q8_0, F16)
    assert np.abs(got - g["v_out"]).max() <= 5e-6
    assert np.abs(got - g["v_out_split2"]).max() <= 5e-6


def test_fa2_prefill_matches_reference(oracle, golden):
    g = golden("fa2_prefill")
    got = oracle.attn(g["q"], g["k"], g["v"], g["pos"], 1, 1 / 16, F16, F16)
    assert np.abs(got - g["out"]).max() <= 5e-6
    assert list(g["usable"]) == [True, False, False, False, True, False]


def test_empty_and_edge_cases(oracle):
    rng = np.random.default_rng(1)
    q = rng.standard_normal((2, 6, 256)).astype(np.float32)
    k = oracle.kv_store_rows(F16, rng.standard_normal((3, 1, 256)).astype(np.float32))
    out = oracle.attn(q, k, k, [-1, 0], 1, 1 / 16, F16, F16)
    assert (out[0] == 0).all()
    vrow = oracle.kv_dequant_rows(F16, k, 3, 256)[0]
    assert np.abs(out[1] - vrow).max() < 1e-6
    # zero-key shard -> empty sentinel (-inf, 0, 0...)
    part = oracle.attn_partials(q[0], k, k, 2, 2, 1, 1 / 16, F16, F16, 2)
    assert np.isneginf(part[:, :, 0]).all() and (part[:, :, 1:] == 0).all()
    with pytest.raises(ValueError):
        oracle.kv_store_rows(Q4_0, np.zeros(33, dtype=np.float32))


def test_rms_norm_bit_exact(oracle, golden):
    """rms_norm_kernel (nn.cuh:23-63): same fmaf chain per thread, same reduction tree."""
    g = golden("rms_norm")
    eps = float(g["eps"])
    assert np.array_equal(oracle.rms_norm(g["x"], g["w"], eps), g["y_w"])
    assert np.array_equal(oracle.rms_norm(g["x"], None, eps), g["y_now"])
    assert np.array_equal(oracle.rms_norm(g["xw"], g["ww"], 1e-5), g["yw"])
    assert (g["y_w"][3] == 0).all()          # an all-zero row stays zero (eps > 0)
