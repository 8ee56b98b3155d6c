"""Generates the golden vectors in this directory.

Every expected value here is produced by the REFERENCE project's own kernels
(kv_store_row_kernel, rope_kernel, attn_kernel, attn_split_kernel,
attn_merge_kernel, attn_batch_kernel, attn_split_batch_kernel,
attn_fa2_prefill_kernel, sigmoid_gate_kernel, rms_norm_kernel and the fp16 helpers), executed on the
CPU by oracle/_ref/librd_ref.so. It therefore only runs where the reference checkout
is present (``make -C oracle ref``); the .npz files it writes are committed and are
what the tests read.

    python tests/golden/gen_golden.py

Inputs come from numpy's PCG64 with fixed seeds plus hand-built hostile rows; they
are stored beside the outputs so that no test depends on regenerating them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.oracle import F16, F32, Q4_0, Q4_1, Q5_0, Q8_0, TYPE_NAMES, Reference  # noqa: E402

NH, NKV, HD = 24, 4, 256
SCALE = 1.0 / 16.0


def hostile_rows(rng):
    """Two repetitions of eight 256-wide rows, each unfair to some format: uniform,
    all-positive, single outlier, constant, zeros, +-1 alternation, bell-shaped,
    wide range (|x| up to 100). Same families as tests/check_kvquant_gpu.hip:101-137."""
    rows = np.zeros((16, HD), dtype=np.float32)
    for rep in range(2):
        u = rng.uniform(-1, 1, size=(8, HD)).astype(np.float32)
        b = rep * 8
        rows[b + 0] = u[0]
        rows[b + 1] = 0.5 * (u[1] + 1.0)
        rows[b + 2] = 1e-3 * u[2]
        rows[b + 2, 7] = 1.0
        rows[b + 3] = 0.5
        rows[b + 4] = 0.0
        rows[b + 5] = np.where(np.arange(HD) % 2 == 1, -1.0, 1.0)
        rows[b + 6] = 0.25 * rng.uniform(-1, 1, size=(4, HD)).sum(axis=0)
        rows[b + 7] = 100.0 * u[7]
    return rows


def gen_rms_norm(ref):
    """rms_norm_kernel (nn.cuh:23-63) on head-sized rows (the q/k norm of the attention
    layers) and on a 5120-wide row (20 elements per thread), with and without weights."""
    rng = np.random.default_rng(77)
    x = rng.standard_normal((9, HD)).astype(np.float32)
    x[3] = 0.0
    x[4] *= 1e-4
    x[5] *= 300.0
    w = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    xw = rng.standard_normal((2, 5120)).astype(np.float32)
    ww = (1.0 + 0.1 * rng.standard_normal(5120)).astype(np.float32)
    np.savez(os.path.join(HERE, "rms_norm.npz"), x=x, w=w, eps=np.float32(1e-6),
             y_w=ref.rms_norm(x, w, 1e-6), y_now=ref.rms_norm(x, None, 1e-6),
             xw=xw, ww=ww, yw=ref.rms_norm(xw, ww, 1e-5))


def main():
    ref = Reference()
    if len(sys.argv) > 1 and sys.argv[1] == "rms_norm":   # only this file (keeps the others' bytes)
        gen_rms_norm(ref)
        return
    gen_rms_norm(ref)
    rng = np.random.default_rng(20250916)

    # ---- fp16 conversion: a spread of magnitudes incl. subnormal/overflow edges
    xs = np.concatenate([rng.standard_normal(64).astype(np.float32) * s
                         for s in (1e-8, 6e-8, 1e-6, 6.1e-5, 1e-3, 1.0, 100.0, 6.5e4, 1e6)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65520.0, 65519.0, 5.96e-8, 2.98e-8,
                                       2.9802325e-8, 8.9406967e-8], dtype=np.float32)])
    h = np.array([ref.float_to_fp16(x) for x in xs], dtype=np.uint16)
    hs = np.arange(0, 0x7C00, 37, dtype=np.uint16)
    hs = np.concatenate([hs, hs | 0x8000, np.arange(0, 1100, dtype=np.uint16)])
    f = np.array([ref.fp16_to_float(v) for v in hs], dtype=np.float32)
    np.savez(os.path.join(HERE, "fp16.npz"), f32_in=xs, f16_out=h, f16_in=hs, f32_out=f)

    # ---- KV append (quantizers), all six storage types
    rows = hostile_rows(rng)
    gauss = rng.standard_normal((16, HD)).astype(np.float32)
    src = np.concatenate([rows, gauss]).astype(np.float32)
    out = {"src": src}
    for t in (F32, F16, Q8_0, Q4_0, Q5_0, Q4_1):
        out["bytes_" + TYPE_NAMES[t]] = ref.kv_store_rows(t, src)
        out["row_bytes_" + TYPE_NAMES[t]] = np.int64(ref.row_bytes(t, HD))
    np.savez(os.path.join(HERE, "kv_store.npz"), **out)

    # ---- synthetic-cache hash
    idx = np.array([0, 1, 2, 255, 256, 1000003, 2**31 - 1, 2**32 - 1], dtype=np.uint64)
    seeds = np.array([3, 11, 22, 0xDEADBEEF], dtype=np.uint64)
    vals = np.array([[ref.kv_rand(int(i), int(s)) for i in idx] for s in seeds], dtype=np.float32)
    fill = {"idx": idx, "seeds": seeds, "vals": vals}
    for t in (F32, F16, Q8_0, Q5_0, Q4_1):  # the reference's q4_0 fill is racy: no fixture
        fill["fill_" + TYPE_NAMES[t]] = ref.kv_fill(t, 6, HD, 11)
    np.savez(os.path.join(HERE, "kv_fill.npz"), **fill)

    # ---- RoPE (K-shaped: 4 heads), positions up to the long-context end
    x = rng.standard_normal((6, NKV, HD)).astype(np.float32)
    pos = np.array([0, 3, 17, 4095, 131000, 262143], dtype=np.int32)
    np.savez(os.path.join(HERE, "rope.npz"), x=x, pos=pos, out=ref.rope(x, pos))

    # ---- sigmoid gate
    g = (4.0 * rng.standard_normal(512)).astype(np.float32)
    y = rng.standard_normal(512).astype(np.float32)
    g2, y2 = ref.sigmoid_gate(g, y)
    np.savez(os.path.join(HERE, "gate.npz"), g=g, y=y, g_out=g2, y_out=y2)

    # ---- merge: finite / tail-empty / all-empty / extremal (+-20) partials
    merge = {}
    for name in ("finite", "tail_empty", "all_empty", "extremal"):
        ns = 8
        p = np.zeros((4, ns, 2 + HD), dtype=np.float32)
        for hh in range(4):
            for s in range(ns):
                empty = name == "all_empty" or (name == "tail_empty" and s >= ns - ns // 2)
                if empty:
                    p[hh, s, 0] = -np.inf
                    continue
                if name == "extremal":
                    p[hh, s, 0] = (20.0 if s % 2 else -20.0) + rng.uniform(-1, 1)
                else:
                    p[hh, s, 0] = 4.0 * rng.uniform(-1, 1)
                p[hh, s, 1] = 1.0 + abs(rng.uniform(-1, 1)) * 10.0
                p[hh, s, 2:] = 2.0 * rng.uniform(-1, 1, size=HD)
        merge["partial_" + name] = p
        merge["out_" + name] = ref.attn_merge(p)
    np.savez(os.path.join(HERE, "merge.npz"), **merge)

    # ---- single-token attention, unsplit and split (reference's strided partials).
    # The three headline type pairs use the full 24/4 head shape and keep the split
    # partial records; the rest use one KV head with its 6 query heads to stay small.
    cases = [(F16, F16, 40, 24), (Q8_0, Q8_0, 33, 24), (Q4_0, Q4_0, 70, 24), (F32, F32, 9, 6),
             (Q8_0, F16, 50, 6), (Q4_0, Q8_0, 17, 6), (F16, Q4_0, 1, 6), (Q4_0, F16, 1, 6),
             (Q8_0, F32, 1, 6), (F32, Q8_0, 1, 6), (Q5_0, Q4_1, 20, 6)]
    attn = {}
    for i, (kt, vt, n, nh) in enumerate(cases):
        nkv = nh // 6
        K = rng.standard_normal((n, nkv, HD)).astype(np.float32)
        V = rng.standard_normal((n, nkv, HD)).astype(np.float32)
        q = rng.standard_normal((nh, HD)).astype(np.float32)
        kc, vc = ref.kv_store_rows(kt, K), ref.kv_store_rows(vt, V)
        o = ref.attn(q, kc, vc, n - 1, nkv, SCALE, kt, vt)
        o4, p4 = ref.attn_split(q, kc, vc, n - 1, nkv, SCALE, kt, vt, 4)
        attn.update({f"c{i}_kt": np.int32(kt), f"c{i}_vt": np.int32(vt), f"c{i}_n": np.int32(n),
                     f"c{i}_q": q, f"c{i}_k": kc, f"c{i}_v": vc, f"c{i}_out": o,
                     f"c{i}_out_split4": o4})
        if nh == 24:
            attn[f"c{i}_partial4"] = p4
    attn["n_cases"] = np.int32(len(cases))
    np.savez(os.path.join(HERE, "attn_decode.npz"), **attn)

    # ---- multi-token (chunk / speculative-verify) attention, 6 query heads on 1 KV head
    batch = {}
    # the reference's own check shape: 16 tokens at positions 0..15, f16 cache
    n = 16
    K = rng.standard_normal((n, 1, HD)).astype(np.float32)
    V = rng.standard_normal((n, 1, HD)).astype(np.float32)
    q = rng.standard_normal((n, 6, HD)).astype(np.float32)
    kc, vc = ref.kv_store_rows(F16, K), ref.kv_store_rows(F16, V)
    pos = np.arange(n, dtype=np.int32)
    batch.update(p_q=q, p_k=kc, p_v=vc, p_pos=pos,
                 p_out=ref.attn_batch(q, kc, vc, pos, 1, SCALE, F16, F16))
    # verify: 4 tokens at the end of a 60-key context, K q8_0 / V f16, split and unsplit
    n = 60
    K = rng.standard_normal((n, 1, HD)).astype(np.float32)
    V = rng.standard_normal((n, 1, HD)).astype(np.float32)
    q = rng.standard_normal((4, 6, HD)).astype(np.float32)
    kc, vc = ref.kv_store_rows(Q8_0, K), ref.kv_store_rows(F16, V)
    pos = np.arange(n - 4, n, dtype=np.int32)
    batch.update(v_q=q, v_k=kc, v_v=vc, v_pos=pos,
                 v_out=ref.attn_batch(q, kc, vc, pos, 1, SCALE, Q8_0, F16),
                 v_out_split2=ref.attn_split_batch(q, kc, vc, pos, 1, SCALE, Q8_0, F16, 2))
    np.savez(os.path.join(HERE, "attn_batch.npz"), **batch)

    # ---- FA2-style prefill tile kernel (f16/f16, one KV head with its 6 query heads)
    n_q, pos0 = 16, 56
    keys_total = pos0 + n_q
    K = rng.standard_normal((keys_total, 1, HD)).astype(np.float32)
    V = rng.standard_normal((keys_total, 1, HD)).astype(np.float32)
    q = rng.standard_normal((n_q, 6, HD)).astype(np.float32)
    kc, vc = ref.kv_store_rows(F16, K), ref.kv_store_rows(F16, V)
    pos = np.arange(pos0, keys_total, dtype=np.int32)
    o = ref.fa2_prefill(q, kc, vc, pos, keys_total - 1, keys_total, 1, SCALE)
    np.savez(os.path.join(HERE, "fa2_prefill.npz"), q=q, k=kc, v=vc, pos=pos, out=o,
             usable=np.array([ref.fa2_prefill_usable(F16, F16, 512, 1536, 24, 4, 256),
                              ref.fa2_prefill_usable(F16, F16, 512, 0, 24, 4, 256),
                              ref.fa2_prefill_usable(Q8_0, F16, 512, 1536, 24, 4, 256),
                              ref.fa2_prefill_usable(F16, F16, 256, 2048, 24, 4, 256),
                              ref.fa2_prefill_usable(F16, F16, 512, 7680, 24, 4, 256),
                              ref.fa2_prefill_usable(F16, F16, 512, 7681, 24, 4, 256)]))

    # ---- tables
    np.savez(os.path.join(HERE, "tables.npz"),
             row_bytes=np.array([ref.row_bytes(t, HD) for t in range(6)], dtype=np.int64),
             parse=np.array([ref.kv_type_parse(nm) if ref.kv_type_parse(nm) is not None else -1
                             for nm in ("f32", "f16", "q8_0", "q4_0", "q5_0", "q4_1", "q5_1", "")],
                            dtype=np.int32),
             split_wpb=np.array([ref.lib.ref_attn_split_wpb(s) for s in range(1, 33)], dtype=np.int32),
             partial_bytes=np.array([ref.lib.ref_attn_partial_bytes(24, 256, s) for s in (1, 4, 16)],
                                    dtype=np.int64))
    total = sum(os.path.getsize(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith(".npz"))
    print("golden vectors written, total bytes:", total)


if __name__ == "__main__":
    main()
