"""The library's decode plan and split rules against the committed table (CPU only: host
arithmetic of the C-ABI library), the analogue of the reference's check-tuning gate."""
import ctypes as C
import importlib
import os

from tests.golden.gen_plan import table

HERE = os.path.dirname(os.path.abspath(__file__))


def test_plan_matches_committed_table():
    want = open(os.path.join(HERE, "golden", "b200_plan.txt")).read()
    assert table() == want


def test_reference_split_rule():
    """Graph::attn_splits_for (graph.cuh:495-526): 1 below 512 keys; ceil(96 / n_head) for
    f16 / f32 caches; min(16, keys / 512) for quantized ones; a forced count wins, capped."""
    rd = importlib.import_module("rdna4-infer_b200")
    f = rd.lib.rd_attn_splits_for
    assert f(511, 3, 3, 24, 0) == 1 and f(0, 1, 1, 24, 0) == 1
    assert f(512, 3, 3, 24, 0) == 1 and f(1024, 2, 1, 24, 0) == 2 and f(4096, 2, 2, 24, 0) == 8
    assert f(131001, 3, 3, 24, 0) == 16 and f(8192, 4, 5, 24, 0) == 16
    assert f(4096, 1, 1, 24, 0) == 4 and f(131072, 0, 1, 24, 0) == 4     # 96 CTAs / 24 heads
    assert f(4096, 1, 1, 6, 0) == 16 and f(4096, 1, 1, 96, 0) == 1 and f(4096, 1, 1, 200, 0) == 1
    assert f(100, 1, 1, 24, 1) == 1 and f(100000, 3, 3, 24, 3) == 3 and f(100, 3, 3, 24, 99) == 16
    assert f(100, 6, 1, 24, 0) == rd.ERR_TYPE and f(-1, 1, 1, 24, 0) == rd.ERR_SHAPE


def test_plan_properties():
    rd = importlib.import_module("rdna4-infer_b200")
    L = rd.lib
    tile, stages, sp = C.c_int(), C.c_int(), C.c_int()
    plan = lambda n, n_tok, kt, vt, sms: (L.rd_attn_plan(n, n_tok, 4, kt, vt, sms, C.addressof(tile),
                                                         C.addressof(stages), C.addressof(sp)),
                                          tile.value, stages.value, sp.value)
    assert plan(131001, 1, 3, 3, 148) == (0, 48, 3, 148)        # the headline shape: one CTA per SM
    assert plan(131001, 1, 3, 3, 132)[3] == 132
    assert plan(100, 1, 3, 3, 148)[3] == 3                      # never more splits than key tiles
    assert plan(0, 1, 3, 3, 148)[3] == 1
    assert plan(32768, 4, 2, 1, 148)[3] == 37                   # 4 tokens share the SMs
    for kt in range(6):
        for vt in range(6):
            rc, t, s, _ = plan(4096, 1, kt, vt, 148)
            assert rc == 0 and t in (16, 32, 48) and 1 <= s <= 8
    assert L.rd_attn_plan(10, 1, 3, 3, 3, 148, None, None, None) == rd.ERR_UNSUPPORTED
    assert L.rd_attn_plan(10, 0, 4, 3, 3, 148, None, None, None) == rd.ERR_SHAPE
    assert L.rd_attn_plan(10, 1, 4, 3, 3, 148, None, None, None) == rd.OK


def test_prefill_plan_properties():
    """rd_attn_prefill_plan: one split unless filling the idle SMs pays; never more CTAs than
    two waves' worth for the reference's FA2 window; argument errors."""
    rd = importlib.import_module("rdna4-infer_b200")
    L = rd.lib
    z, ctas = C.c_int(), C.c_int()
    plan = lambda n_q, keys, sms=148: (L.rd_attn_prefill_plan(n_q, keys, 24, sms, C.addressof(z), C.addressof(ctas)),
                                       z.value, ctas.value)
    assert plan(512, 512) == (0, 1, 96) and plan(512, 4096) == (0, 1, 96)
    assert plan(512, 8192) == (0, 3, 288)                       # 96 -> 288 CTAs: two full waves of 148 SMs
    assert plan(8192, 8192) == (0, 1, 64 * 24)                  # enough token tiles already
    for keys in (1, 127, 128, 129, 1000, 5000, 100000):
        rc, s, c = plan(512, keys)
        assert rc == 0 and 1 <= s <= 8 and c == 4 * 24 * s
        assert s == 1 or (keys + 127) // 128 // s >= 8          # a split keeps at least 8 tiles per CTA
    assert plan(512, 8192, 96)[1] == 1                          # 96 SMs are full with one wave
    assert L.rd_attn_prefill_plan(0, 10, 24, 148, None, None) == rd.ERR_SHAPE
    assert L.rd_attn_prefill_plan(10, 0, 24, 148, None, None) == rd.ERR_SHAPE
    assert L.rd_attn_prefill_plan(10, 10, 24, 148, None, None) == rd.OK
