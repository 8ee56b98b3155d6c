"""Writes b200_plan.txt: the decode plan of the library (tile keys, TMA ring stages, internal
split count) for every K x V type pair at the benchmark context lengths on a 148-SM B200,
and the reference's caller-side split rule for the same shapes. Needs only the built
library (host arithmetic, no GPU):

    python tests/golden/gen_plan.py            # rewrite the golden file
    python tests/golden/gen_plan.py --print    # print the table instead

tests/test_plan_golden.py compares the library against the committed file, as the
reference's check-tuning does for its own tuning table."""
import ctypes as C
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
NAMES = ("f32", "f16", "q8_0", "q4_0", "q5_0", "q4_1")
CONTEXTS = (1, 100, 512, 4096, 32768, 131001)


def table():
    rd = importlib.import_module("rdna4-infer_b200")
    L = rd.lib
    lines = ["# decode plan on 148 SMs, 4 KV heads: K V | tile_keys ring_stages | splits at n_tok=1 per context "
             + " ".join(str(c) for c in CONTEXTS) + " | splits at n_tok=4 | reference rule (24 heads)"]
    for kt in range(6):
        for vt in range(6):
            tile, stages = C.c_int(), C.c_int()
            s1, s4, ref = [], [], []
            for n in CONTEXTS:
                for n_tok, out in ((1, s1), (4, s4)):
                    sp = C.c_int()
                    rd.check(L.rd_attn_plan(n, n_tok, 4, kt, vt, 148, C.addressof(tile), C.addressof(stages),
                                            C.addressof(sp)))
                    out.append(sp.value)
                ref.append(L.rd_attn_splits_for(n, kt, vt, 24, 0))
            lines.append(f"{NAMES[kt]} {NAMES[vt]} | {tile.value} {stages.value} | "
                         + " ".join(map(str, s1)) + " | " + " ".join(map(str, s4)) + " | "
                         + " ".join(map(str, ref)))
    lines.append("# prefill plan on 148 SMs, 24 heads: n_q keys_total | key splits, CTAs of the tile-kernel launch")
    for n_q, keys in ((1, 1), (200, 200), (512, 512), (512, 2048), (512, 4096), (512, 8192), (512, 16384),
                      (512, 131072), (2048, 8192), (8192, 8192), (130, 4130)):
        z, ctas = C.c_int(), C.c_int()
        rd.check(L.rd_attn_prefill_plan(n_q, keys, 24, 148, C.addressof(z), C.addressof(ctas)))
        lines.append(f"{n_q} {keys} | {z.value} {ctas.value}")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    text = table()
    if "--print" in sys.argv:
        sys.stdout.write(text)
    else:
        with open(os.path.join(HERE, "b200_plan.txt"), "w") as f:
            f.write(text)
        print("wrote b200_plan.txt,", len(text), "bytes")
