"""Source-level rules of the product library (CPU only)."""
import glob
import os
import re

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rdna4-infer_b200", "csrc")


def test_environment_is_read_only_in_timing_switch_builds():
    """Every getenv of the library sits inside #ifdef RD_TIMING_SWITCHES: a default build
    takes nothing from the environment, so a stray variable cannot change a result."""
    for path in glob.glob(os.path.join(CSRC, "*")):
        depth, guarded = [], 0
        for line in open(path):
            s = line.strip()
            if re.match(r"#\s*if", s):
                is_guard = "RD_TIMING_SWITCHES" in s and s.startswith("#ifdef")
                depth.append(is_guard)
                guarded += is_guard
            elif re.match(r"#\s*else", s) and depth and depth[-1]:
                guarded -= 1
                depth[-1] = False
            elif re.match(r"#\s*endif", s) and depth:
                guarded -= depth.pop()
            elif "getenv(" in s and not s.startswith("//"):
                assert guarded > 0, f"{os.path.basename(path)}: unguarded getenv: {s}"


def test_product_sources_do_not_name_the_oracle():
    for path in glob.glob(os.path.join(CSRC, "*")):
        assert "oracle" not in open(path).read().lower(), path
