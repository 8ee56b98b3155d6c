"""CPU-only checks of the C-ABI boundary: the library loads, exports every symbol the
header declares, and rejects bad arguments on the host before touching a device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rd_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rd_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(rd):
    syms = declared_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(rd.lib, s), f"{s} declared in include/rd_attn.h but not exported"
        assert s in rd.SIGNATURES, f"{s} has no ctypes signature"
    assert set(rd.SIGNATURES) == set(syms)
    assert b"sm_100a" in rd.lib.rd_version()


def test_missing_library_fails_loudly(rd, tmp_path, monkeypatch):
    import importlib.util
    spec = importlib.util.spec_from_file_location("rd_copy", os.path.join(rd.HERE, "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    monkeypatch.setattr(os.path, "exists", lambda p: False if p.endswith("librd_attn_b200.so") else True)
    with pytest.raises(ImportError):
        spec.loader.exec_module(mod)


def test_kv_tables(rd, golden):
    g = golden("tables")
    assert [rd.row_bytes(t, 256) for t in range(6)] == list(g["row_bytes"])
    assert rd.lib.rd_kv_row_bytes(99, 256) == 0
    names = ("f32", "f16", "q8_0", "q4_0", "q5_0", "q4_1", "q5_1", "")
    for nm, want in zip(names, g["parse"]):
        out = C.c_int(-7)
        rc = rd.lib.rd_kv_type_parse(nm.encode(), C.byref(out))
        if want >= 0:
            assert rc == rd.OK and out.value == want
            assert rd.lib.rd_kv_type_name(int(want)) == nm.encode()
        else:
            assert rc == rd.ERR_TYPE  # a name llama.cpp has and this engine does not
    assert rd.lib.rd_kv_type_name(99) is None
    assert rd.lib.rd_kv_bytes_per_elem(rd.Q4_0) == 18.0 / 32.0
    assert rd.lib.rd_kv_bytes_per_elem(99) == 0.0
    assert [rd.lib.rd_attn_partial_bytes(24, 256, s) for s in (1, 4, 16)] == list(g["partial_bytes"])
    # exact cache budgets at 131072 tokens (tests/check_kvtype.hip:157-163 of the reference)
    per_tok = lambda k, v: 16 * 4 * (rd.row_bytes(k) + rd.row_bytes(v))
    assert 131072 * per_tok(rd.Q4_0, rd.Q4_0) == 2415919104
    assert 131072 * per_tok(rd.Q8_0, rd.Q4_1) == 3623878656


def test_argument_validation_happens_on_the_host(rd):
    L = rd.lib
    buf = np.zeros(4096, dtype=np.float32)
    p = buf.ctypes.data  # a host pointer: never dereferenced, validation fails first
    # unknown enum: dispatchers refuse instead of guessing (kv.h:58-69 / check_kvtype.hip:249-279)
    assert L.rd_kv_store_rows(99, p, p, 256, None) == rd.ERR_TYPE
    assert L.rd_kv_fill(-1, p, 4, 256, 1, None) == rd.ERR_TYPE
    assert L.rd_attn_decode(p, p, p, p, 5, 24, 4, 256, 0.0625, 99, rd.F16, None) == rd.ERR_TYPE
    assert L.rd_kv_store_rows(rd.Q4_0, p, p, 33, None) == rd.ERR_SHAPE
    assert L.rd_kv_store_rows(rd.Q4_0, None, p, 64, None) == rd.ERR_NULL
    assert L.rd_kv_store_rows(rd.Q4_0, p, p + 1, 64, None) == rd.ERR_ALIGN
    assert L.rd_kv_store_rows(rd.Q4_0, p, p, 0, None) == rd.OK
    # shapes the reference accepts but this build refuses, with their own code
    assert L.rd_attn_decode(p, p, p, p, 5, 24, 4, 128, 0.0625, rd.F16, rd.F16, None) == rd.ERR_UNSUPPORTED
    assert L.rd_attn_decode(p, p, p, p, 5, 32, 4, 256, 0.0625, rd.F16, rd.F16, None) == rd.ERR_UNSUPPORTED
    assert L.rd_attn_decode(p, p, p, p, 5, 24, 4, 256, 0.0625, 6, rd.F16, None) == rd.ERR_TYPE
    assert L.rd_attn_decode(p, p, p, p, 5, 24, 4, 100, 0.0625, rd.F16, rd.F16, None) == rd.ERR_SHAPE
    assert L.rd_attn_decode(p, p, p, p, 5, 24, 5, 256, 0.0625, rd.F16, rd.F16, None) == rd.ERR_SHAPE
    assert L.rd_attn_decode_split(p, p, p, p, p, 5, 24, 4, 256, 0.0625, rd.F16, rd.F16, 0, None) == rd.ERR_SHAPE
    assert L.rd_attn_decode(p, None, p, p, 5, 24, 4, 256, 0.0625, rd.F16, rd.F16, None) == rd.ERR_NULL
    assert L.rd_attn_decode(p, p + 4, p, p, 5, 24, 4, 256, 0.0625, rd.F16, rd.F16, None) == rd.ERR_ALIGN
    assert L.rd_attn_decode_ws(p, p, p, p, p, 0, 5, 24, 4, 256, 0.0625, rd.F16, rd.F16, 1, None, None, 0,
                               None) == rd.ERR_WORKSPACE
    assert L.rd_attn_merge(p, p, 24, 256, 0, None, None) == rd.ERR_SHAPE
    assert L.rd_attn_merge(p, p, 24, 128, 2, None, None) == rd.ERR_UNSUPPORTED
    assert L.rd_rope(p, 1, 4, 256, 63, 1e7, p, None) == rd.ERR_SHAPE
    assert L.rd_fa2_prefill_usable(rd.F16, rd.F16, 512, 0, 24, 4, 256) == 1
    assert L.rd_fa2_prefill_usable(rd.Q8_0, rd.F16, 512, 0, 24, 4, 256) == 0
    assert L.rd_fa2_prefill_usable(rd.F16, rd.F16, 512, 0, 24, 4, 128) == 0
    for code in range(-9, 1):
        assert rd.strerror(code) and "unknown" not in rd.strerror(code)


def test_cpp_wrappers_compile_and_behave(rd, tmp_path):
    """include/rdna4/ gives reference-named C++17 wrappers: a caller written against
    the reference's names builds against them and links to the C-ABI library."""
    import shutil
    import subprocess
    if shutil.which("g++") is None or not os.path.isdir("/usr/local/cuda/include"):
        pytest.skip("no host C++ toolchain / CUDA headers")
    exe = str(tmp_path / "wrapper_check")
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror",
                           "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "tests", "cpp", "wrapper_check.cpp"), "-o", exe,
                           "-L" + rd.HERE, "-lrd_attn_b200", "-Wl,-rpath," + rd.HERE])
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
