"""A C++ caller written against the reference's names (tests/cpp/graph_caller.cpp: the
sequence of Graph::full_attn and Graph::forward_batch_layer) is compiled with the host
compiler, linked to the C-ABI library, run on the GPU, and its outputs are recomputed
with the CPU oracle from the same LCG inputs."""
import importlib
import os
import shutil
import subprocess

import numpy as np
import pytest

from oracle.oracle import TYPE_NAMES, lcg_stream
from tests.conftest import check_attn

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NH, NKV, HD = 24, 4, 256


@pytest.fixture(scope="module")
def exe(cuda, tmp_path_factory):
    rd = importlib.import_module("rdna4-infer_b200")
    if shutil.which("g++") is None or not os.path.isdir("/usr/local/cuda/include"):
        pytest.skip("no host C++ toolchain / CUDA headers")
    out = str(tmp_path_factory.mktemp("cpp") / "graph_caller")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror",
                           "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "tests", "cpp", "graph_caller.cpp"), "-o", out,
                           "-L" + rd.HERE, "-lrd_attn_b200", "-Wl,-rpath," + rd.HERE,
                           "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"])
    return out


class Lcg:
    """Draws from one stream in the order the C++ program does."""

    def __init__(self, total):
        self.v = lcg_stream(12345, total)
        self.i = 0

    def take(self, n, amp):
        out = (np.float32(amp) * self.v[self.i:self.i + n]).astype(np.float32)
        self.i += n
        return out


@pytest.mark.parametrize("kt,vt,n_prefix,n_batch", [(3, 3, 700, 8), (3, 3, 2100, 4), (1, 1, 1000, 8),
                                                    (2, 1, 1500, 4), (4, 5, 600, 3)])
def test_graph_shaped_caller(exe, oracle, tmp_path, kt, vt, n_prefix, n_batch):
    n_layers = 2
    out_file = str(tmp_path / "out.bin")
    r = subprocess.run([exe, out_file, TYPE_NAMES[kt], TYPE_NAMES[vt], str(n_prefix), str(n_batch),
                        str(n_layers)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(out_file, dtype=np.float32)
    per_layer = (n_batch + 1) * NH * HD
    assert got.size == n_layers * per_layer
    per_tok = NH * 2 * HD + 2 * NKV * HD
    lcg = Lcg(n_layers * (2 * HD + (n_batch + 1) * per_tok))
    rk, rv = oracle.row_bytes(kt, HD) * NKV, oracle.row_bytes(vt, HD) * NKV
    for il in range(n_layers):
        kc = np.zeros((n_prefix + n_batch + 1) * rk, dtype=np.uint8)
        vc = np.zeros((n_prefix + n_batch + 1) * rv, dtype=np.uint8)
        kc[:n_prefix * rk] = oracle.kv_fill(kt, n_prefix * NKV, HD, 100 + il)
        vc[:n_prefix * rv] = oracle.kv_fill(vt, n_prefix * NKV, HD, 200 + il)
        wq = (1.0 + 0.1 * lcg.take(HD, 1.0)).astype(np.float32)
        wk = (1.0 + 0.1 * lcg.take(HD, 1.0)).astype(np.float32)
        off = il * per_layer
        for n, pos0 in ((n_batch, n_prefix), (1, n_prefix + n_batch)):
            proj = lcg.take(n * NH * 2 * HD, 2.0).reshape(n, NH, 2 * HD)
            ks = lcg.take(n * NKV * HD, 2.0).reshape(n, NKV, HD)
            vs = lcg.take(n * NKV * HD, 1.0).reshape(n, NKV, HD)
            pos = np.arange(pos0, pos0 + n, dtype=np.int32)
            q, gate = oracle.deinterleave_q_gate(proj, n, NH, HD)
            q = oracle.rope(oracle.rms_norm(q, wq, 1e-6), pos)
            k = oracle.rope(oracle.rms_norm(ks, wk, 1e-6), pos)
            kc[pos0 * rk:(pos0 + n) * rk] = oracle.kv_store_rows(kt, k)
            vc[pos0 * rv:(pos0 + n) * rv] = oracle.kv_store_rows(vt, vs)
            y = oracle.attn(q, kc, vc, pos, NKV, 1 / 16, kt, vt)
            _, want = oracle.sigmoid_gate(gate, y)
            check_attn(got[off:off + n * NH * HD].reshape(n, NH, HD), want,
                       what=f"layer {il}, {n} token(s) at {pos0}")
            off += n * NH * HD
    assert lcg.i == lcg.v.size
