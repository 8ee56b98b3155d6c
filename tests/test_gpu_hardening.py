"""The product path cannot be bent by the environment, and bounded waits are always
reported -- each case in a fresh process, so that the call under test is the first one the
library sees there."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.conftest import check_attn

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
NH, NKV, HD = 24, 4, 256


def run_child(mode, extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    out = subprocess.run([sys.executable, os.path.join(HERE, "hardening_child.py"), mode], env=env,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_timing_switch_variables_change_nothing(cuda):
    """RD_DECODE_DEBUG / RD_PREFILL_DEBUG / RD_PDL only exist in -DRD_TIMING_SWITCHES builds."""
    res = run_child("env_switches", {"RD_DECODE_DEBUG": "65", "RD_PREFILL_DEBUG": "63", "RD_PDL": "0"})
    assert res["rc"] == 0 and res["rc_prefill"] == 0 and res["status"] == 0
    assert res["max_abs"] <= 2e-3 and res["cos"] >= 0.9999, res
    assert res["max_abs_prefill"] <= 2e-3, res


def test_first_call_time_out_is_reported(cuda):
    """No allocating entry and no rd_device_status() ran before: the status word exists anyway."""
    import importlib
    rd = importlib.import_module("rdna4-infer_b200")
    res = run_child("first_call_timeout")
    assert res["rc"] == rd.OK
    assert res["status_first"] == rd.ERR_DEVICE, res
    assert res["status_second"] == rd.OK
    assert res["zeros"]


def test_multi_twice_on_one_workspace_with_growing_context(cuda, oracle):
    """The per-sequence tensor maps are rewritten at the same workspace address by the
    second call: the kernel must read the new ones (newest keys attended)."""
    import ctypes as C
    from tests import gpu_util as G
    rd, lib = G.rd, G.lib
    rng = np.random.default_rng(11)
    n_max = 2600
    K = rng.standard_normal((n_max, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n_max, NKV, HD)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(2, K), oracle.kv_store_rows(3, V)
    dk, dv = G.dev(kc), G.dev(vc)
    q = rng.standard_normal((1, NH, HD)).astype(np.float32)
    dq = G.dev(q)
    nbytes = lib.rd_attn_multi_workspace_bytes(1, 1, NH, HD)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    arr = (rd.AttnSeq * 1)()
    for n in (700, 1900, n_max):
        out = G.poison((1, NH, HD))
        arr[0].q, arr[0].k, arr[0].v, arr[0].out, arr[0].gate, arr[0].t = rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), \
            rd.ptr(out), None, n - 1
        rd.check(lib.rd_attn_decode_multi(C.addressof(arr), 1, 1, NH, NKV, HD, 1 / 16, 2, 3, rd.ptr(ws), nbytes,
                                          G.st()))
        torch.cuda.synchronize()
        want = oracle.attn(q, kc, vc, np.array([n - 1], dtype=np.int32), NKV, 1 / 16, 2, 3)
        check_attn(G.host(out), want, what=f"{n} keys")
    G.status_ok()
