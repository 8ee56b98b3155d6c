"""Child process of tests/test_gpu_hardening.py: each mode runs in a FRESH process, so the
library call it makes is that process's first one. Prints one line 'RESULT <json>'."""
import ctypes as C
import importlib
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle.oracle import Oracle  # noqa: E402  (the checker; the product never imports it)

oracle = Oracle()

rd = importlib.import_module("rdna4-infer_b200")
lib = rd.lib
NH, NKV, HD = 24, 4, 256


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def mode_env_switches():
    """Timing-switch variables are set by the parent: a default build must ignore them."""
    rng = np.random.default_rng(3)
    n = 3000
    K = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    V = rng.standard_normal((n, NKV, HD)).astype(np.float32)
    q = rng.standard_normal((NH, HD)).astype(np.float32)
    kc, vc = oracle.kv_store_rows(3, K), oracle.kv_store_rows(3, V)
    want = oracle.attn(q[None], kc, vc, [n - 1], NKV, 1 / 16, 3, 3)[0]
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    out = torch.full((NH, HD), float("nan"), device="cuda")
    wsb = lib.rd_attn_workspace_bytes(1, NH, HD)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    rc = lib.rd_attn_decode_ws(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), None, 0, n - 1, NH, NKV, HD,
                               1 / 16, 3, 3, 1, None, rd.ptr(ws), wsb, rd.stream_ptr())
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    err = float(np.abs(got - want).max())
    cos = float((got * want).sum() / np.sqrt((got * got).sum() * (want * want).sum()))
    # prefill too (f16 caches)
    nq = 128
    Kf = rng.standard_normal((nq, NKV, HD)).astype(np.float32)
    Vf = rng.standard_normal((nq, NKV, HD)).astype(np.float32)
    qf = rng.standard_normal((nq, NH, HD)).astype(np.float32)
    kcf, vcf = oracle.kv_store_rows(1, Kf), oracle.kv_store_rows(1, Vf)
    pos = np.arange(nq, dtype=np.int32)
    wantp = oracle.attn(qf, kcf, vcf, pos, NKV, 1 / 16, 1, 1)
    outp = torch.full((nq, NH, HD), float("nan"), device="cuda")
    dqf, dkf, dvf, dpos = dev(qf), dev(kcf), dev(vcf), dev(pos)   # kept alive across the launch
    rcp = lib.rd_fa2_prefill(rd.ptr(dqf), rd.ptr(dkf), rd.ptr(dvf), rd.ptr(outp), rd.ptr(dpos),
                             nq, nq - 1, nq, NH, NKV, HD, 1 / 16, rd.stream_ptr())
    torch.cuda.synchronize()
    errp = float(np.abs(outp.cpu().numpy() - wantp).max())
    return {"rc": rc, "max_abs": err, "cos": cos, "rc_prefill": rcp, "max_abs_prefill": errp,
            "status": lib.rd_device_status()}


def mode_first_call_timeout():
    """The process's FIRST library call is a workspace entry whose exchange wait runs out
    (rank 1 of the group never pushes): the time-out must be reported."""
    world = 2
    nbytes = lib.rd_shard_xbuf_bytes(NH, HD, world)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    group = rd.shard_group(0, [rd.ptr(b) for b in bufs], 20000)   # wait at most 20 ms
    n = 64
    kc = torch.zeros(n * NKV * 144, dtype=torch.uint8, device="cuda")
    q = torch.zeros(NH, HD, device="cuda")
    out = torch.full((NH, HD), float("nan"), device="cuda")
    wsb = 4 << 20
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    rc = lib.rd_attn_decode_sharded(rd.ptr(q), rd.ptr(kc), rd.ptr(kc), rd.ptr(out), n - 1, NH, NKV, HD, 1 / 16,
                                    3, 3, None, rd.ptr(ws), wsb, C.addressof(group), rd.stream_ptr())
    torch.cuda.synchronize()
    first = lib.rd_device_status()
    second = lib.rd_device_status()
    return {"rc": rc, "status_first": first, "status_second": second, "zeros": bool((out == 0).all())}


if __name__ == "__main__":
    res = {"env_switches": mode_env_switches, "first_call_timeout": mode_first_call_timeout}[sys.argv[1]]()
    print("RESULT " + json.dumps(res))
