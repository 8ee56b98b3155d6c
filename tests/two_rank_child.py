"""One rank of tests/test_gpu_two_ranks.py (launched by torch.distributed.run, one process
per GPU): context-sharded decode through the fused peer-store exchange on REAL peers, every
rank checking the merged output against the CPU oracle over the whole context."""
import ctypes as C
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle.oracle import Oracle  # noqa: E402  (the checker)

rd = importlib.import_module("rdna4-infer_b200")
lib = rd.lib
NH, NKV, HD = 24, 4, 256


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import torch.distributed._symmetric_memory as symm
    xbytes = lib.rd_shard_xbuf_bytes(NH, HD, world)
    xbuf = symm.empty(xbytes, dtype=torch.uint8, device=torch.device("cuda", local))
    hdl = symm.rendezvous(xbuf, dist.group.WORLD)
    xbuf.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    group = rd.shard_group(rank, [int(p) for p in hdl.buffer_ptrs], 2_000_000)   # waits give up after 2 s
    ora = Oracle()
    ora.set_threads(max(1, (os.cpu_count() or 2) // world))
    worst = 0.0
    for kt, vt, n_keys in ((3, 3, 20011), (2, 1, 4097), (4, 5, 333)):
        rng = np.random.default_rng(1000 * kt + vt)            # same data on every rank
        K = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
        V = rng.standard_normal((n_keys, NKV, HD)).astype(np.float32)
        kc, vc = ora.kv_store_rows(kt, K), ora.kv_store_rows(vt, V)
        rk, rv = rd.row_bytes(kt) * NKV, rd.row_bytes(vt) * NKV
        per = (n_keys + world - 1) // world
        b, e = rank * per, min(n_keys, (rank + 1) * per)
        owner = b < n_keys <= e                                 # this rank's slice ends with the newest key
        ks, vs = kc[b * rk:max(e, b + 1) * rk].copy(), vc[b * rv:max(e, b + 1) * rv].copy()
        if owner:                                               # ... which its fused append stores
            ks[-rk:], vs[-rv:] = 0xEE, 0xEE
        dk, dv = torch.from_numpy(ks).cuda(), torch.from_numpy(vs).cuda()
        dkn, dvn = torch.from_numpy(K[n_keys - 1]).cuda(), torch.from_numpy(V[n_keys - 1]).cuda()
        wsb = lib.rd_attn_workspace_bytes(1, NH, HD)
        ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
        for call in range(3):                                   # both parities of the buffer, and reuse
            q = rng.standard_normal((NH, HD)).astype(np.float32)
            gate = rng.standard_normal((NH, HD)).astype(np.float32)
            y = ora.attn(q[None], kc, vc, [n_keys - 1], NKV, 1 / 16, kt, vt)[0]
            want_g, want = ora.sigmoid_gate(gate.copy(), y)
            dq, dg = torch.from_numpy(q).cuda(), torch.from_numpy(gate).cuda()
            out = torch.full((NH, HD), float("nan"), device="cuda")
            if owner:
                rc = lib.rd_attn_decode_sharded_append(rd.ptr(dq), rd.ptr(dkn), rd.ptr(dvn), rd.ptr(dk), rd.ptr(dv),
                                                       rd.ptr(out), e - b - 1, NH, NKV, HD, 1 / 16, kt, vt,
                                                       rd.ptr(dg), rd.ptr(ws), wsb, C.addressof(group),
                                                       rd.stream_ptr())
            else:
                rc = lib.rd_attn_decode_sharded(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), e - b - 1, NH, NKV,
                                                HD, 1 / 16, kt, vt, rd.ptr(dg), rd.ptr(ws), wsb, C.addressof(group),
                                                rd.stream_ptr())
            assert rc == rd.OK, rc
            torch.cuda.synchronize()
            if owner:
                assert np.array_equal(dk.cpu().numpy()[-rk:], kc[(n_keys - 1) * rk:n_keys * rk])
                assert np.array_equal(dv.cpu().numpy()[-rv:], vc[(n_keys - 1) * rv:n_keys * rv])
            got = out.cpu().numpy()
            err = float(np.abs(got - want).max())
            cos = float((got * want).sum() / np.sqrt((got * got).sum() * (want * want).sum()))
            assert err <= 2e-3 and cos >= 0.9999, (rank, kt, vt, n_keys, call, err, cos)
            assert float(np.abs(dg.cpu().numpy() - want_g).max()) <= 1e-6
            worst = max(worst, err)
    assert lib.rd_device_status() == rd.OK
    dist.barrier()
    print(f"RANK {rank} OK worst max-abs {worst:.2e}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
