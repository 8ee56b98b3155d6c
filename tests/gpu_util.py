"""Helpers for the GPU tests: move numpy data to torch device tensors and call the
C-ABI library with raw pointers (nothing here computes anything)."""
import importlib

import numpy as np
import torch

rd = importlib.import_module("rdna4-infer_b200")
lib = rd.lib
NH, NKV, HD = 24, 4, 256
SCALE = 1.0 / 16.0


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host(t):
    return t.detach().cpu().numpy()


def st():
    return rd.stream_ptr()


def status_ok():
    assert lib.rd_device_status() == rd.OK


def kv_store(t, src_np):
    """numpy f32 -> numpy uint8 bytes through rd_kv_store_rows."""
    src = dev(src_np.astype(np.float32).reshape(-1))
    n = src.numel()
    nbytes = n * 4 if t == rd.F32 else n * 2 if t == rd.F16 else n // 32 * rd.row_bytes(t, 32)
    dst = torch.full((nbytes,), 0xA5, dtype=torch.uint8, device="cuda")
    rd.check(lib.rd_kv_store_rows(t, rd.ptr(src), rd.ptr(dst), n, st()), "rd_kv_store_rows")
    torch.cuda.synchronize()
    return host(dst)


def poison(shape):
    """f32 device tensor full of NaN (unwritten elements must not survive)."""
    return torch.full(shape, float("nan"), dtype=torch.float32, device="cuda")


def attn_decode(q, kc, vc, t, kt, vt, nkv=NKV, n_splits=None, scale=SCALE, inplace=False):
    """q [n_head][256] numpy; kc/vc numpy uint8 caches. Returns out numpy."""
    n_head = q.shape[0]
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    out = dq if inplace else poison(q.shape)
    if n_splits is None:
        rc = lib.rd_attn_decode(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), t, n_head, nkv, HD,
                                scale, kt, vt, st())
    else:
        part = poison((n_head, n_splits, 2 + HD))
        rc = lib.rd_attn_decode_split(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), rd.ptr(part),
                                      t, n_head, nkv, HD, scale, kt, vt, n_splits, st())
    rd.check(rc, "rd_attn_decode")
    torch.cuda.synchronize()
    return host(out)


def attn_partials(q, kc, vc, t, kt, vt, n_splits, nkv=NKV, scale=SCALE):
    n_head = q.shape[0]
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    part = poison((n_head, n_splits, 2 + HD))
    rc = lib.rd_attn_decode_split(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), None, rd.ptr(part), t, n_head,
                                  nkv, HD, scale, kt, vt, n_splits, st())
    rd.check(rc, "rd_attn_decode_split(partials)")
    torch.cuda.synchronize()
    return host(part)


def attn_batch(q, kc, vc, pos, kt, vt, nkv=NKV, n_splits=None, scale=SCALE):
    n_tok, n_head, _ = q.shape
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    dpos = dev(np.asarray(pos, dtype=np.int32))
    out = poison(q.shape)
    if n_splits is None:
        rc = lib.rd_attn_batch(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), rd.ptr(dpos), n_tok,
                               n_head, nkv, HD, scale, kt, vt, st())
    else:
        part = poison((n_tok, n_head, n_splits, 2 + HD))
        rc = lib.rd_attn_split_batch(rd.ptr(dq), rd.ptr(dk), rd.ptr(dv), rd.ptr(out), rd.ptr(part),
                                     rd.ptr(dpos), n_tok, n_head, nkv, HD, scale, kt, vt, n_splits,
                                     st())
    rd.check(rc, "rd_attn_batch")
    torch.cuda.synchronize()
    return host(out)


def merge(partial_np, gate_np=None):
    p = dev(partial_np.astype(np.float32))
    n_rows, n_splits, rec = partial_np.shape
    out = poison((n_rows, rec - 2))
    g = dev(gate_np) if gate_np is not None else None
    rd.check(lib.rd_attn_merge(rd.ptr(p), rd.ptr(out), n_rows, rec - 2, n_splits, rd.ptr(g), st()),
             "rd_attn_merge")
    torch.cuda.synchronize()
    return (host(out), host(g)) if g is not None else host(out)
