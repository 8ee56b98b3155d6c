"""ctypes bindings of the CPU checker. TEST INFRASTRUCTURE ONLY.

Two libraries, both built by ``oracle/Makefile``:

* ``Oracle``    -> ``_build/librd_oracle.so``, the plain-C restatement (rd_oracle.c);
* ``Reference`` -> ``_ref/librd_ref.so``, the reference project's own kernels run on
  CPU fibers (ref_driver.cpp). It can only be (re)built where the reference checkout
  exists; it is used to pin the restatement and to generate ``tests/golden``.

Nothing in the product package imports this module; the test-suite, the smoke check
and the benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16, Q8_0, Q4_0, Q5_0, Q4_1 = range(6)
TYPE_NAMES = {F32: "f32", F16: "f16", Q8_0: "q8_0", Q4_0: "q4_0", Q5_0: "q5_0", Q4_1: "q4_1"}


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def reference_dir() -> str | None:
    """The reference checkout: $RD_REFERENCE_DIR, else a directory named `reference` beside
    this repository; None where neither holds the headers."""
    cand = os.environ.get("RD_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "include", "rdna4")) else None


def build(ref: bool = True) -> None:
    """Compile the checker libraries (the reference one only if its checkout is there)."""
    subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    if ref and reference_dir() is not None:
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", "REF=" + reference_dir()])


class _AttnMixin:
    """Shared shape helpers."""

    @staticmethod
    def row_bytes_static(t, head_dim=256):
        blocks = (head_dim + 31) // 32
        return {F32: head_dim * 4, F16: head_dim * 2, Q8_0: blocks * 34, Q4_0: blocks * 18,
                Q5_0: blocks * 22, Q4_1: blocks * 20}[t]


class Oracle(_AttnMixin):
    def __init__(self, path: str | None = None):
        path = path or os.path.join(HERE, "_build", "librd_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = self.lib = C.CDLL(path)
        L.rdo_fp16_to_float.restype = C.c_float
        L.rdo_fp16_to_float.argtypes = [C.c_uint16]
        L.rdo_float_to_fp16.restype = C.c_uint16
        L.rdo_float_to_fp16.argtypes = [C.c_float]
        L.rdo_kv_row_bytes.restype = C.c_uint64
        L.rdo_kv_row_bytes.argtypes = [C.c_int, C.c_int]
        L.rdo_kv_store_rows.restype = C.c_int
        L.rdo_kv_store_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        L.rdo_kv_dequant_rows.restype = C.c_int
        L.rdo_kv_dequant_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int]
        L.rdo_kv_rand.restype = C.c_float
        L.rdo_kv_rand.argtypes = [C.c_uint32, C.c_uint32]
        L.rdo_kv_fill_values.restype = None
        L.rdo_kv_fill_values.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_uint32]
        L.rdo_kv_fill.restype = C.c_int
        L.rdo_kv_fill.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_uint32]
        L.rdo_rope.restype = None
        L.rdo_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]
        L.rdo_sigmoid_gate.restype = None
        L.rdo_sigmoid_gate.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int]
        L.rdo_rms_norm.restype = None
        L.rdo_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float]
        L.rdo_deinterleave_q_gate.restype = None
        L.rdo_deinterleave_q_gate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int]
        L.rdo_attn.restype = C.c_int
        L.rdo_attn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                               C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int]
        L.rdo_attn_partials.restype = C.c_int
        L.rdo_attn_partials.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                        C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int]
        L.rdo_attn_merge.restype = None
        L.rdo_attn_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.rdo_num_threads.restype = C.c_int
        L.rdo_set_threads.argtypes = [C.c_int]

    # -- scalars
    def fp16_to_float(self, h):
        return float(self.lib.rdo_fp16_to_float(int(h)))

    def float_to_fp16(self, f):
        return int(self.lib.rdo_float_to_fp16(float(f)))

    def row_bytes(self, t, head_dim=256):
        return int(self.lib.rdo_kv_row_bytes(t, head_dim))

    def kv_rand(self, idx, seed):
        return float(self.lib.rdo_kv_rand(idx & 0xFFFFFFFF, seed & 0xFFFFFFFF))

    def num_threads(self):
        return int(self.lib.rdo_num_threads())

    def set_threads(self, n):
        self.lib.rdo_set_threads(int(n))

    # -- KV
    def kv_store_rows(self, t, src):
        """f32 array (any shape, size multiple of 32 for block types) -> uint8 bytes."""
        src = _f32(src).reshape(-1)
        if t in (F32, F16):
            nbytes = src.size * (4 if t == F32 else 2)
        else:
            nbytes = src.size // 32 * self.row_bytes(t, 32)
        dst = np.zeros(nbytes, dtype=np.uint8)
        rc = self.lib.rdo_kv_store_rows(t, _ptr(src), _ptr(dst), src.size)
        if rc != 0:
            raise ValueError(f"rdo_kv_store_rows rc={rc}")
        return dst

    def kv_dequant_rows(self, t, raw, n_rows, head_dim=256):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty((n_rows, head_dim), dtype=np.float32)
        rc = self.lib.rdo_kv_dequant_rows(t, _ptr(raw), _ptr(out), n_rows, head_dim)
        if rc != 0:
            raise ValueError(f"rdo_kv_dequant_rows rc={rc}")
        return out

    def kv_fill_values(self, n_rows, head_dim, seed):
        out = np.empty((n_rows, head_dim), dtype=np.float32)
        self.lib.rdo_kv_fill_values(_ptr(out), n_rows, head_dim, seed)
        return out

    def kv_fill(self, t, n_rows, head_dim, seed):
        out = np.zeros(n_rows * self.row_bytes(t, head_dim), dtype=np.uint8)
        rc = self.lib.rdo_kv_fill(t, _ptr(out), n_rows, head_dim, seed)
        if rc != 0:
            raise ValueError(f"rdo_kv_fill rc={rc}")
        return out

    # -- RoPE / gate
    def rope(self, x, pos, n_rot=64, freq_base=1e7):
        x = _f32(x).copy()
        n_tok, n_heads, hd = x.shape
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        self.lib.rdo_rope(_ptr(x), n_tok, n_heads, hd, n_rot, freq_base, _ptr(pos))
        return x

    def sigmoid_gate(self, g, y, store_sigmoid=True):
        g = _f32(g).copy()
        y = _f32(y).copy()
        self.lib.rdo_sigmoid_gate(_ptr(g), _ptr(y), g.size, 1 if store_sigmoid else 0)
        return g, y

    def rms_norm(self, x, w, eps):
        """x [rows][cols] f32, w [cols] or None."""
        x = _f32(x)
        y = np.empty_like(x)
        rows, cols = x.reshape(-1, x.shape[-1]).shape
        wp = _ptr(_f32(w)) if w is not None else None
        self.lib.rdo_rms_norm(_ptr(x), wp, _ptr(y), rows, cols, eps)
        return y

    def deinterleave_q_gate(self, yq, n_tok, n_head, head_dim):
        yq = _f32(yq)
        q = np.empty((n_tok, n_head, head_dim), dtype=np.float32)
        g = np.empty((n_tok, n_head, head_dim), dtype=np.float32)
        self.lib.rdo_deinterleave_q_gate(_ptr(yq), _ptr(q), _ptr(g), n_tok, n_head, head_dim)
        return q, g

    # -- attention
    def attn(self, q, k, v, pos, n_head_kv, scale, kt, vt, f64=False):
        """q [n_tok][n_head][hd] f32; k, v raw uint8 caches; pos int32 [n_tok]."""
        q = _f32(q)
        n_tok, n_head, hd = q.shape
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        k = np.ascontiguousarray(k, dtype=np.uint8)
        v = np.ascontiguousarray(v, dtype=np.uint8)
        out = np.empty_like(q)
        rc = self.lib.rdo_attn(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(pos), n_tok, n_head,
                               n_head_kv, hd, scale, kt, vt, 1 if f64 else 0)
        if rc != 0:
            raise ValueError(f"rdo_attn rc={rc}")
        return out

    def attn_partials(self, q, k, v, key_begin, key_end, n_head_kv, scale, kt, vt, n_splits):
        q = _f32(q)
        n_head, hd = q.shape
        k = np.ascontiguousarray(k, dtype=np.uint8)
        v = np.ascontiguousarray(v, dtype=np.uint8)
        part = np.empty((n_head, n_splits, 2 + hd), dtype=np.float32)
        rc = self.lib.rdo_attn_partials(_ptr(q), _ptr(k), _ptr(v), _ptr(part), key_begin, key_end,
                                        n_head, n_head_kv, hd, scale, kt, vt, n_splits)
        if rc != 0:
            raise ValueError(f"rdo_attn_partials rc={rc}")
        return part

    def attn_merge(self, partial, f64=False):
        """partial [n_rows][n_splits][2+hd] -> [n_rows][hd]."""
        partial = _f32(partial)
        n_rows, n_splits, rec = partial.shape
        out = np.empty((n_rows, rec - 2), dtype=np.float32)
        self.lib.rdo_attn_merge(_ptr(partial), _ptr(out), n_rows, rec - 2, n_splits, 1 if f64 else 0)
        return out


class Reference(_AttnMixin):
    """The reference's own kernels on CPU fibers (slow: small cases only)."""

    def __init__(self, path: str | None = None):
        path = path or os.path.join(HERE, "_ref", "librd_ref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = self.lib = C.CDLL(path)
        L.ref_float_to_fp16.restype = C.c_uint16
        L.ref_float_to_fp16.argtypes = [C.c_float]
        L.ref_fp16_to_float.restype = C.c_float
        L.ref_fp16_to_float.argtypes = [C.c_uint16]
        L.ref_kv_rand.restype = C.c_float
        L.ref_kv_rand.argtypes = [C.c_uint, C.c_uint]
        L.ref_kv_row_bytes.restype = C.c_uint64
        L.ref_kv_row_bytes.argtypes = [C.c_int, C.c_int]
        L.ref_kv_bytes_per_elem.restype = C.c_double
        L.ref_kv_bytes_per_elem.argtypes = [C.c_int]
        L.ref_kv_type_name.restype = C.c_char_p
        L.ref_kv_type_name.argtypes = [C.c_int]
        L.ref_kv_type_parse.argtypes = [C.c_char_p, C.c_void_p]
        L.ref_attn_split_wpb.argtypes = [C.c_int]
        L.ref_attn_partial_bytes.restype = C.c_uint64
        L.ref_attn_partial_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ref_kv_store_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.ref_kv_fill.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_uint]
        L.ref_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]
        L.ref_sigmoid_gate.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        L.ref_attn.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_int]
        L.ref_attn_batch.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_int]
        L.ref_attn_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.ref_attn_split.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_int, C.c_int]
        L.ref_attn_split_batch.argtypes = [C.c_void_p] * 6 + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_int, C.c_int]
        L.ref_fa2_prefill.argtypes = [C.c_void_p] * 5 + [C.c_int] * 6 + [C.c_float]
        L.ref_fa2_prefill_usable.argtypes = [C.c_int] * 7

    def float_to_fp16(self, f):
        return int(self.lib.ref_float_to_fp16(float(f)))

    def fp16_to_float(self, h):
        return float(self.lib.ref_fp16_to_float(int(h)))

    def kv_rand(self, idx, seed):
        return float(self.lib.ref_kv_rand(idx & 0xFFFFFFFF, seed & 0xFFFFFFFF))

    def row_bytes(self, t, head_dim=256):
        return int(self.lib.ref_kv_row_bytes(t, head_dim))

    def kv_type_parse(self, name):
        out = C.c_int(-1)
        rc = self.lib.ref_kv_type_parse(name.encode(), C.byref(out))
        return None if rc else out.value

    def kv_store_rows(self, t, src):
        src = _f32(src).reshape(-1)
        if t in (F32, F16):
            nbytes = src.size * (4 if t == F32 else 2)
        else:
            nbytes = src.size // 32 * self.row_bytes(t, 32)
        dst = np.zeros(nbytes, dtype=np.uint8)
        rc = self.lib.ref_kv_store_rows(t, _ptr(src), _ptr(dst), src.size)
        assert rc == 0
        return dst

    def kv_fill(self, t, n_rows, head_dim, seed):
        out = np.zeros(n_rows * self.row_bytes(t, head_dim), dtype=np.uint8)
        assert self.lib.ref_kv_fill(t, _ptr(out), n_rows, head_dim, seed) == 0
        return out

    def rope(self, x, pos, n_rot=64, freq_base=1e7):
        x = _f32(x).copy()
        n_tok, n_heads, hd = x.shape
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        self.lib.ref_rope(_ptr(x), n_tok, n_heads, hd, n_rot, freq_base, _ptr(pos))
        return x

    def sigmoid_gate(self, g, y):
        g = _f32(g).copy()
        y = _f32(y).copy()
        self.lib.ref_sigmoid_gate(_ptr(g), _ptr(y), g.size)
        return g, y

    def rms_norm(self, x, w, eps):
        x = _f32(x)
        y = np.full_like(x, np.nan)
        rows, cols = x.reshape(-1, x.shape[-1]).shape
        wp = _ptr(_f32(w)) if w is not None else None
        self.lib.ref_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float]
        assert self.lib.ref_rms_norm(_ptr(x), wp, _ptr(y), rows, cols, eps) == 0
        return y

    def attn(self, q, k, v, t, n_head_kv, scale, kt, vt):
        q = _f32(q)
        n_head, hd = q.shape
        out = np.full_like(q, np.nan)
        rc = self.lib.ref_attn(_ptr(q), _ptr(k), _ptr(v), _ptr(out), t, n_head, n_head_kv, hd, scale, kt, vt)
        assert rc == 0
        return out

    def attn_batch(self, q, k, v, pos, n_head_kv, scale, kt, vt):
        q = _f32(q)
        n_tok, n_head, hd = q.shape
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        out = np.full_like(q, np.nan)
        rc = self.lib.ref_attn_batch(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(pos), n_tok, n_head,
                                     n_head_kv, hd, scale, kt, vt)
        assert rc == 0
        return out

    def attn_merge(self, partial):
        partial = _f32(partial)
        n_head, n_splits, rec = partial.shape
        out = np.full((n_head, rec - 2), np.nan, dtype=np.float32)
        self.lib.ref_attn_merge(_ptr(partial), _ptr(out), n_head, rec - 2, n_splits)
        return out

    def attn_split(self, q, k, v, t, n_head_kv, scale, kt, vt, n_splits):
        """Returns (out, partial[n_head][n_splits][2+hd])."""
        q = _f32(q)
        n_head, hd = q.shape
        out = np.full_like(q, np.nan)
        part = np.full((n_head, n_splits, 2 + hd), np.nan, dtype=np.float32)
        rc = self.lib.ref_attn_split(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(part), t, n_head,
                                     n_head_kv, hd, scale, kt, vt, n_splits)
        assert rc == 0
        return out, part

    def attn_split_batch(self, q, k, v, pos, n_head_kv, scale, kt, vt, n_splits):
        q = _f32(q)
        n_tok, n_head, hd = q.shape
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        out = np.full_like(q, np.nan)
        part = np.full((n_tok, n_head, n_splits, 2 + hd), np.nan, dtype=np.float32)
        rc = self.lib.ref_attn_split_batch(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(part), _ptr(pos),
                                           n_tok, n_head, n_head_kv, hd, scale, kt, vt, n_splits)
        assert rc == 0
        return out

    def fa2_prefill(self, q, k, v, pos, kmax, keys_total, n_head_kv, scale):
        q = _f32(q)
        n_q, n_head, hd = q.shape
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        out = np.full_like(q, np.nan)
        rc = self.lib.ref_fa2_prefill(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(pos), n_q, kmax,
                                      keys_total, n_head, n_head_kv, hd, scale)
        assert rc == 0
        return out

    def fa2_prefill_usable(self, kt, vt, n_q, pos0, n_head, n_head_kv, head_dim):
        return bool(self.lib.ref_fa2_prefill_usable(kt, vt, n_q, pos0, n_head, n_head_kv, head_dim))


class ReferenceGpu:
    """oracle/_ref/librd_ref_gpu.so: the reference project's own GPU launchers compiled
    unmodified for sm_100a (ref_gpu_driver.cu). Takes raw device pointers (ints). Raises
    FileNotFoundError where the library was not built (no reference checkout)."""

    def __init__(self):
        path = os.path.join(HERE, "_ref", "librd_ref_gpu.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = C.CDLL(path)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        L.refgpu_attn.argtypes = [P, P, P, P, I, I, I, I, F, I, I, P]
        L.refgpu_attn_split.argtypes = [P, P, P, P, P, I, I, I, I, F, I, I, I, P]
        L.refgpu_fa2_prefill.argtypes = [P, P, P, P, P, I, I, I, I, I, I, F, P]
        L.refgpu_kv_store_rows.argtypes = [I, P, P, I, P]
        for f in (L.refgpu_attn, L.refgpu_attn_split, L.refgpu_fa2_prefill, L.refgpu_kv_store_rows):
            f.restype = I
        self.lib = L


def lcg_stream(seed: int, n: int) -> np.ndarray:
    """The reference tests' generator (tests/check_rope_gpu.hip:36-39): s = s*1664525 +
    1013904223, value ((s>>8)/2^24 - 0.5)*2 in f32. Returns n values."""
    out = np.empty(n, dtype=np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = (np.float32(s >> 8) / np.float32(1 << 24) - np.float32(0.5)) * np.float32(2.0)
    return out
