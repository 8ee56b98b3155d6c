"""Python-side loader of ``librd_attn_b200.so`` -- the sm_100a attention / KV-cache
library that drops in under rdna4-infer's launch API (``include/rd_attn.h``).

The product is the C-ABI library; this module only binds it with ctypes so that the
tests and the benchmark can drive it with torch-owned device memory. There is no CPU
fallback of any kind: if the library has not been built, importing raises.

The directory name carries a hyphen, so import it with
``importlib.import_module("rdna4-infer_b200")``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librd_attn_b200.so")

F32, F16, Q8_0, Q4_0, Q5_0, Q4_1 = range(6)
TYPE_NAMES = ("f32", "f16", "q8_0", "q4_0", "q5_0", "q4_1")

OK = 0
ERR_TYPE, ERR_SHAPE, ERR_UNSUPPORTED, ERR_NULL, ERR_ALIGN, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE, \
    ERR_LIMIT = -1, -2, -3, -4, -5, -6, -7, -8, -9

# name -> (restype, argtypes); mirrors include/rd_attn.h one to one
_P, _I, _F, _L = C.c_void_p, C.c_int, C.c_float, C.c_int64
SIGNATURES = {
    "rd_version": (C.c_char_p, []),
    "rd_strerror": (C.c_char_p, [_I]),
    "rd_kv_type_name": (C.c_char_p, [_I]),
    "rd_kv_type_parse": (_I, [C.c_char_p, _P]),
    "rd_kv_bytes_per_elem": (C.c_double, [_I]),
    "rd_kv_row_bytes": (C.c_uint64, [_I, _I]),
    "rd_kv_store_rows": (_I, [_I, _P, _P, _L, _P]),
    "rd_kv_append": (_I, [_I, _I, _P, _P, _P, _P, _I, _I, _I, _P, _I, _F, _P]),
    "rd_kv_fill": (_I, [_I, _P, _L, _I, C.c_uint32, _P]),
    "rd_rope": (_I, [_P, _I, _I, _I, _I, _F, _P, _P]),
    "rd_deinterleave_q_gate": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "rd_sigmoid_gate": (_I, [_P, _P, _L, _P]),
    "rd_rms_norm": (_I, [_P, _P, _P, _L, _L, _F, _P]),
    "rd_pre_attn_fused": (_I, [_P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _I,
                               _F, _P]),
    "rd_attn_splits_for": (_I, [_I, _I, _I, _I, _I]),
    "rd_attn_prefill_plan": (_I, [_I, _I, _I, _I, _P, _P]),
    "rd_attn_plan": (_I, [_I, _I, _I, _I, _I, _I, _P, _P, _P]),
    "rd_attn_partial_bytes": (C.c_size_t, [_I, _I, _I]),
    "rd_attn_workspace_bytes": (C.c_size_t, [_I, _I, _I]),
    "rd_attn_decode": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P]),
    "rd_attn_decode_split": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P]),
    "rd_attn_decode_ws": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P,
                               C.c_size_t, _P]),
    "rd_attn_decode_append_ws": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, C.c_size_t,
                                      _P]),
    "rd_attn_multi_workspace_bytes": (C.c_size_t, [_I, _I, _I, _I]),
    "rd_attn_decode_multi": (_I, [_P, _I, _I, _I, _I, _I, _F, _I, _I, _P, C.c_size_t, _P]),
    "rd_attn_multi_plan_bytes": (C.c_size_t, [_I, _I]),
    "rd_attn_multi_plan": (_I, [_P, _I, _I, _I, _I, _I, _I, _I, _I, _P, C.c_size_t]),
    "rd_attn_multi_launch": (_I, [_P, _F, _P, C.c_size_t, _P]),
    "rd_shard_xbuf_bytes": (C.c_size_t, [_I, _I, _I]),
    "rd_attn_decode_sharded": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, C.c_size_t,
                                    _P, _P]),
    "rd_attn_decode_sharded_append": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, C.c_size_t,
                                           _P, _P]),
    "rd_attn_shard_push": (_I, [_P, _I, _I, _I, _P, _P]),
    "rd_attn_shard_merge": (_I, [_P, _P, _I, _I, _P, _P]),
    "rd_attn_decode_noalloc": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P]),
    "rd_attn_merge": (_I, [_P, _P, _I, _I, _I, _P, _P]),
    "rd_attn_batch": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P]),
    "rd_attn_split_batch": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P]),
    "rd_fa2_prefill_usable": (_I, [_I, _I, _I, _I, _I, _I, _I]),
    "rd_fa2_prefill": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "rd_attn_prefill_fused": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _F, _P]),
    "rd_attn_prefill_append_fused": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _F, _P]),
    "rd_attn_prefill_workspace_bytes": (C.c_size_t, [_I, _I, _I, _I, _I, _I, _I]),
    "rd_attn_prefill_typed": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _F, _P,
                                   C.c_size_t, _P]),
    "rd_device_status": (_I, []),
    "rd_device_timeout_site": (_I, []),
}


def build(verbose: bool = False) -> str:
    """Compile the library in-tree with nvcc for sm_100a (needs no GPU)."""
    cmd = ["make", "-C", HERE, "-j", str(os.cpu_count() or 4)]
    if not verbose:
        cmd.insert(1, "-s")
    subprocess.check_call(cmd)
    return LIB_PATH


class AttnSeq(C.Structure):
    """`rd_attn_seq` of include/rd_attn.h: one sequence of rd_attn_decode_multi."""

    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
                ("gate", C.c_void_p), ("t", C.c_int32), ("reserved", C.c_int32)]


class ShardGroup(C.Structure):
    """`rd_shard_group` of include/rd_attn.h."""

    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("xbuf", C.POINTER(C.c_void_p)),
                ("wait_limit_us", C.c_uint32), ("reserved", C.c_uint32)]


def shard_group(rank, xbuf_ptrs, wait_limit_us=0):
    """Build a ShardGroup (keeps the pointer array alive as an attribute)."""
    arr = (C.c_void_p * len(xbuf_ptrs))(*[int(p) for p in xbuf_ptrs])
    g = ShardGroup(rank, len(xbuf_ptrs), C.cast(arr, C.POINTER(C.c_void_p)), wait_limit_us, 0)
    g._keepalive = arr
    return g


class RdError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: rc={code}")


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {HERE}` (or __graft_entry__.build()); "
            "this package has no fallback path")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def strerror(code: int) -> str:
    return lib.rd_strerror(code).decode()


def check(code: int, what: str = "rd call") -> None:
    if code != OK:
        raise RdError(code, f"{what} ({strerror(code)})")


def row_bytes(t: int, head_dim: int = 256) -> int:
    return int(lib.rd_kv_row_bytes(t, head_dim))


def ptr(x):
    """Device (or host) address of a torch tensor / numpy array / None / int."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return x.ctypes.data


def stream_ptr(stream=None):
    """cudaStream_t of a torch stream (None = torch's current stream)."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream
