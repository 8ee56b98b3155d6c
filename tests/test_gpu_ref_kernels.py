"""Second, GPU-side cross-check: the reference project's OWN launchers (compiled unmodified
for sm_100a into oracle/_ref/librd_ref_gpu.so) and the product kernels on the same device,
same bytes. Skipped where that library was not built (no reference checkout at build
time); the primary oracle is the CPU restatement.

Only f16 / f32 caches go through the reference's attention kernels here: its q8_0 / q4_0 /
q5_0 / q4_1 loaders read 32-bit words at block + 2 (kv.h:281-283, 299-301 of the
reference), which RDNA splits and an NVIDIA GPU rejects as a misaligned address, so those
instantiations are never launched. The quantizing STORE kernels write bytes and halves at
their natural alignment and are compared for all six types."""
import numpy as np
import pytest
import torch

from tests.conftest import check_attn

pytestmark = pytest.mark.gpu
NH, NKV, HD = 24, 4, 256


@pytest.fixture(scope="module")
def G(cuda):
    from tests import gpu_util
    return gpu_util


@pytest.fixture(scope="module")
def refgpu():
    from oracle.oracle import ReferenceGpu
    try:
        return ReferenceGpu()
    except (FileNotFoundError, OSError) as e:
        pytest.skip(f"reference GPU library not built: {e}")


@pytest.mark.parametrize("kt,vt,n,splits", [(1, 1, 4096, 4), (1, 1, 700, 4), (0, 0, 1500, 3), (1, 0, 300, 1),
                                            (0, 1, 33, 1)])
def test_decode_against_reference_kernels(G, refgpu, kt, vt, n, splits):
    rd, lib = G.rd, G.lib
    st = G.st()
    kc = torch.empty(n * NKV * rd.row_bytes(kt), dtype=torch.uint8, device="cuda")
    vc = torch.empty(n * NKV * rd.row_bytes(vt), dtype=torch.uint8, device="cuda")
    rd.check(lib.rd_kv_fill(kt, rd.ptr(kc), n * NKV, HD, 5, st))
    rd.check(lib.rd_kv_fill(vt, rd.ptr(vc), n * NKV, HD, 6, st))
    q = torch.randn(NH, HD, device="cuda", generator=torch.Generator(device="cuda").manual_seed(n))
    ours, theirs = G.poison((NH, HD)), G.poison((NH, HD))
    part = G.poison((NH, max(splits, 1), 2 + HD))
    rd.check(lib.rd_attn_decode(rd.ptr(q), rd.ptr(kc), rd.ptr(vc), rd.ptr(ours), n - 1, NH, NKV, HD, 1 / 16,
                                kt, vt, st))
    if splits > 1:
        rc = refgpu.lib.refgpu_attn_split(rd.ptr(q), rd.ptr(kc), rd.ptr(vc), rd.ptr(theirs), rd.ptr(part),
                                          n - 1, NH, NKV, HD, 1 / 16, kt, vt, splits, st)
    else:
        rc = refgpu.lib.refgpu_attn(rd.ptr(q), rd.ptr(kc), rd.ptr(vc), rd.ptr(theirs), n - 1, NH, NKV, HD,
                                    1 / 16, kt, vt, st)
    assert rc == 0
    torch.cuda.synchronize()
    check_attn(G.host(ours), G.host(theirs), what="product vs reference kernel")
    G.status_ok()


def test_kv_store_bytes_against_reference_kernel(G, refgpu):
    rd, lib = G.rd, G.lib
    src = torch.randn(64 * NKV * HD, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    for t in range(6):
        nbytes = 64 * NKV * rd.row_bytes(t)
        a = torch.full((nbytes,), 0xA5, dtype=torch.uint8, device="cuda")
        b = torch.full((nbytes,), 0xA5, dtype=torch.uint8, device="cuda")
        rd.check(lib.rd_kv_store_rows(t, rd.ptr(src), rd.ptr(a), src.numel(), G.st()))
        assert refgpu.lib.refgpu_kv_store_rows(t, rd.ptr(src), rd.ptr(b), src.numel(), G.st()) == 0
        torch.cuda.synchronize()
        assert torch.equal(a, b), f"type {t}"


def test_prefill_against_reference_fa2(G, refgpu):
    rd, lib = G.rd, G.lib
    n_q, pos0 = 512, 1536
    keys = pos0 + n_q
    st = G.st()
    kc = torch.empty(keys * NKV * 512, dtype=torch.uint8, device="cuda")
    vc = torch.empty_like(kc)
    rd.check(lib.rd_kv_fill(1, rd.ptr(kc), keys * NKV, HD, 11, st))
    rd.check(lib.rd_kv_fill(1, rd.ptr(vc), keys * NKV, HD, 22, st))
    q = torch.randn(n_q, NH, HD, device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    pos = torch.arange(pos0, keys, dtype=torch.int32, device="cuda")
    ours, theirs = G.poison((n_q, NH, HD)), G.poison((n_q, NH, HD))
    rd.check(lib.rd_fa2_prefill(rd.ptr(q), rd.ptr(kc), rd.ptr(vc), rd.ptr(ours), rd.ptr(pos), n_q, keys - 1,
                                keys, NH, NKV, HD, 1 / 16, st))
    assert refgpu.lib.refgpu_fa2_prefill(rd.ptr(q), rd.ptr(kc), rd.ptr(vc), rd.ptr(theirs), rd.ptr(pos), n_q,
                                         keys - 1, keys, NH, NKV, HD, 1 / 16, st) == 0
    torch.cuda.synchronize()
    check_attn(G.host(ours), G.host(theirs), what="prefill vs reference FA2 kernel")
    G.status_ok()
