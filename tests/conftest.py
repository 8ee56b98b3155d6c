import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name + ".npz"))
    return load


@pytest.fixture(scope="session")
def rd():
    """The product package (directory name carries a hyphen, so import by string)."""
    return importlib.import_module("rdna4-infer_b200")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


def cos_sim(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / (na * nb))


def check_attn(got, want, max_abs=2e-3, min_cos=0.9999, what=""):
    """The stated gates for attention output: max-abs error 2e-3, cosine >= 0.9999."""
    got = np.asarray(got)
    want = np.asarray(want)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max())
    cs = cos_sim(got, want)
    assert err <= max_abs, f"{what}: max-abs {err:.3e} > {max_abs}"
    assert cs >= min_cos, f"{what}: cosine {cs:.6f} < {min_cos}"
    return err, cs
