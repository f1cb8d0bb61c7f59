import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def cases_of(gold):
    """Case names in a golden file: the part of each key before the first dot."""
    return sorted({k.split(".")[0] for k in gold if "." in k})


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bit_equal(a, b):
    """Same float32 bit patterns (distinguishes -0 from +0, treats identical NaNs as equal)."""
    a = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    b = np.ascontiguousarray(np.asarray(b, dtype=np.float32))
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    return O.restatement()


@pytest.fixture(scope="session")
def reference_backend():
    """The reference's compiled CPU backend when its library is present, else None."""
    import oracle as O
    ref = O.reference()
    if ref is not None:
        O.reference_use_plain_blas()
    return ref


@pytest.fixture(scope="session")
def gpu():
    """(nn, mat, ctx) on cuda:0; the tests that use it are marked gpu."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test collected on a machine without CUDA"
    from matconvnet_b200 import mat, nn
    torch.cuda.set_device(0)
    return nn, mat, nn.default_context()
