"""Shared test plumbing: the `gpu` marker, import paths, and the golden fixtures."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "box-convolutions_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden", "boxconv_golden.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return dict(np.load(GOLDEN))


def max_rel(a, b):
    """max|a-b| / max|b| -- the error measure used for outputs and gradients (element-wise
    relative error is meaningless for zero-mean tensors)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.abs(b).max()
    if denom == 0:
        return np.abs(a - b).max()
    return np.abs(a - b).max() / denom
