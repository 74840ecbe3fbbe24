"""Shared pytest configuration: the ``gpu`` marker and common helpers."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def rel_err(a, b):
    """max|a - b| / max|b| -- the reference's own parity metric
    (tests/test_fused_regularization.py:36-39 of the reference)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = max(float(np.abs(b).max()) if b.size else 0.0, 1e-300)
    return float(np.abs(a - b).max() / den) if b.size else 0.0


def pytest_sessionstart(session):
    """The package refuses to import without its CUDA library: build it (nvcc cross-compiles
    without a GPU) when it is missing or older than its sources."""
    import importlib.util
    # loaded by path: importing the package itself already needs an up-to-date library
    spec = importlib.util.spec_from_file_location("_kan_b200_build", os.path.join(ROOT, "torchsplinekan_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all()
