"""Shared pytest configuration: registers the ``gpu`` marker and puts the repository
root on ``sys.path`` so that ``oracle`` and the package shim import from a checkout."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    """Loader for the fixtures produced by tests/golden/make_golden.py (reference outputs)."""
    cache = {}

    def load(name):
        if name not in cache:
            cache[name] = np.load(os.path.join(GOLDEN, f"golden_{name}.npz"))
        return cache[name]
    return load
