"""pytest configuration: registers the ``gpu`` marker and puts the repository root
(for ``oracle``) and the package directory (for ``polarquant_kv``) on sys.path."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "polarquant-kv_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device")


@pytest.fixture(scope="session")
def golden():
    """Committed fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
    path = os.path.join(ROOT, "tests", "golden", "pq4_golden.npz")
    with np.load(path) as z:
        return {k: z[k] for k in z.files}
