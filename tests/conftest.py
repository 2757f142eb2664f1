import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def rel_err(a, b):
    """max |a-b| / max |b| : the 'max relative error' every parity test uses, per tensor"""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    m = np.abs(b).max() if b.size else 0.0
    return float(np.abs(a - b).max() / (m if m > 0 else 1.0)) if b.size else 0.0


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
