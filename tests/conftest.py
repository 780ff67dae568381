import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def dev():
    """One ug_b200.Device for the whole session (device 0)."""
    import ug_b200
    d = ug_b200.Device(0)
    yield d
    d.synchronize()


def rel_err(got, ref, floor=1e-30):
    """max |got - ref| / max(|ref|, floor) elementwise."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor))) if ref.size else 0.0
