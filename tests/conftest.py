"""Shared fixtures.  Tests marked `gpu` need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def same_bits(a, b):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    from oracle import Ref
    if not Ref.available():
        pytest.skip("reference library not built here")
    return Ref()


@pytest.fixture(scope="session")
def gpu():
    """The initialised CUDA library (python mirror).  Fails, never skips, when the
    library cannot be loaded: a silent fallback would hide a broken build."""
    import moty_b200 as mb
    mb.init([0])
    yield mb
