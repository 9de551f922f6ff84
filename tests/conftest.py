"""pytest configuration: registers the ``gpu`` marker and puts the repo root on sys.path."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.tqo import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_vectors.npz"))


@pytest.fixture
def force_path():
    """Returns a function force(path, umma=None) that forces a kernel path / tensor-core kernel of the library
    for the rest of the test (tqt_cuda_debug_set_path); the automatic choice is restored afterwards."""
    from __graft_entry__ import load
    pkg = load()

    def force(path, umma=None):
        pkg.debug_set_path(path, umma)

    yield force
    pkg.debug_set_path(None, None)
