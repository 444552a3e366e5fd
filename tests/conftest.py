import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# The unmodified upstream library mis-dispatches on AVX-512 hosts unless told to stay on AVX.
os.environ.setdefault("XNOR_NN_ISA", "2")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.pyoracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "upstream_golden.npz")
    return np.load(path)
