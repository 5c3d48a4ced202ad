import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ext():
    """The operator module; importing it fails loudly if it has not been built."""
    import bw1000_dsv4_kernels_b200 as pkg
    return pkg.dsv4_native_ext


@pytest.fixture(scope="session")
def cabi():
    from tests import cabi_calls
    return cabi_calls
