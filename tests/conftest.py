import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lk():
    """The ctypes binding of the CUDA library; GPU tests fail loudly if it cannot run."""
    from loki_b200 import _lib
    assert _lib.device_count() > 0, "no CUDA device visible: GPU tests cannot run"
    return _lib
