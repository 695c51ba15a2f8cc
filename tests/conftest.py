import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# GPU files in order of importance: the benchmarked scan first, the rows next to the path
# after it.  Files not named keep their alphabetical place between the two groups.
_FIRST = ["test_gpu_scan.py", "test_gpu_configs.py", "test_gpu_gemm.py", "test_gpu_multi_f32.py", "test_gpu_multi.py",
          "test_gpu_embedindex.py", "test_gpu_services.py", "test_gpu_hamming.py"]
_LAST = ["test_zz_no_alloc.py"]


def pytest_collection_modifyitems(session, config, items):
    def rank(item):
        name = os.path.basename(str(item.fspath))
        if name in _FIRST:
            return _FIRST.index(name)
        if name in _LAST:
            return len(_FIRST) + 1 + _LAST.index(name)
        return len(_FIRST)

    items.sort(key=rank)  # stable: order inside a file and among unnamed files is kept


@pytest.fixture(scope="session")
def lk():
    """The ctypes binding of the CUDA library; GPU tests fail loudly if it cannot run."""
    from loki_b200 import _lib
    assert _lib.device_count() > 0, "no CUDA device visible: GPU tests cannot run"
    return _lib
