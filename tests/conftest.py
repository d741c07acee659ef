import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def runtime_lib():
    """Builds (if needed) and loads the C-ABI library."""
    from numba_mlir_b200 import build, runtime

    build.build()
    return runtime.load()


@pytest.fixture(scope="session")
def queue(runtime_lib):
    from numba_mlir_b200 import runtime

    return runtime.get_queue()
