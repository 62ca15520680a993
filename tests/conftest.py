import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built():
    """The product library and the oracle, built if stale."""
    from soliton_b200 import build
    from oracle import build as obuild
    build.build()
    obuild.build_oracle()
    return True


@pytest.fixture(scope="session")
def lib(built):
    from soliton_b200._C import lib as L
    return L


@pytest.fixture(scope="session")
def cuda(lib):
    """Initialises cuda:0 through the library once per session."""
    from soliton_b200 import tensor as T
    if lib.sl_cuda_count() < 1:
        pytest.fail("a test marked gpu ran without a CUDA device")
    T._dev(T.CUDA)
    lib.slb_set_option(b"timeout_ms", 3000)  # a protocol bug should end a test in seconds, not hang it
    return T.CUDA
