import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


def _has_cuda():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope="session")
def ops():
    """The backend through its C ABI. GPU tests fail (not skip) when the library is missing."""
    from libnd4j_b200.native_ops import NativeOps
    if not _has_cuda():
        pytest.skip("no CUDA device")
    return NativeOps()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU implementation (oracle/_ref), or the port when it was not built."""
    from oracle import reference
    if reference.available():
        return reference.Reference()
    from oracle import port
    return port.Port()


@pytest.fixture(scope="session")
def real_ref():
    from oracle import reference
    if not reference.available():
        pytest.skip("oracle/_ref/libnd4jref.so not built (needs the reference checkout)")
    return reference.Reference()


@pytest.fixture(scope="session")
def maybe_ref():
    """The reference build when oracle/_ref is present, else None: GPU tests of the memory-movement utilities
    compare with it directly in addition to the restatements it pins (tests/test_oracle_utilities.py)."""
    from oracle import reference
    return reference.Reference() if reference.available() else None
