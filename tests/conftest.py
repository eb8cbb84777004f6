import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from harness import OracleBackend
    return OracleBackend()


@pytest.fixture(scope="session")
def cuda():
    """The CUDA library through the reference's calling pattern.  Fails (does not skip)
    when the library is missing: there is no fallback path to test instead."""
    from harness import CudaBackend
    from maidenx_b200 import _lib
    _lib.load()
    return CudaBackend()


@pytest.fixture(scope="session")
def cuda_hostmeta():
    from harness import CudaBackend
    from maidenx_b200 import _lib
    _lib.load()
    return CudaBackend(metadata_on_host=True)
