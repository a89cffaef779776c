import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Make sure the product library and the oracle are built (both cross-compile without a GPU)."""
    from smat_b200 import _build
    _build.build()
    import oracle
    if not os.path.exists(os.path.join(ROOT, "oracle", "libsmat_oracle.so")):
        oracle.build()
    yield


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
