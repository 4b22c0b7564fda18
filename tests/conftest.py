import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on the B200 box)")


@pytest.fixture(scope="session")
def backend():
    """One CudaBackend on cuda:0 for the whole session; fails (not skips) without a GPU."""
    from agention_infer_b200 import CudaBackend
    be = CudaBackend(0)
    yield be
    be.close()
