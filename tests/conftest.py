import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def native_built():
    """Builds (if stale) and returns the paths of the native artefacts. nvcc works without a GPU."""
    from hipkittens_b200 import _build

    return _build.build_all()
