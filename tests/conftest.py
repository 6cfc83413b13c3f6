import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The CUDA extension must exist; tests never fall back to anything else."""
    from flaxattention_b200 import _cabi

    if not os.path.exists(_cabi.LIB_PATH):
        from flaxattention_b200.csrc.build import build_library

        build_library()
    yield
