import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def goldens():
    from support import load_goldens
    return load_goldens()


@pytest.fixture(scope="session")
def built_lib():
    """The product library, built in-tree (cross-compiles without a GPU)."""
    from dlf_b200 import build
    build.build()
    import dlf_b200
    return dlf_b200.lib()
