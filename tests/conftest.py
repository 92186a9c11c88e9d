import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The built shared library (compiled on first use; nvcc cross-compiles without a GPU)."""
    from anchor_attention_b200.build import build_library
    build_library()
    from anchor_attention_b200 import _lib
    return _lib.load()
