import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle_libs():
    """Builds the C oracle and the CPU baseline once per session."""
    from oracle import build
    build.build()
    return build


@pytest.fixture(scope="session")
def hb_lib():
    """Builds (if stale) and loads libheron_b200.so."""
    from heron_b200 import _lib, build
    build.build()
    return _lib.load()
