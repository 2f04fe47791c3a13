import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box with -m gpu)")


@pytest.fixture(scope="session")
def engine_lib():
    """The CUDA library, built if needed.  GPU tests must run the real thing: no skip when it fails to load."""
    from graphtsetlinmachine_b200 import build, _lib

    build.build()
    return _lib.load()
