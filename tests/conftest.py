import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lib_built():
    from vexel_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def be(lib_built):
    """One CUDA backend context for the whole GPU session."""
    from vexel_b200 import Backend
    b = Backend(0)
    yield b
    b.close()
