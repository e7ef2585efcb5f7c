import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def backend():
    from webgpu_b200 import backend as B
    return B.load()


@pytest.fixture(scope="session")
def ctx(backend):
    """One context on cuda:0 for the whole session; fails loudly without a GPU."""
    c = backend.create_context(0)
    yield c
    c.destroy()
