import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on a GPU box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (compiled on first use)."""
    import oracle as _oracle
    _oracle.build()
    return _oracle


@pytest.fixture(scope="session")
def engine():
    """One engine on cuda:0 shared by the GPU tests."""
    import volta_b200
    eng = volta_b200.Engine(0)
    yield eng
    eng.close()
