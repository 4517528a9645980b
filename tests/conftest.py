import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device")


@pytest.fixture(scope="session")
def orc():
    from oracle import native
    return native.oracle()


@pytest.fixture(scope="session")
def gpu():
    """The loaded lmz_b200.gpu module; fails loudly when the library is unusable."""
    from lmz_b200 import gpu as g
    ok, why = g.available()
    assert ok, f"the CUDA library must load on a GPU box: {why}"
    return g
