import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device")
    config.addinivalue_line("markers", "timeout: per-test limit (pytest-timeout, where installed)")


def pytest_collection_modifyitems(config, items):
    """A GPU test that has not finished in 15 minutes is stuck in a kernel: end the run instead
    of waiting on it (pytest-timeout's watchdog thread; nothing happens where the plugin is
    absent, and CPU tests get no watchdog, so their worker pools fork from one thread)."""
    if not config.pluginmanager.hasplugin("timeout"):
        return
    for item in items:
        if item.get_closest_marker("gpu") and not item.get_closest_marker("timeout"):
            item.add_marker(pytest.mark.timeout(900, method="thread"))


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
