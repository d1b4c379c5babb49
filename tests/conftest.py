import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def _has_gpu():
    try:
        from libinferbit_b200 import _ffi
        return _ffi.load_ibcu().ibcu_device_count() > 0
    except OSError:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no GPU visible")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def cpu_libs():
    """The two CPU checkers: this repo's restatement and (when it has been built) the reference."""
    from tests import _cpu
    return _cpu.load()


@pytest.fixture(scope="session")
def backend():
    from libinferbit_b200 import Backend
    be = Backend(0)
    yield be
    be.close()
