import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def registry():
    from harp_b200.backend import B200BackendRegistry
    return B200BackendRegistry()


@pytest.fixture(scope="session")
def dev(registry):
    """One device for the whole session.  GPU tests fail (not skip) when the
    CUDA library or the device is missing: there is no other execution path."""
    d = registry.create_device(0)
    yield d
    d.synchronize()
