import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 and the built libwrk.so")


@pytest.fixture(scope="session")
def wrk():
    """The ctypes harness over libwrk.so (package directory `web-rwkv_b200`)."""
    return importlib.import_module("web-rwkv_b200")


@pytest.fixture(scope="session")
def ctx(wrk):
    c = wrk.Context(0)
    yield c
    c.synchronize()
