import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def api():
    from nextsycl_b200 import api as a
    return a.load()


@pytest.fixture(scope="session")
def gpu(api):
    """GPU 0 opened through the C ABI. The library has no CPU path: without a device this fails loudly."""
    from nextsycl_b200 import Gpu
    g = Gpu(0, api)
    yield g
    g.close()


@pytest.fixture(scope="session")
def ops(gpu):
    from nextsycl_b200 import Ops
    return Ops(gpu)
