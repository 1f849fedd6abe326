import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def sm100():
    """The CUDA library through its C ABI; fails (never skips) when it cannot run on a GPU box."""
    from scrapgpulibrary_b200 import capi
    capi.require_device()
    return capi


@pytest.fixture(scope="session")
def stream(sm100):
    s = sm100.Stream(0)
    yield s
    s.close()
