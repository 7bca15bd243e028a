import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture
def device_ok():
    """For GPU tests: after the test body, no bounded device-side wait may have run out."""
    yield
    from flashck_b200 import _lib
    assert _lib.device_status() == 0, "a device-side wait timed out"
