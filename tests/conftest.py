import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a); run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def gpu():
    """The library's device handle.  A missing library or device is an error, never a skip to CPU."""
    import ratchet_b200 as rb

    return rb.Device.request_device(rb.DeviceRequest.GPU)
