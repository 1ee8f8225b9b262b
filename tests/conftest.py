import os
import sys

import pytest

# The data-parallel tests tear communicators down after a host-injected failure; NCCL must then have no
# buffer bound to an NVLink multicast object, so NVLS stays off in the test process (set before the
# library loads NCCL).
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda_device():
    from quabla_b200 import _lib

    if _lib.load().qb200_device_count() < 1:
        pytest.fail("a test marked gpu ran without a CUDA device: the qb200 backend has no CPU fallback")
    return 0
