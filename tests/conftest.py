import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def device():
    """A CudaDevice on GPU 0.  GPU tests must run the CUDA library: no skip, no fallback."""
    from candy_b200.backend import CudaDevice
    return CudaDevice(int(os.environ.get("CANDYQ_TEST_DEVICE", "0")))
