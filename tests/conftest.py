import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    config.addinivalue_line("markers", "slow: long-running test")


@pytest.fixture(scope="session")
def native_lib():
    """Build (if needed) and load the native kernel library."""
    from kempnerforge_b200.ops.build import build

    build()
    from kempnerforge_b200.ops import cuda as kcuda

    kcuda.lib()
    return kcuda
