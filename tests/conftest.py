import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def built_lib():
    """libffa_b200.so, built in-tree if it is stale or missing (nvcc only, no GPU needed)."""
    from ffa_speedtest_b200 import build
    return build.build()
