import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def seed_torch():
    # the reference's tests seed torch the same way (tests/conftest.py:25-27)
    torch.manual_seed(0)


@pytest.fixture(scope="session")
def built_library():
    """Build the CUDA library if needed (nvcc cross-compiles without a GPU) and return its path."""
    from wave_b200 import build
    return build.build()
