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


def pytest_sessionfinish(session, exitstatus):
    """When the session ran against the debug-checked build of the library
    (WAVE_B200_LIB=wave_b200/libwave_b200_checks.so python -m pytest tests -m gpu), no index predicate of the kernels may
    have failed in any test: read the device-side record and turn a non-empty one into a failing exit status."""
    import ctypes
    import os
    if "checks" not in os.path.basename(os.environ.get("WAVE_B200_LIB", "")) or not torch.cuda.is_available():
        return
    from wave_b200 import _lib
    record = (ctypes.c_ulonglong * 3)()
    if _lib.load().wb200_debug_checks(record, 0) == _lib.WB200_OK and record[2]:
        print(f"\nwave_b200 checked build: {record[2]} predicate(s) failed; first: code {record[0] & 0xFFFFFFFF}, "
              f"CTA {record[0] >> 32}, detail {record[1]}")
        session.exitstatus = 1
    else:
        print("\nwave_b200 checked build: no predicate failed")
