import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "metaattention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built if necessary (nvcc cross-compiles without a GPU)."""
    from core.native import lib
    lib.build_library()
    return lib.load_library()
