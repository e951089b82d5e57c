import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "metaattention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def reference_root():
    """Directory of a checkout of the reference project (the one holding examples/ and testing/test.py), or None.
    Looked for in $ATTN_B200_REFERENCE, then baseline/_ref/ of this repository, then the checkout the build environment provides."""
    for cand in (os.environ.get("ATTN_B200_REFERENCE"), os.path.join(ROOT, "baseline", "_ref"), "/root/reference"):
        if cand and os.path.isfile(os.path.join(cand, "testing", "test.py")) and os.path.isdir(os.path.join(cand, "examples")):
            return cand
    return None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built if necessary (nvcc cross-compiles without a GPU)."""
    from core.native import lib
    lib.build_library()
    return lib.load_library()
