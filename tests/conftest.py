import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def oxlib():
    """The CUDA library, built if stale.  No fallback: a build failure fails the test."""
    from oxcamlgpu_b200 import build
    build.build_library()
    from oxcamlgpu_b200 import _lib
    return _lib.lib()
