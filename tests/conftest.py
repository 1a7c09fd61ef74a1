import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "triton-flash-attention-with-flexible-masks_b200")
for p in (PKG, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def repo_root():
    return ROOT


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library is built in-tree before any test runs (nvcc needs no GPU)."""
    so = os.path.join(PKG, "flash_b200", "libfa_b200.so")
    if not os.path.exists(so):
        sys.path.insert(0, PKG)
        import build
        build.build()
    return so
