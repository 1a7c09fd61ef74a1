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


# largest errors seen by the GPU parity tests: (test, output) -> (max-abs, max-abs over elements below 2.56)
_ERRORS = {}


def record_error(test, what, worst, worst_small):
    key = (test, what)
    old = _ERRORS.get(key, (0.0, 0.0))
    _ERRORS[key] = (max(old[0], worst), max(old[1], worst_small))


def pytest_terminal_summary(terminalreporter):
    if not _ERRORS:
        return
    tr = terminalreporter
    tr.write_line("largest absolute errors against the fp32 reference evaluation (all / elements with |ref| < 2.56):")
    per_test = {}
    for (test, what), (a, b) in _ERRORS.items():
        fmt = (lambda x: f"{x:.4f}") if a >= 1e-3 else (lambda x: f"{x:.1e}")
        per_test.setdefault(test, []).append(f"{what.split()[-1] if ' ' in what else what} {fmt(a)}/{fmt(b)}")
    for test, items in per_test.items():
        tr.write_line(f"  {test}: " + "  ".join(items[:12]) + (" ..." if len(items) > 12 else ""))
