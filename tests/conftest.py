import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu); everything else runs on CPU")


@pytest.fixture(scope="session", autouse=True)
def native_libs():
    """Both native libraries are built in-tree before any test touches them."""
    from msnhnet_b200 import build
    build.build_all()
    yield


def _has_gpu():
    try:
        import ctypes
        from msnhnet_b200 import _ffi
        n = ctypes.c_int()
        return _ffi.kernel_lib().msnh_b200_device_count(ctypes.byref(n)) == 0 and n.value > 0
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    # GPU tests fail loudly without a device when they are selected with -m gpu; they are only
    # skipped when the whole suite is collected on a CPU box without a marker expression.
    if config.getoption("-m"):
        return
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no GPU in this process; run with -m gpu on a B200")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
