import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "reads_status: the test inspects the device status block itself")


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library, built on demand (nvcc cross-compiles without a GPU)."""
    from fast_route_b200 import _lib, build
    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test the device status block must be clean (no expired waits,
    no out-of-range ids) unless the test reads it itself."""
    yield
    if request.node.get_closest_marker("gpu") and not request.node.get_closest_marker("reads_status"):
        import torch
        if torch.cuda.is_available():
            from fast_route_b200 import _lib
            code, detail, block, count = _lib.device_status()
            assert code == 0, f"device status {code} detail {detail:#x} block {block} count {count}"
