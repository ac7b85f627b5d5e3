import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# Set by tests/test_gpu_bounds_checked.py for the pytest run it starts: every suite then runs on the bounds-checked build
# of the library (pixienn_b200/debug.py), and a test fails when one of its kernels made an access outside the live
# allocations.
BOUNDS_CHECKED = os.environ.get("PXE_TEST_BOUNDS_CHECKED") == "1"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    if BOUNDS_CHECKED:
        from pixienn_b200 import debug
        debug.use_checked_library()


@pytest.fixture(autouse=True)
def _no_refused_accesses():
    yield
    if BOUNDS_CHECKED:
        import torch
        from pixienn_b200 import debug
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            rep = debug.read_report(reset=True)
            assert rep.violations == 0, debug.describe(rep)


@pytest.fixture(scope="session")
def oracle():
    from oracle import pxoracle
    pxoracle.lib()
    return pxoracle


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    from pixienn_b200 import capi
    capi.lib()          # raises when libpxe.so is missing: no fallback
    return torch.device("cuda:0")
