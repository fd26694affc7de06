import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; the parity tests proper")


@pytest.fixture(scope="session")
def pkg():
    """The package bound to the built C-ABI library (built on demand; no fallback exists)."""
    import __graft_entry__ as ge
    ge.build()
    return ge.load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch
    assert torch.cuda.is_available(), "gpu-marked test run without a GPU"
    torch.cuda.set_device(0)
    assert pkg.num_sms() > 0, "libb200gemm.so could not initialise an sm_100 device"
    return torch
