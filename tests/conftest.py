import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    """The product package; the library must be built (no fallback)."""
    p = graft.load_package()
    if not os.path.exists(p.LIB_PATH):
        p.build()
    p.lib()
    return p


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure)."""
    o = graft.load_oracle()
    o.lib()
    return o


@pytest.fixture(scope="session")
def synth(pkg):
    import importlib
    return importlib.import_module(graft.PKG_NAME + ".synth")


@pytest.fixture(scope="session")
def dev(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
