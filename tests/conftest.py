import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    """The product package (deeplink.framework_b200/) under its importable name."""
    import __graft_entry__ as entry
    return entry.load_package()


@pytest.fixture(scope="session")
def diopi(pkg):
    return pkg.diopi


@pytest.fixture(scope="session")
def devapis(pkg):
    return pkg.devapis


@pytest.fixture()
def ctx(diopi):
    import torch
    assert torch.cuda.is_available()
    c = diopi.Context()
    yield c
    torch.cuda.synchronize()
    c.release_workspace()
