"""Shared fixtures.  GPU tests are marked `gpu`; everything else runs on a CPU-only box."""
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

from __graft_entry__ import load_package  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def hom(pkg):
    """The loaded C-ABI library.  Raises (does not skip) when the library is missing."""
    return pkg.runner()


@pytest.fixture(scope="session")
def oracle():
    from oracle import hom_oracle
    hom_oracle.lib()
    return hom_oracle


@pytest.fixture()
def cuda(hom):
    """A CUDA device with the library bound to torch's current stream."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    hom.clear_error()
    hom.use_torch_stream()
    yield torch.device("cuda:0")
    hom.synchronize()
