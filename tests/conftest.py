import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure), built on demand."""
    from oracle import oracle as O
    O.build()
    O.lib()
    return O


@pytest.fixture(scope="session")
def brrr():
    """The product library through its ctypes binding (built on demand; nvcc needs no GPU)."""
    import cpubrrr_b200
    from cpubrrr_b200 import build
    build.build()
    cpubrrr_b200.lib()
    return cpubrrr_b200


@pytest.fixture(scope="session")
def dev():
    import torch
    torch.cuda.init()
    return torch.device("cuda:0")


def to_dev(a, dev):
    """numpy -> torch CUDA tensor keeping the dtype (uint16 carried as int16 bits)."""
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(dev)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(dev)
    return torch.from_numpy(a).to(dev)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
