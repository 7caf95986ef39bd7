import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: test needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="session")
def native_built():
    """Build the extension once per session (nvcc cross-compiles without a GPU)."""
    from helix_a2a_b200 import _build
    _build.build()
    return True


@pytest.fixture(scope="session")
def host_lib():
    import ctypes
    from helix_a2a_b200 import _build
    path = _build.build_host_lib()
    return ctypes.CDLL(str(path))
