import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (run with -m gpu on a GPU box)")


@pytest.fixture(scope="session")
def dccl_lib():
    """The native library, built on demand."""
    from dccl_b200 import _lib
    return _lib.lib()


@pytest.fixture(scope="session")
def build_dir(dccl_lib):
    """Directory with the command-line tools (dccl_cli, helloworld, ...)."""
    from dccl_b200 import _lib
    d = os.path.join(ROOT, "build")
    if not os.path.exists(os.path.join(d, "dccl_cli")):
        _lib.build()
    return d


def gpu_count():
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0
