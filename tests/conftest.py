"""Shared test setup.  Tests marked ``gpu`` need a CUDA device and are the parity tests
proper: they call the sm_100a kernels through the C ABI and compare with the CPU oracle."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built_lib():
    """Path of libmonet_b200.so.  The build is incremental on source mtimes, so it is called
    whenever nvcc is present: a library older than its sources is never tested."""
    import shutil
    from monet_b200 import _lib, build
    if shutil.which("nvcc") or not _lib.LIB_PATH.exists():
        build.build()
    return _lib.LIB_PATH


@pytest.fixture(scope="session")
def cuda(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda:0")
