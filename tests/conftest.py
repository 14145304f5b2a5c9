"""pytest configuration: the `gpu` marker and import paths.

GPU tests call the kernels through the C ABI (ctypes -> libemmyb200.so) and check them against
the CPU oracle in `oracle/`; everything unmarked runs without a GPU.
"""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "emmy-ptx-compiler_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The built kernel library; building it is the job of `__graft_entry__.build()`."""
    from emmyptx import runtime
    return runtime.library()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked `gpu` ran without a CUDA device")
    return torch.device("cuda:0")
