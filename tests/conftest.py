import os
import shutil
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """The CUDA library must exist before anything imports the kernels layer.  Build it when it is
    missing or stale and nvcc is at hand; otherwise use the prebuilt file that travelled with the tree."""
    from cpm_kernels_b200 import build
    if build.is_stale() and shutil.which(os.environ.get("NVCC", "nvcc")):
        build.build_library()
    return build.LIB_PATH


@pytest.fixture(scope="session")
def c_oracle():
    from oracle import quant_linear
    return quant_linear.COracle()
