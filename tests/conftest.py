import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "amd-kernels_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library must exist before any test imports the package."""
    sys.path.insert(0, PKG)
    import build as ma_build  # amd-kernels_b200/build.py

    ma_build.build()
    oracle_lib = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(oracle_lib):
        import subprocess

        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True)
    yield


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    os.environ["MOONMATH_CHECK"] = "1"  # every forward() call checks the device status word
    return torch.device("cuda:0")
