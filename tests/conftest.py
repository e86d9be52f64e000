"""pytest configuration: the `gpu` marker and the one-time build of libwsl.so.

`-m "not gpu"` tests run anywhere (oracle vs golden fixtures, host logic, C-ABI symbol
checks, gloo data-parallel logic). `-m gpu` tests are the parity tests proper and call the
CUDA kernels through the C ABI on a B200.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100)")


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """Build libwsl.so when it is missing or stale and nvcc is present; otherwise use the
    prebuilt file that travelled with the tree."""
    from weightshared_torchtitan_b200 import build
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if build.needs_build() and os.path.exists(nvcc):
        build.build_library()
    if not os.path.exists(build.LIB_PATH):
        pytest.exit("libwsl.so is missing and nvcc is not available to build it", returncode=3)
    return build.LIB_PATH


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
