import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def fa_lib():
    """The C-ABI library, built on demand (nvcc cross-compiles without a GPU)."""
    from tfg_flashattention_b200 import _lib, build
    build.build_library()
    return _lib.load()


@pytest.fixture(scope="session")
def torch_binding(fa_lib):
    """The compiled pybind11 / torch-extension binding, built on demand (g++ against the installed
    torch); None where it cannot be built, so that the tests of the ctypes route still run."""
    from tfg_flashattention_b200 import build
    try:
        build.build_torch_binding()
    except Exception as e:      # no compiler, no torch headers
        return None
    from tfg_flashattention_b200 import _custom_flash_attn_ext
    return _custom_flash_attn_ext


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
