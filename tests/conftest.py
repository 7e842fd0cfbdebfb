import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on first use."""
    from oracle import build_oracle
    build_oracle.build_oracle()
    from oracle import oracle as orc
    return orc


@pytest.fixture(scope="session")
def pspmm_lib():
    """libpspmm.so through ctypes, built on first use (nvcc cross-compiles without a GPU)."""
    from paramspmm_ae_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
