import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def lib():
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.build import build

    build()
    return _lib.load()


@pytest.fixture(scope="session")
def oracle():
    from oracle import nvfp4_oracle

    nvfp4_oracle.build_c()
    return nvfp4_oracle
