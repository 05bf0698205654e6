import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import build_oracle, oracle_py
    build_oracle.build()
    return oracle_py


@pytest.fixture(scope="session")
def cuda_lib():
    from linmt_b200 import build, _lib
    build.build()
    return _lib.load()
