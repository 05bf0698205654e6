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


@pytest.fixture(scope="session")
def cpp_caller(cuda_lib, tmp_path_factory):
    """tests/cpp/decoder_sentence_main.cpp (the reference's sentence-decoding loop written against
    include/linmt_decoder_sentence.hpp), compiled and linked against the CUDA library."""
    import subprocess
    out = str(tmp_path_factory.mktemp("cpp") / "decoder_sentence_main")
    libdir = os.path.join(ROOT, "linmt_b200")
    subprocess.run(["g++", "-std=c++17", "-I" + os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "decoder_sentence_main.cpp"), "-o", out,
                    "-L" + libdir, "-llinmt_decoder", "-Wl,-rpath," + libdir], check=True)
    return out
