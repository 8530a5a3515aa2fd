import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure), built on first use."""
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def model_dir(tmp_path_factory):
    d = os.environ.get("WICK_SYNTH_CACHE") or str(tmp_path_factory.mktemp("wick_models"))
    os.makedirs(d, exist_ok=True)
    return d


@pytest.fixture(scope="session")
def cuda_lib():
    """The product library; building needs nvcc, running needs a GPU."""
    from wick_b200 import _lib, build
    build.build()
    return _lib.load()
