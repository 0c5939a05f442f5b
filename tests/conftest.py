import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on a GPU box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU checker (oracle/liboracle.so), built on demand with gcc."""
    from oracle import oracle as O

    O.build()
    O.lib()
    return O


@pytest.fixture(scope="session")
def gpu_lib():
    """libbnkgpu.so on a machine with a GPU; the tests never fall back to anything else."""
    from bnk_b200 import _build, _lib

    if not os.path.exists(_build.LIB_PATH):
        _build.build()
    L = _lib.lib()
    n = L.bnk_device_count()
    assert n > 0, "no CUDA device visible: " + L.bnk_last_error_string(None).decode()
    return L
