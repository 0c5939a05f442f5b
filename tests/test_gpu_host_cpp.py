"""Runs the C++ host-mirror tests (tests/cpp/host_test.cpp): the reference's Go filter / TUN tests restated in
C++ and a two-device round trip, all through libbnkgpu.so on the GPU."""
import os
import subprocess

import pytest


def test_host_mirror_compiles_and_links():
    """CPU-side check: the C++ host layer and its test build against the C ABI."""
    from bnk_b200 import _build

    exe = _build.build_host_test()
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_reference_go_tests_restated_in_cpp(gpu_lib):
    from bnk_b200 import _build

    exe = _build.build_host_test()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "0 failed" in res.stdout and res.stdout.count("ran Test") == 14
