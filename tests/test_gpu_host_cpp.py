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
    assert "0 failed" in res.stdout and res.stdout.count("ran Test") == 15


@pytest.mark.gpu
def test_threads_share_a_context(gpu_lib):
    """Eight host threads, two batches in flight each, one context: counters, replay verdicts and plaintext stay
    right (bnk_b200/host/apps/mt_stress.cpp); once with copies, once on the pinned host arrays."""
    from bnk_b200 import _build

    exe = _build.build_mt_stress()
    for env_extra, packets, size in (({}, 128, 1420), ({}, 32, 576), ({"BNK_HOST_DIRECT_BYTES": "0"}, 32, 576)):
        res = subprocess.run([exe, "8", "60", str(packets), str(size), "2"], capture_output=True, text=True, timeout=300,
                             env={**os.environ, **env_extra})
        print(res.stdout[-500:], res.stderr[-2000:])
        assert res.returncode == 0 and res.stdout.startswith("OK"), res.stdout[-500:] + res.stderr[-2000:]
