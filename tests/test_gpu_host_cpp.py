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
    assert "0 failed" in res.stdout and res.stdout.count("ran Test") == 17


@pytest.mark.gpu
def test_threads_share_a_context(gpu_lib):
    """Eight host threads, two batches in flight each, one context: counters, replay verdicts and plaintext stay
    right (bnk_b200/host/apps/mt_stress.cpp); on the pinned host arrays (the default for batches this small), with
    copies, and with 24 batches in flight, more than may run on the host arrays at a time, so that both ways mix."""
    from bnk_b200 import _build

    exe = _build.build_mt_stress()
    for env_extra, threads, packets, size, lanes in (({}, 8, 128, 1420, 2), ({}, 8, 32, 576, 2), ({}, 6, 128, 1420, 4),
                                                    ({"BNK_HOST_DIRECT_BYTES": "0"}, 8, 128, 1420, 2),
                                                    ({"BNK_HOST_DIRECT_BYTES": "0"}, 8, 32, 576, 2)):
        res = subprocess.run([exe, str(threads), "60", str(packets), str(size), str(lanes)], capture_output=True, text=True,
                             timeout=300, env={**os.environ, **env_extra})
        print(res.stdout[-500:], res.stderr[-2000:])
        assert res.returncode == 0 and res.stdout.startswith("OK"), res.stdout[-500:] + res.stderr[-2000:]



@pytest.mark.gpu
def test_threads_share_the_submit_queues(gpu_lib):
    """The same eight threads hand their 128-packet calls to two shared submit queues (bnk_queue) instead of
    batches of their own: nonces per keypair in call order, plaintext back, second delivery refused."""
    from bnk_b200 import _build

    exe = _build.build_mt_stress()
    # (threads, calls outstanding per thread, 1 = copying calls / 2 = spans on the pinned ring); 24 threads: more
    # callers than cores, the waiting ones give their cores away
    for threads, lanes, mode in ((8, 2, 1), (5, 3, 1), (8, 2, 2), (5, 3, 2), (24, 2, 1)):
        res = subprocess.run([exe, str(threads), "60", "128", "1420", str(lanes), str(mode)], capture_output=True, text=True, timeout=300)
        print(res.stdout[-500:], res.stderr[-2000:])
        assert res.returncode == 0 and "\nOK mode=queue" in "\n" + res.stdout, res.stdout[-500:] + res.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["asan", "tsan"])
def test_host_layer_under_sanitizers(gpu_lib, kind):
    """The library's host code (C ABI plumbing, submit queue, dispatcher, C++ mirror) built with
    AddressSanitizer + UndefinedBehaviorSanitizer, and with ThreadSanitizer, runs the restated Go tests and the
    threaded stress (own batches and shared queues) without a report.  Device code is not instrumented; the GPU
    calls are ordinary host API calls to the sanitizers."""
    from bnk_b200 import _build

    out = _build.build_sanitized(kind)
    env = dict(os.environ)
    if kind == "asan":
        # the CUDA driver maps memory where ASan keeps a gap, and keeps allocations of its own for the process's lifetime
        env["ASAN_OPTIONS"] = "protect_shadow_gap=0:detect_leaks=0:abort_on_error=0"
        env["UBSAN_OPTIONS"] = "print_stacktrace=1"
    else:
        env["TSAN_OPTIONS"] = "report_signal_unsafe=0"
    runs = [[os.path.join(out, "host_test")],
            [os.path.join(out, "mt_stress"), "4", "20", "128", "1420", "2", "0"],
            [os.path.join(out, "mt_stress"), "4", "20", "128", "1420", "2", "1"],
            [os.path.join(out, "mt_stress"), "4", "20", "128", "1420", "2", "2"]]
    for cmd in runs:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        text = res.stdout + res.stderr
        print(text[-1500:])
        assert res.returncode == 0, text[-3000:]
        for mark in ("ThreadSanitizer", "AddressSanitizer", "runtime error"):
            assert mark not in text, text[-3000:]
