"""Builds bnk_b200/libbnkgpu.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import glob
import os
import shutil
import subprocess

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libbnkgpu.so")
BENCH_CSRC = os.path.join(PKG_DIR, "bench_csrc")
BENCH_LIB_PATH = os.path.join(PKG_DIR, "libbnkgpu_bench.so")  # measurement helpers, not part of the drop-in

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]


HOST = os.path.join(PKG_DIR, "host")


def sources() -> list[str]:
    """CUDA kernels + C ABI, and the C++ host mirror of the reference's interfaces."""
    return sorted(glob.glob(os.path.join(CSRC, "*.cu"))) + sorted(glob.glob(os.path.join(HOST, "*.cpp")))


def bench_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(BENCH_CSRC, "*.cu")))


def _deps() -> list[str]:
    inc = os.path.join(os.path.dirname(PKG_DIR), "include", "bnk_gpu.h")
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HOST, "*.hpp")) + [inc]


def _bench_deps() -> list[str]:
    inc = os.path.join(os.path.dirname(PKG_DIR), "include")
    return bench_sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(inc, "bnk_gpu.h"),
                                                                     os.path.join(inc, "bnk_gpu_bench.h")]


def _stale(lib: str, deps: list[str]) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(p) > t for p in deps)


def is_stale() -> bool:
    return _stale(LIB_PATH, _deps()) or _stale(BENCH_LIB_PATH, _bench_deps())


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found: libbnkgpu.so cannot be built")
    return p


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ into libbnkgpu.so and bench_csrc/ into libbnkgpu_bench.so.  Returns the
    path of the former."""
    for lib, srcs, deps in ((LIB_PATH, sources(), _deps()), (BENCH_LIB_PATH, bench_sources(), _bench_deps())):
        if not force and not _stale(lib, deps):
            continue
        cmd = [nvcc_path(), *NVCC_FLAGS]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", lib, *srcs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        if verbose:
            print(res.stderr)
    return LIB_PATH


def _build_cpp(src: str, exe: str, force: bool) -> str:
    build()
    deps = [src, LIB_PATH, os.path.join(HOST, "bnk_host.hpp"), os.path.join(os.path.dirname(PKG_DIR), "include", "bnk_gpu.h")]
    if not force and os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    cxx = shutil.which("g++") or "g++"
    rel = os.path.relpath(PKG_DIR, os.path.dirname(exe))
    cmd = [cxx, "-O2", "-std=c++17", "-Wall", "-pthread", "-o", exe, src, "-L" + PKG_DIR, "-lbnkgpu",
           "-Wl,-rpath," + PKG_DIR, "-Wl,-rpath,$ORIGIN/" + rel]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return exe


def build_host_test(force: bool = False) -> str:
    """Compiles tests/cpp/host_test.cpp (the reference's Go tests restated in C++) against libbnkgpu.so."""
    root = os.path.dirname(PKG_DIR)
    return _build_cpp(os.path.join(root, "tests", "cpp", "host_test.cpp"), os.path.join(root, "tests", "cpp", "host_test"), force)


def build_mt_stress(force: bool = False) -> str:
    """Compiles bnk_b200/host/apps/mt_stress.cpp: several host threads driving one context through the C ABI, with
    its own checks; used by the tests and by the benchmark's small-batch section."""
    return _build_cpp(os.path.join(HOST, "apps", "mt_stress.cpp"), os.path.join(HOST, "apps", "mt_stress"), force)


SAN_FLAGS = {"asan": "-fsanitize=address,-fsanitize=undefined", "tsan": "-fsanitize=thread"}


def sanitized_dir(kind: str) -> str:
    return os.path.join(os.path.dirname(PKG_DIR), "build", "sanitized", kind)


def build_sanitized(kind: str, force: bool = False) -> str:
    """The library's host code (C ABI, submit queue, dispatcher, C++ mirror) and the two C++ test programs built
    with AddressSanitizer + UndefinedBehaviorSanitizer ("asan") or ThreadSanitizer ("tsan"): nvcc hands the
    flag to the host compiler, the device code is untouched.  Returns the directory that holds libbnkgpu.so,
    host_test and mt_stress of that kind."""
    out = sanitized_dir(kind)
    lib = os.path.join(out, "libbnkgpu.so")
    root = os.path.dirname(PKG_DIR)
    progs = {"host_test": os.path.join(root, "tests", "cpp", "host_test.cpp"),
             "mt_stress": os.path.join(HOST, "apps", "mt_stress.cpp")}
    deps = _deps() + list(progs.values())
    if not force and os.path.exists(lib) and all(os.path.exists(os.path.join(out, p)) for p in progs) and \
            all(os.path.getmtime(d) <= os.path.getmtime(lib) for d in deps):
        return out
    os.makedirs(out, exist_ok=True)
    flag = SAN_FLAGS[kind]
    runtime = ["-Xlinker", "-lasan", "-Xlinker", "-lubsan"] if kind == "asan" else ["-Xlinker", "-ltsan"]
    cmd = [nvcc_path(), "-O1", "-g", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler",
           "-fPIC," + flag + ",-fno-omit-frame-pointer", "-shared", "-o", lib, *sources(), *runtime]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc (sanitized) failed:\n" + res.stdout + res.stderr)
    cxx = shutil.which("g++") or "g++"
    for name, src in progs.items():
        cmd = [cxx, "-O1", "-g", "-std=c++17", "-pthread", *flag.split(","), "-fno-omit-frame-pointer", "-o", os.path.join(out, name),
               src, "-L" + out, "-lbnkgpu", "-Wl,-rpath,$ORIGIN"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("g++ (sanitized) failed:\n" + res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
