"""The C-ABI library loads without a GPU and exports every symbol include/bnk_gpu.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="bnk_gpu.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bnk_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    from bnk_b200 import _lib

    assert declared_symbols() == sorted(_lib.SYMBOLS)
    assert declared_symbols("bnk_gpu_bench.h") == sorted(_lib.BENCH_SYMBOLS)


def test_bench_library_exports_its_header_and_nothing_of_the_drop_in():
    from bnk_b200 import _build, _lib

    if _build.is_stale():
        _build.build()
    L = ctypes.CDLL(_lib.lib_path())  # the helpers work on the product library's handles
    B = ctypes.CDLL(_build.BENCH_LIB_PATH)
    for name in declared_symbols("bnk_gpu_bench.h"):
        assert hasattr(B, name), name
        assert not hasattr(L, name), f"{name} is a measurement helper and must not be exported by libbnkgpu.so"


def test_library_exports_every_declared_symbol():
    from bnk_b200 import _build, _lib

    if _build.is_stale():
        _build.build()
    L = ctypes.CDLL(_lib.lib_path())
    for name in declared_symbols():
        assert hasattr(L, name), name
    assert _lib.lib().bnk_abi_version() == 1
    assert _lib.lib().bnk_strerror(-4) == b"timed out"


def test_struct_layouts_match_header():
    from bnk_b200 import _lib

    assert ctypes.sizeof(_lib.Cfg) == 32
    assert ctypes.sizeof(_lib.AclTuple) == 12
    assert ctypes.sizeof(_lib.BatchView) == 80
    assert ctypes.sizeof(_lib.BatchStats) == 144
    assert ctypes.sizeof(_lib.TableStats) == 64


def test_no_cpu_fallback_in_product_path():
    """Nothing under bnk_b200/ may import or link the CPU checker."""
    pkg = os.path.join(ROOT, "bnk_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                src = open(os.path.join(dirpath, fn), errors="replace").read()
                assert "oracle" not in src.lower(), os.path.join(dirpath, fn)


def test_header_compiles_as_c_and_the_shim_calls_link(tmp_path):
    """cgo hands include/bnk_gpu.h to a C compiler (not C++): the header must be plain C, and the calls the Go shim
    of INTEGRATION.md makes (tests/c/cgo_shim_calls.c: the same calls with the same argument types) must compile
    without a warning and link against libbnkgpu.so.  Nothing is run: the calls need a GPU."""
    import shutil
    import subprocess

    from bnk_b200 import _build

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    inc = os.path.join(root, "include")
    strict = ["-Wall", "-Wextra", "-Werror", "-pedantic"]
    for std, header in (("c99", "bnk_gpu.h"), ("c11", "bnk_gpu.h"), ("c99", "bnk_gpu_bench.h")):
        res = subprocess.run([gcc, f"-std={std}", *strict, "-I", inc, "-fsyntax-only", "-x", "c", os.path.join(inc, header)],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
    lib = _build.build()
    out = str(tmp_path / "libshim.so")
    res = subprocess.run([gcc, "-std=c11", *strict, "-I", inc, "-shared", "-fPIC", os.path.join(root, "tests", "c", "cgo_shim_calls.c"),
                          "-o", out, "-L", os.path.dirname(lib), "-lbnkgpu", "-Wl,--no-undefined"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
