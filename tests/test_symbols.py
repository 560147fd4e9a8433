"""The C-ABI library loads and exports every function include/mlu_op.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for header in ("mlu_op.h", "mlu_op_trace.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mluOp[A-Za-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_function_is_exported(ops):
    names = declared_functions()
    assert len(names) >= 32
    lib = ctypes.CDLL(ops.LIB_PATH)
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(ops.SIGNATURES), set(names) ^ set(ops.SIGNATURES)


def test_header_compiles_as_plain_c(tmp_path):
    import subprocess
    src = tmp_path / "use.c"
    src.write_text('#include "mlu_op.h"\n#include "mlu_op_trace.h"\nint main(void) { mluOpHandle_t h = 0; (void)h; return MLUOP_STATUS_SUCCESS; }\n')
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c",
                           str(src), "-o", str(tmp_path / "use.o")])


def test_missing_library_fails_loudly(ops, monkeypatch):
    import pytest
    monkeypatch.setattr(ops, "_lib", None)
    monkeypatch.setattr(ops, "LIB_PATH", "/nonexistent/libmluops_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        ops.lib()


def test_public_headers_compile_as_c_and_cxx(tmp_path):
    """include/mlu_op.h and include/mlu_op_trace.h are a C API: they must compile as C11 and as C++17."""
    import shutil
    import subprocess
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if shutil.which("gcc") is None or not os.path.isfile(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("gcc or the CUDA headers are not available")
    src = tmp_path / "uses_headers.c"
    src.write_text('#include "mlu_op.h"\n#include "mlu_op_trace.h"\n'
                   "int main(void) { mluOpHandle_t h = 0; (void)h; return (int)MLUOP_STATUS_SUCCESS; }\n")
    inc = ["-I", os.path.join(ROOT, "include"), "-I", cuda_inc]
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only"] + inc + [str(src)])
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++"] + inc + [str(src)])


def test_cxx_caller_links_and_runs(tmp_path):
    """tests/cabi/abi_check.cpp, a C++ caller in the style of the reference's API tests, builds
    against include/ and the shared library and gets the expected status codes (host-only handle)."""
    import shutil
    import subprocess
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if shutil.which("g++") is None or not os.path.isfile(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("g++ or the CUDA headers are not available")
    lib_dir = os.path.join(ROOT, "mlu-ops_b200", "lib")
    exe = str(tmp_path / "abi_check")
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-o", exe, os.path.join(ROOT, "tests", "cabi", "abi_check.cpp"),
                           "-I", os.path.join(ROOT, "include"), "-I", cuda_inc, "-L", lib_dir, "-lmluops_b200",
                           "-Wl,-rpath," + lib_dir])
    env = dict(os.environ, MLUOP_B200_HOST_ONLY_HANDLE="1", MLUOP_MIN_LOG_LEVEL="3")
    r = subprocess.run([exe], env=env, capture_output=True, text=True)
    assert r.returncode == 0 and "abi_check: ok" in r.stdout, r.stdout + r.stderr
