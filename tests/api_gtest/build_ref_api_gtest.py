"""Compiles the reference's own API tests of the hot path, from where they lie in the
reference tree, against THIS library's headers and shared library, into
tests/api_gtest/_build/ref_api_gtest (git-ignored).

    python tests/api_gtest/build_ref_api_gtest.py [/path/to/reference]

Nothing is copied out of the reference: its six test sources
(test/mlu_op_gtest/api_gtest/src/gtest/{get_indice_pairs,indice_convolution_forward}/*.cpp),
its api_test_tools.h and its vendored googletest are read in place.  What they include
resolves as follows:
  mlu_op.h, cnrt.h, cn_api.h          -> include/ of this repository
  core/context.h, core/tensor.h,
  core/logging.h                      -> mlu-ops_b200/csrc/core/ (same names, same fields the tests
                                         read: handle->queue, handle->arch)
  tools.h                             -> tests/api_gtest/shim/tools.h (the check macros and the vendor
                                         runtime calls cnrtMalloc / cnrtFree / cnrtQueueSync)
The tests only check status codes, so the binary runs with or without a GPU
(MLUOP_B200_HOST_ONLY_HANDLE=1 gives it a handle without one).
When the reference tree is absent the script does nothing and returns None.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT_DIR = os.path.join(HERE, "_build")
EXE = os.path.join(OUT_DIR, "ref_api_gtest")
OPERATORS = ("get_indice_pairs", "indice_convolution_forward")


def build(reference="/root/reference", force=False):
    gtest_root = os.path.join(reference, "test", "mlu_op_gtest")
    api_src = os.path.join(gtest_root, "api_gtest", "src", "gtest")
    if not os.path.isdir(api_src):
        return EXE if os.path.isfile(EXE) else None
    sources = []
    for op in OPERATORS:
        sources += sorted(glob.glob(os.path.join(api_src, op, "*.cpp")))
    assert len(sources) == 6, sources
    googletest = os.path.join(gtest_root, "googletest")
    gtest_sources = [os.path.join(googletest, "src", n) for n in
                     ("gtest.cc", "gtest-death-test.cc", "gtest-filepath.cc", "gtest-port.cc", "gtest-printers.cc",
                      "gtest-test-part.cc", "gtest-typed-test.cc")]
    csrc = os.path.join(ROOT, "mlu-ops_b200", "csrc")
    lib_dir = os.path.join(ROOT, "mlu-ops_b200", "lib")
    own = [os.path.join(HERE, "main.cpp"), os.path.join(csrc, "core", "logging.cpp"), os.path.join(csrc, "core", "type.cpp")]
    deps = sources + gtest_sources + own + [os.path.join(HERE, "shim", "tools.h"), os.path.join(ROOT, "include", "mlu_op.h"),
                                            os.path.join(lib_dir, "libmluops_b200.so")]
    if not force and os.path.isfile(EXE) and all(os.path.getmtime(p) <= os.path.getmtime(EXE) for p in deps):
        return EXE
    os.makedirs(OUT_DIR, exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", "-w", "-o", EXE,
           "-I", os.path.join(HERE, "shim"), "-I", os.path.join(gtest_root, "api_gtest", "include"),
           "-I", os.path.join(ROOT, "include"), "-I", csrc, "-I", os.path.join(googletest, "include"),
           "-I", googletest, "-I", os.path.join(cuda, "include"), "-DMLUOP_B200_HAVE_CUDA_RUNTIME",
           "-DMLUOP_WIN_API="] + sources + gtest_sources + own + [
           "-L", lib_dir, "-lmluops_b200", "-Wl,-rpath," + lib_dir,
           "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-lpthread"]
    subprocess.check_call(cmd)
    return EXE


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), force=True))
