"""Builds libmluops_b200.so: the C-ABI library with the sm_100a kernels.

One nvcc invocation over the C++ host sources and the CUDA kernels; the output
is placed next to this file under lib/ (git-ignored, shipped as a built
artefact).  nvcc cross-compiles, so no GPU is needed to build.

Usage: python mlu-ops_b200/build.py [--force] [--verbose]
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libmluops_b200.so")


def sources():
    out = []
    for pattern in ("core/*.cpp", "kernels/sparse_conv/*.cpp", "kernels/sparse_conv/*.cu",
                    "kernels/voxelization/*.cpp", "kernels/voxelization/*.cu",
                    "kernels/dynamic_point_to_voxel/*.cpp", "kernels/dynamic_point_to_voxel/*.cu"):
        out += sorted(glob.glob(os.path.join(CSRC, pattern)))
    return out


def headers():
    out = glob.glob(os.path.join(ROOT, "include", "*.h"))
    for pattern in ("core/*.h", "kernels/sparse_conv/*.h", "kernels/sparse_conv/*.cuh", "kernels/voxelization/*.h",
                    "kernels/dynamic_point_to_voxel/*.h"):
        out += glob.glob(os.path.join(CSRC, pattern))
    return out


def up_to_date():
    if not os.path.isfile(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(p) <= t for p in sources() + headers())


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [
        nvcc, "-shared", "-o", LIB, "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
        "-DMLUOP_WIN_API=__attribute__((visibility(\"default\")))",
        "-x", "cu",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("MLUOP_B200_NVCC_FLAGS", "").split()  # extra compiler flags (experiments)
    cmd += sources()
    cmd += ["-lcudart_static", "-lpthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
