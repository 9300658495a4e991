"""Compile the CUDA library in-tree for sm_100a:  python -m medvision_b200.build"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmvr.so")
SOURCES = ["mvr_api.cu"]
HEADERS = ["mvr_arith.cuh", "mvr_geom.cuh", "mvr_generic.cuh", "mvr_stream3d.cuh", "mvr_tma3d.cuh", "mvr_bwd3d.cuh", "mvr_offset.cuh", "mvr_cubic3d.cuh", "mvr_flat.cuh", "mvr_label.cuh", "mvr_plane2d.cuh",
           os.path.join("..", "..", "include", "mvr.h")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """nvcc cross-compiles without a GPU; the .so stays beside the package."""
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
