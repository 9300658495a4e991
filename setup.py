"""Build and install medvision_b200: one CUDA library (libmvr.so) for sm_100a, the Python package
around it, and the C header of its ABI.

Counterpart of the reference's setup.py (one CUDAExtension over every .cu of the package, flags
from $NVCC_FLAGS, links curand: setup.py:33-71) cut down to the resampling path: nvcc is called
directly with `-gencode arch=compute_100a,code=sm_100a` and nothing else -- no other
architecture, no Triton, no CPU implementation, no curand, no torch headers (the library's
interface is plain C; torch is only a run-time dependency of the Python wrappers).

    pip install --no-build-isolation -e .      # or: python setup.py build_py
"""
import os
import shutil
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _compile_library():
    sys.path.insert(0, ROOT)
    try:
        from medvision_b200 import build as lib_build  # imports nothing but the standard library
    finally:
        sys.path.pop(0)
    return lib_build.build()


class BuildWithLibrary(build_py):
    """Compiles libmvr.so in-tree (where an editable install and the tests look for it), then lets
    the normal build_py copy the package; the library and the header travel as package data."""

    def run(self):
        lib = _compile_library()
        header_copy = os.path.join(ROOT, "medvision_b200", "include", "mvr.h")
        os.makedirs(os.path.dirname(header_copy), exist_ok=True)
        shutil.copyfile(os.path.join(ROOT, "include", "mvr.h"), header_copy)
        super().run()
        if not getattr(self, "editable_mode", False):
            target = os.path.join(self.build_lib, "medvision_b200")
            os.makedirs(target, exist_ok=True)
            shutil.copyfile(lib, os.path.join(target, os.path.basename(lib)))


setup(
    name="medvision-b200",
    version="0.2.0",
    description="RoI Align / RoI Align Rotated / affine resampling of MedVision for NVIDIA B200 (sm_100a only)",
    packages=find_packages(include=["medvision_b200", "medvision_b200.*"]),
    package_data={"medvision_b200": ["libmvr.so", "include/mvr.h", "csrc/*.cu", "csrc/*.cuh"]},
    python_requires=">=3.9",
    install_requires=["torch", "numpy"],
    cmdclass={"build_py": BuildWithLibrary},
    zip_safe=False,
)
