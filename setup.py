"""Builds the native library in-tree (nvcc, sm_100a) before the package is collected.

    python setup.py build_ext --inplace      # or: python -m distdl_b200._build
    pip install -e .

The library is plain C ABI loaded with ctypes, so no PyTorch C++ headers are involved;
nvcc cross-compiles without a GPU.  Set DISTDL_SKIP_NATIVE=1 to install the Python parts
only (CPU plumbing and tests still work; CUDA tensors then raise at the first native op).
"""
import os
import sys

from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    if os.environ.get("DISTDL_SKIP_NATIVE", "0") == "1":
        return
    sys.path.insert(0, HERE)
    from distdl_b200 import _build
    _build.build()


class BuildExt(build_ext):
    def run(self):
        _build_native()


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


setup(cmdclass={"build_ext": BuildExt, "build_py": BuildPy})
