"""Build contract: `pip install -e .` (or `pip install .`) compiles the one sm_100a
library with nvcc (elman_b200/build.py) and installs the package together with the
top-level `hasty_pytorch_lib` module, the name the reference's model files import.
The reference's own contract is `cd elman/cuda && make hasty && pip install -e .`
(README.md:50-51 of the reference)."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

HERE = os.path.dirname(os.path.abspath(__file__))


def _compile_cuda_library():
    sys.path.insert(0, HERE)
    try:
        from elman_b200 import build as nvcc_build
        nvcc_build.build(force=False)
    finally:
        sys.path.pop(0)


class BuildPyWithCuda(build_py):
    def run(self):
        _compile_cuda_library()
        super().run()


class DevelopWithCuda(develop):
    def run(self):
        _compile_cuda_library()
        super().run()


setup(cmdclass={"build_py": BuildPyWithCuda, "develop": DevelopWithCuda})
