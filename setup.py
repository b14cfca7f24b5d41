"""Builds the C-ABI CUDA library in-tree:  python setup.py build_ext --inplace

The extension is not a Python C extension: `build_ext` runs nvcc (sm_100a) over
fairseq-apollo_b200/csrc/*.cu and leaves fairseq-apollo_b200/libmega_b200.so, which the package binds with ctypes.
"""
import importlib.util
import os

from setuptools import Command, setup

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildCuda(Command):
    description = "compile libmega_b200.so with nvcc for sm_100a"
    user_options = [("inplace", "i", "ignored: the library is always built in-tree"), ("force", "f", "rebuild")]

    def initialize_options(self):
        self.inplace = 1
        self.force = 0

    def finalize_options(self):
        pass

    def run(self):
        spec = importlib.util.spec_from_file_location("_mega_build", os.path.join(ROOT, "fairseq-apollo_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        print(mod.build(force=bool(self.force)))


setup(
    name="fairseq-apollo-b200",
    version="0.1.0",
    description="Mega EMA layer, TimestepNorm and SequenceNorm on hand-written sm_100a CUDA kernels",
    py_modules=["fairseq_apollo_b200"],
    cmdclass={"build_ext": BuildCuda},
)
