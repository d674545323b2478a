"""Builds the CUDA extension in-tree (nvcc, sm_100a) before the Python package is collected.

The kernels are plain ``extern "C"`` launchers bound through ctypes, so no torch headers are compiled and
no ``torch.utils.cpp_extension`` machinery is needed: ``tokenweave_b200/build.py`` drives nvcc directly.
"""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        import importlib.util
        import pathlib
        spec = importlib.util.spec_from_file_location(
            "tw_build", pathlib.Path(__file__).parent / "tokenweave_b200" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
