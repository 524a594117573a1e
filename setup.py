"""Build hook: compiles the CUDA kernels into sklearn_numba_dpex_b200/libkmb200.so (nvcc,
sm_100a) before the package files are collected, so that `pip install .` and
`pip install -e . --no-build-isolation` both ship the library the package cannot work without.
All metadata lives in pyproject.toml."""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_library():
    # the package itself cannot be imported before its library exists: load build.py by path
    spec = importlib.util.spec_from_file_location(
        "_kmb_build", os.path.join(HERE, "sklearn_numba_dpex_b200", "build.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module.build()


class BuildPyWithKernels(build_py):
    def run(self):
        _build_library()
        super().run()


setup(cmdclass={"build_py": BuildPyWithKernels})
