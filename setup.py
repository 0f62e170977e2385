"""Build hook: compile the CUDA sources into aitherkvcache_b200/libakv_b200.so (nvcc, sm_100a) before the
package is collected, so that `pip install .` ships the library the Python layer loads with ctypes."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithKernels(build_py):
    def run(self):
        sys.path.insert(0, ROOT)
        from aitherkvcache_b200 import _build
        _build.build()
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
