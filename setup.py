"""Builds libtbik_b200.so (nvcc, sm_100a) before the Python files are collected, so that wheels and editable
installs carry the CUDA library.  All metadata lives in pyproject.toml."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildWithCuda(build_py):
    def run(self):
        from llm_reproducibility_b200 import _build
        _build.build()
        super().run()


setup(cmdclass={"build_py": BuildWithCuda})
