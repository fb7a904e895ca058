"""Packaging for torchft_b200.  The metadata lives in ``pyproject.toml``; this file only makes the
build run the in-tree native build (``torchft_b200/_build.py``: nvcc for the sm_100a kernel library,
g++ for the control-plane module) before the package files are collected, and marks the wheel as
platform specific.  The reference builds its native half with maturin (pyproject.toml:1-3,46-48);
here there is no separate build system, the package carries its own."""

import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.dist import Distribution


def _native_build_module():
    # loaded by path: importing the package itself would need torch at build time
    path = Path(__file__).resolve().parent / "torchft_b200" / "_build.py"
    spec = importlib.util.spec_from_file_location("_ftb200_build", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class build_py_with_native(build_py):
    def run(self):
        _native_build_module().build_all()
        super().run()


class BinaryDistribution(Distribution):
    def has_ext_modules(self):
        return True


setup(cmdclass={"build_py": build_py_with_native}, distclass=BinaryDistribution)
