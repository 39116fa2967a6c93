"""Packaging of disagmoe_b200. The native parts are built in-tree by ``disagmoe_b200/build.py`` (nvcc for the sm_100a
kernel library, g++ for the pybind11 runtime); ``python setup.py build_ext --inplace`` and ``pip install -e .`` both
run it, so the built ``.so`` files sit next to the sources they were built from."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.develop import develop as _develop

ROOT = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    sys.path.insert(0, ROOT)
    from disagmoe_b200 import build
    print("built:", build.build_all())


class build_ext(_build_ext):
    def run(self):
        _build_native()


class develop(_develop):
    def run(self):
        _build_native()
        super().run()


class build_native(Command):
    description = "build the sm_100a kernel library and the native runtime in-tree"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


setup(
    name="disagmoe_b200",
    version="0.1.0",
    description="Blackwell-native disaggregated MoE serving engine",
    packages=find_packages(include=["disagmoe_b200", "disagmoe_b200.*", "benchmark", "benchmark.*", "simulator"]),
    package_data={"disagmoe_b200": ["lib/*.so", "*.so", "csrc/kernels/*", "csrc/runtime/*"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy", "pybind11"],
    cmdclass={"build_ext": build_ext, "develop": develop, "build_native": build_native},
)
