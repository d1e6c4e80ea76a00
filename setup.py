"""Packaging: builds the sm_100a extension in-tree (``deepep_efa_b200/_build/_dx.so``) and installs the package with it.

    python setup.py build_ext --inplace      # same as: python __graft_entry__.py
    pip install --no-build-isolation .

Unlike the reference's setup.py (setup.py:61-69) nothing outside CUDA and PyTorch is linked: no libfabric, no GDRCopy.
"""
import os
import sys

import setuptools
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _build_native():
    from deepep_efa_b200 import _ext
    _ext.build(verbose=True)


class build_ext(_build_ext):
    def run(self):
        _build_native()


class build_py(_build_py):
    def run(self):
        _build_native()
        super().run()


if __name__ == "__main__":
    setuptools.setup(
        name="deepep_efa_b200",
        version="0.1.0",
        description="Blackwell-native MoE expert-parallel communication (deep_ep.Buffer API) for one NVSwitch domain",
        packages=setuptools.find_packages(include=["deepep_efa_b200", "deepep_efa_b200.*"]),
        package_data={"deepep_efa_b200": ["_build/_dx.so", "_build/_dx.hash", "csrc/host/*", "csrc/kernels/*"]},
        python_requires=">=3.10",
        install_requires=["torch"],
        cmdclass={"build_ext": build_ext, "build_py": build_py},
    )
