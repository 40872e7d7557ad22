"""Installs ``eccv26_tad_b200`` (with ``libsvtad.so`` built for sm_100a) and a top-level ``opentad_sparse_ops`` module.

The reference's ``setup.py`` (:21-34) builds a ``CUDAExtension(name="opentad_sparse_ops")`` so that
``opentad/models/bricks/sparse_conv_layer.py:12-13`` can ``import opentad_sparse_ops``.  After

    pip install --no-build-isolation .

the same import resolves to this package's five callables on top of ``libsvtad.so`` - no ``install()`` call, no JIT
build of the reference's CUDA sources.  The library is compiled by ``eccv26_tad_b200/build.py`` (plain nvcc, no torch
extension machinery) during ``build_py``.
"""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithLibrary(build_py):
    def run(self):
        sys.path.insert(0, ROOT)
        from eccv26_tad_b200.build import build_library
        build_library()
        super().run()


setup(
    name="eccv26_tad_b200",
    version="0.2.0",
    description="B200-native SparseConv2D (SV-TAD): neighbor tables, sparse forward / backward, drop-in opentad_sparse_ops",
    packages=["eccv26_tad_b200"],
    py_modules=["opentad_sparse_ops"],
    package_data={"eccv26_tad_b200": ["libsvtad.so"]},
    include_package_data=True,
    cmdclass={"build_py": BuildWithLibrary},
    python_requires=">=3.9",
)
