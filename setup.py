#!/usr/bin/env python3
"""Installer: ``pip install .`` / ``pip install -e .`` (``--no-build-isolation`` so that the installed torch is the
one the extension links against).

The native extension ``planmoe_b200/_C.so`` (every sm_100a kernel, the symmetric-heap runtime, the CPU reference
ops) is built by ``planmoe_b200/utils/build.py`` with ``nvcc -gencode arch=compute_100a,code=sm_100a`` before the
Python files are collected, so wheels and editable installs carry it.  nvcc cross-compiles without a GPU.  Takes the
place of the reference's ``setup.py`` CUDAExtension (setup.py:57-163), which passes no architecture flags and links
libzfp / NCCL; this package needs neither.  Metadata lives in ``pyproject.toml``.
"""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

ROOT = os.path.dirname(os.path.abspath(__file__))


def build_native():
    if os.environ.get('PLANMOE_SKIP_NATIVE_BUILD', '0') == '1':
        return
    sys.path.insert(0, ROOT)
    try:
        from planmoe_b200.utils import build
        print('building', build.build(verbose=os.environ.get('PLANMOE_BUILD_VERBOSE', '0') == '1'))
    finally:
        sys.path.pop(0)


class BuildPy(build_py):
    def run(self):
        build_native()
        super().run()


class Develop(develop):
    def run(self):
        build_native()
        super().run()


setup(cmdclass={'build_py': BuildPy, 'develop': Develop})
