"""Build hook: ``pip install -e .`` (or ``python setup.py build_py``) compiles the native libraries in-tree —
the C++ runtime, the pluggable allocator, the CPU back end and every CUDA kernel for sm_100a — through
``iris_b200._build`` before the Python files are collected.

Role in the reference: ``setup.py:13-84`` (a custom ``build_py`` that runs hipcc on the allocator and ships the
``.so`` as package data)."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from iris_b200 import _build
        libs = _build.build_all(verbose=bool(os.environ.get("IRIS_BUILD_VERBOSE")))
        for name, path in libs.items():
            print(f"built {name}: {path}")
        super().run()


setup(cmdclass={"build_py": BuildNative})
