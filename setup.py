"""Builds the native core (C++ and CUDA for sm_100a, `falcata_b200/build.py`) before the Python files are collected,
so that an installed or wheel-packaged copy carries `falcata_b200/lib/libfalcata_core.so` and the CLI binary.

    python -m pip install --no-build-isolation .        # compiles with nvcc (cross-compiles without a GPU)
    python setup.py build_native                        # just the native build, in place
"""
import sys
from pathlib import Path

from setuptools import Command, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


def _build_native() -> None:
    sys.path.insert(0, str(ROOT))
    from falcata_b200 import build as native

    native.build(verbose=True)
    native._build_cli()


class BuildNative(Command):
    description = "compile libfalcata_core.so and the command line tool in the source tree"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


class BuildPyWithNative(build_py):
    def run(self):
        _build_native()
        super().run()


setup(cmdclass={"build_native": BuildNative, "build_py": BuildPyWithNative})
