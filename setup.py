"""Builds the cubins (nvcc, sm_100a), the native library and the `kern` binary in-tree before packaging, so a wheel
carries them (`pip wheel . --no-build-isolation`); the sources stay importable from a checkout without installing."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        import os
        import sys

        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from kern_b200 import _build

        _build.build_all()
        super().run()


setup(cmdclass={"build_py": BuildNative})
