"""Builds the cubins (nvcc, sm_100a), the native library and the `kern` binary in-tree before packaging, so a wheel
carries them (`pip wheel . --no-build-isolation`); the sources stay importable from a checkout without installing."""
from setuptools import setup
from setuptools.dist import Distribution
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        import os
        import sys

        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from kern_b200 import _build

        _build.build_all()
        super().run()


class Binary(Distribution):
    """The wheel carries native files (the extension module, two binaries, cubins): it is tagged for this platform and
    interpreter, not `py3-none-any`."""

    def has_ext_modules(self):
        return True


setup(cmdclass={"build_py": BuildNative}, distclass=Binary)
