"""Builds the native libraries in-tree (nvcc for sm_100a + g++) before packaging; `pip install .` and
`python setup.py build_ext --inplace` both end with mscclpp_b200/lib/*.so in place."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNativeFirst(build_py):
    def run(self):
        from mscclpp_b200 import _build

        _build.build(verbose=True)
        super().run()


setup(cmdclass={"build_py": BuildNativeFirst})
