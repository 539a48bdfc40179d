"""Builds the native libraries in-tree (nvcc for sm_100a + g++) before packaging; `pip install .`, `pip wheel .` and
`python setup.py build_ext --inplace` all end with mscclpp_b200/lib/*.so in place."""
import importlib.util
import os

from setuptools import Distribution, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    # by path: a PEP 517 build runs without the source directory on sys.path, and the package itself needs torch
    spec = importlib.util.spec_from_file_location("_mscclpp_b200_build", os.path.join(HERE, "mscclpp_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildNativeFirst(build_py):
    def run(self):
        _load_builder().build(verbose=True)
        super().run()


class BinaryDistribution(Distribution):
    """The wheel carries compiled libraries: it gets a platform tag, not `py3-none-any`."""

    def has_ext_modules(self):
        return True


setup(cmdclass={"build_py": BuildNativeFirst}, distclass=BinaryDistribution)
