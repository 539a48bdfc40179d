"""Loader of the compiled runtime (``lib/_native*.so``).

The extension is built in-tree by :mod:`mscclpp_b200._build`. Importing it never needs a GPU; calling
into it on a machine with a GPU but without the built library raises immediately instead of
falling back to anything slower.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_native = None


class NativeLibraryMissing(ImportError):
    pass


def lib_dir() -> Path:
    return _LIB_DIR


def load(build_if_missing: bool = False):
    """Return the ``_native`` extension module, importing it on first use."""
    global _native
    if _native is not None:
        return _native
    from .. import _build

    path = _build.native_module_path()
    if not path.exists():
        if not build_if_missing:
            raise NativeLibraryMissing(
                f"{path} is missing: build it with `python -m mscclpp_b200._build` "
                "(there is no pure-Python fallback for the GPU paths)"
            )
        _build.build(verbose=False)
    spec = importlib.util.spec_from_file_location("mscclpp_b200.lib._native", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mscclpp_b200.lib._native"] = mod
    spec.loader.exec_module(mod)
    _native = mod
    return mod


def available() -> bool:
    from .. import _build

    return _build.native_module_path().exists()
