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
    mod.RawGpuBuffer.to_dlpack = _raw_buffer_to_dlpack
    _native = mod
    return mod


def parse_torch_dtype(name: str):
    """'torch.float16' / 'float16' / a torch.dtype -> torch.dtype."""
    import torch

    if isinstance(name, torch.dtype):
        return name
    dtype = getattr(torch, str(name).replace("torch.", ""), None)
    if not isinstance(dtype, torch.dtype):
        raise ValueError(f"unknown data type {name!r}")
    return dtype


def _raw_buffer_to_dlpack(self, data_type, shape=(), strides=()):
    """DLPack capsule over this allocation (reference: python/csrc/gpu_utils_py.cpp:60-111). `data_type` is a torch dtype
    or its name ('torch.float16'); `shape` defaults to all the elements that fit, `strides` (in elements) to contiguous.
    The capsule's tensor keeps the allocation alive."""
    import torch
    from torch.utils.dlpack import to_dlpack

    from .symm import tensor_from_pointer

    dtype = parse_torch_dtype(data_type)
    itemsize = torch.empty((), dtype=dtype).element_size()
    shape = tuple(int(x) for x in shape) or (self.nelems() // itemsize,)
    numel = 1
    for x in shape:
        numel *= x
    if strides:
        span = 1 + sum((n - 1) * int(st) for n, st in zip(shape, strides)) if numel else 0
    else:
        span = numel
    if span * itemsize > self.bytes():
        raise ValueError("shape and strides reach beyond the allocation")
    flat = tensor_from_pointer(self.data(), (max(span, 1),), dtype, torch.device("cuda", self.device_id()), owner=self)
    view = flat[:numel].view(shape) if not strides else flat.as_strided(shape, tuple(int(st) for st in strides))
    return to_dlpack(view)


def available() -> bool:
    from .. import _build

    return _build.native_module_path().exists()
