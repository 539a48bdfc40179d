"""`GpuBuffer`: a torch tensor over physical (VMM) device memory that can be exported to peers and bound to
NVLink multicast (reference: python/mscclpp/_core/buffer.py:16-37 does the same on a cupy array)."""
from __future__ import annotations

import math
from typing import Sequence, Union

import torch

from . import native as _loader
from .symm import tensor_from_pointer

__all__ = ["GpuBuffer", "GpuBufferGranularity"]


def __getattr__(name):
    if name == "GpuBufferGranularity":  # the native enum, resolved on first use (the library may not be built yet)
        return _loader.load().GpuBufferGranularity
    raise AttributeError(name)


def GpuBuffer(shape: Union[int, Sequence[int]], dtype: torch.dtype = torch.float32, device=None, granularity=None) -> torch.Tensor:
    """Allocate `shape` elements of `dtype` with the multicast granularity and return them as a tensor.
    `granularity`: a `GpuBufferGranularity` (default: the driver's recommended multicast granularity).

    The tensor keeps the allocation alive; `tensor.data_ptr()` is what `Communicator.register_memory` and
    `NvlsConnection.bind_allocated_memory` take."""
    if isinstance(shape, int):
        shape = (shape,)
    shape = tuple(int(s) for s in shape)
    if any(s <= 0 for s in shape):
        raise ValueError("Shape must be positive.")
    nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
    n = _loader.load()
    raw = n.RawGpuBuffer(nbytes) if granularity is None else n.RawGpuBuffer(nbytes, granularity)
    dev = torch.device(device) if device is not None else torch.device("cuda", raw.device_id())
    return tensor_from_pointer(raw.data(), shape, dtype, dev, owner=raw)
