"""Python face of the symmetric heap: torch tensors that live in peer-mapped (and multicast-bound)
memory, plus process-group style construction.

``SymmetricMemory`` owns one native ``SymmetricHeap``. ``tensor()`` carves a torch tensor out of it;
as long as every rank performs the same sequence of ``tensor()`` / ``release()`` calls the tensors
sit at identical offsets on all ranks, which is what the zero-copy kernels rely on.
"""
from __future__ import annotations

import atexit
import math
import os
import weakref
from typing import Optional, Sequence

import torch

from . import native

_DTYPE_MAP = None


def torch_dtype_to_native(dtype: torch.dtype):
    """torch dtype -> native DataType (same role as the reference's torch_dtype_to_mscclpp_dtype,
    python/mscclpp/utils.py:184-206)."""
    global _DTYPE_MAP
    n = native.load()
    if _DTYPE_MAP is None:
        _DTYPE_MAP = {
            torch.float16: n.DataType.float16,
            torch.bfloat16: n.DataType.bfloat16,
            torch.float32: n.DataType.float32,
            torch.int32: n.DataType.int32,
            torch.uint8: n.DataType.uint8,
            torch.float8_e4m3fn: n.DataType.float8_e4m3,
            torch.float8_e5m2: n.DataType.float8_e5m2,
        }
        if hasattr(torch, "uint32"):
            _DTYPE_MAP[torch.uint32] = n.DataType.uint32
    if dtype not in _DTYPE_MAP:
        raise ValueError(f"unsupported dtype {dtype}")
    return _DTYPE_MAP[dtype]


_TYPESTR = {
    torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int8: "|i1",
    torch.int64: "<i8", torch.float64: "<f8", torch.int16: "<i2",
}


class _RawCudaBuffer:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap foreign device memory."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }
        self._owner = owner  # keeps the heap alive while the tensor exists


def tensor_from_pointer(ptr: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device, owner=None) -> torch.Tensor:
    nbytes = int(math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_RawCudaBuffer(ptr, max(nbytes, 1), owner), device=device)
    return raw[:nbytes].view(dtype).view(*shape)


_live_heaps: "weakref.WeakSet[SymmetricMemory]" = weakref.WeakSet()


def _destroy_all():
    for h in list(_live_heaps):
        try:
            h.destroy()
        except Exception:
            pass


atexit.register(_destroy_all)


class SymmetricMemory:
    def __init__(self, heap, device: torch.device, bootstrap=None):
        self.heap = heap
        self.device = device
        self.bootstrap = bootstrap
        self._allocs = {}
        _live_heaps.add(self)

    # ------------------------------------------------------------------ construction
    @classmethod
    def emulated(cls, world: int, nbytes: int = 256 << 20, ll_slot_bytes: int = 0, timeout_ms: int = 2000,
                 device: Optional[torch.device] = None) -> "SymmetricMemory":
        """`world` heaps on one GPU; collective kernels run all ranks in one cooperative launch."""
        n = native.load()
        device = device or torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(device):
            heap = n.SymmetricHeap.create_emulated(world, nbytes, ll_slot_bytes, timeout_ms)
        return cls(heap, device)

    @classmethod
    def from_env(cls, nbytes: int = 0, enable_nvls: bool = True, ll_slot_bytes: int = 0, timeout_ms: int = -1,
                 port_offset: int = 1) -> "SymmetricMemory":
        """One rank per process, rank/world/rendezvous taken from the torchrun environment."""
        n = native.load()
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        bootstrap = n.TcpBootstrap(rank, world)
        bootstrap.initialize(f"{addr}:{port}", 120)
        heap = n.SymmetricHeap.create(bootstrap, nbytes, ll_slot_bytes, enable_nvls, timeout_ms)
        return cls(heap, device, bootstrap)

    @classmethod
    def from_bootstrap(cls, bootstrap, device: torch.device, nbytes: int = 0, enable_nvls: bool = True,
                       ll_slot_bytes: int = 0, timeout_ms: int = -1) -> "SymmetricMemory":
        n = native.load()
        torch.cuda.set_device(device)
        heap = n.SymmetricHeap.create(bootstrap, nbytes, ll_slot_bytes, enable_nvls, timeout_ms)
        return cls(heap, device, bootstrap)

    # ------------------------------------------------------------------ properties
    @property
    def rank(self) -> int:
        return self.heap.rank

    @property
    def world(self) -> int:
        return self.heap.world

    @property
    def emulated_mode(self) -> bool:
        return self.heap.emulated

    @property
    def nvls(self) -> bool:
        return self.heap.nvls

    # ------------------------------------------------------------------ tensors
    def tensor(self, shape: Sequence[int], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        nbytes = int(math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        ptr = self.heap.alloc(max(nbytes, 16), 256)
        t = tensor_from_pointer(ptr, shape, dtype, self.device, owner=self)
        self._allocs[t.data_ptr()] = ptr
        if zero:
            if self.emulated_mode:
                for r in range(self.world):
                    self.rank_view(t, r).zero_()
            else:
                t.zero_()
        return t

    def release(self, t: torch.Tensor) -> None:
        ptr = self._allocs.pop(t.data_ptr())
        self.heap.free(ptr)

    def rank_view(self, t: torch.Tensor, r: int) -> torch.Tensor:
        """The tensor at the same heap offset in rank r's heap (peer-mapped memory; in emulated mode
        simply the emulated rank's copy)."""
        off = t.data_ptr() - self.heap.local_base
        return tensor_from_pointer(self.heap.peer_base(r) + off, tuple(t.shape), t.dtype, self.device, owner=self)

    def contains(self, t: torch.Tensor) -> bool:
        return self.heap.contains(t.data_ptr(), max(t.numel() * t.element_size(), 1))

    def barrier(self) -> None:
        """Host-side barrier over the ranks of the heap, after this rank's GPU work has finished. Needed after
        initialising symmetric memory that peers write into (a late zero-fill would wipe what an early peer wrote)."""
        torch.cuda.synchronize(self.device)
        if not self.emulated_mode and self.bootstrap is not None and self.world > 1:
            self.bootstrap.barrier()

    # ------------------------------------------------------------------ health
    def check(self) -> None:
        """Raise if a device-side wait of an earlier launch gave up (call after a synchronize)."""
        self.heap.check_status()

    def destroy(self) -> None:
        if self.heap is not None:
            torch.cuda.synchronize(self.device)
            self.heap.destroy()
            self.heap = None
