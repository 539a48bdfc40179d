"""Run-time kernel compilation helpers for tests and user kernels: `KernelBuilder`, `Kernel`, `pack`,
`get_device_arch`, dtype conversion (reference: python/mscclpp/utils.py:35-200)."""
from __future__ import annotations

import ctypes
import os
import struct
import subprocess
import tempfile
from typing import Any, Optional

import numpy as np

from .._core import native as _loader

__all__ = ["Kernel", "KernelBuilder", "pack", "get_device_arch", "torch_dtype_to_mscclpp_dtype", "is_torch_tensor"]


def get_device_arch() -> str:
    return "sm_100a"


def is_torch_tensor(tensor: Any) -> bool:
    try:
        import torch
    except ImportError:
        return False
    return isinstance(tensor, torch.Tensor)


def torch_dtype_to_mscclpp_dtype(dtype):
    from .._core.symm import torch_dtype_to_native

    return torch_dtype_to_native(dtype)


class Kernel:
    """One `__global__` function of a loaded cubin."""

    def __init__(self, cubin: bytes, kernel_name: str):
        n = _loader.load()
        self._module = n.CudaModule(cubin)
        self._function = self._module.function(kernel_name)

    def launch_kernel(self, params: bytes, nblocks: int, nthreads: int, shared: int = 0, stream=None, grid_y: int = 1,
                      cooperative: bool = False, offsets=()):
        """`params` is the packed parameter block (see `pack`). A cooperative launch also needs the byte offset of
        every parameter inside it."""
        cuda_stream = 0
        if stream is not None:
            if hasattr(stream, "cuda_stream"):  # torch.cuda.Stream (0 = the default stream)
                cuda_stream = int(stream.cuda_stream)
            elif hasattr(stream, "ptr"):  # cupy stream
                cuda_stream = int(stream.ptr)
            else:
                cuda_stream = int(stream)
        _loader.load().launch_packed(self._function, bytes(params), nblocks, grid_y, nthreads, shared, cuda_stream, cooperative,
                                     list(offsets))


class KernelBuilder:
    """Compile one kernel of a .cu file to a cubin for sm_100a with this library's headers on the include path."""

    kernel_map: dict = {}   # (source, macros, kernel name) -> Kernel
    cubin_map: dict = {}    # (source, macros) -> cubin bytes: several kernels of one file share one compilation

    @staticmethod
    def get_key(file, kernel_name, macro_dict):
        return f"{file}:{kernel_name}:" + "-".join(f"{k}={macro_dict[k]}" for k in sorted(macro_dict))

    def __init__(self, file: str, kernel_name: str, file_dir: Optional[str] = None, macro_dict: Optional[dict] = None, load: bool = True):
        macro_dict = macro_dict or {}
        self._dir = file_dir if file_dir else os.getcwd()
        self._source = os.path.join(self._dir, file)
        cubin_key = self.get_key(self._source, "", macro_dict)
        if cubin_key not in self.cubin_map:
            self.cubin_map[cubin_key] = self._compile_cuda(self._source, [f"-D{k}={v}" for k, v in macro_dict.items()])
        self.cubin = self.cubin_map[cubin_key]
        self._kernel = None
        if load:
            key = self.get_key(self._source, kernel_name, macro_dict)
            if key not in self.kernel_map:
                self.kernel_map[key] = Kernel(self.cubin, kernel_name)
            self._kernel = self.kernel_map[key]

    @staticmethod
    def _compile_cuda(source_file: str, macros, std_version: str = "c++17") -> bytes:
        from .. import get_include

        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        nvcc = os.path.join(cuda_home, "bin", "nvcc")
        nvcc = nvcc if os.path.exists(nvcc) else "nvcc"
        with tempfile.TemporaryDirectory() as tmp:
            out = os.path.join(tmp, "kernel.cubin")
            cmd = [nvcc, f"-std={std_version}", "-cubin", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
                   f"-I{get_include()}", source_file, "-o", out] + list(macros)
            try:
                subprocess.run(cmd, capture_output=True, text=True, check=True, stdin=subprocess.DEVNULL)
            except subprocess.CalledProcessError as e:
                raise RuntimeError("Compilation failed: " + " ".join(cmd) + "\n" + e.stderr) from e
            with open(out, "rb") as f:
                return f.read()

    def get_compiled_kernel(self) -> Kernel:
        if self._kernel is None:
            raise RuntimeError("the kernel was compiled with load=False")
        return self._kernel


def pack(*args) -> bytes:
    """Concatenate launch arguments into one parameter block. The caller orders and pads them like the kernel's
    parameter list (ints are 4 bytes, pointers and size_t 8 bytes, bytes are copied as they are)."""
    res = b""
    for arg in args:
        if isinstance(arg, bool):
            res += struct.pack("i", int(arg))
        elif isinstance(arg, int):
            res += struct.pack("i", arg)
        elif isinstance(arg, ctypes.c_size_t):
            res += struct.pack("N", arg.value)
        elif isinstance(arg, ctypes.c_void_p):
            res += struct.pack("P", arg.value or 0)
        elif isinstance(arg, float):
            res += struct.pack("f", arg)
        elif isinstance(arg, np.ndarray):
            res += struct.pack("P", arg.ctypes.data)
        elif is_torch_tensor(arg):
            res += struct.pack("P", arg.data_ptr())
        elif hasattr(arg, "__cuda_array_interface__"):
            res += struct.pack("P", arg.__cuda_array_interface__["data"][0])
        elif isinstance(arg, (bytes, bytearray)):
            res += bytes(arg)
        else:
            raise RuntimeError(f"Unsupported type: {type(arg)}")
    return res
