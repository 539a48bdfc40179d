"""mscclpp_b200: a Blackwell-native (sm_100a) GPU-driven communication stack with the capabilities,
public API and execution-plan format of MSCCL++, written from scratch around a symmetric
NVSwitch heap, with collectives fused into the compute that produces or consumes them."""
import os as _os

__version__ = "0.9.0+b200.1"
version = {"version": __version__, "git_commit": "unknown"}

from ._core import native as _native_loader  # noqa: E402
from ._core.symm import SymmetricMemory, tensor_from_pointer, torch_dtype_to_native  # noqa: E402,F401
from ._core.algorithm import Algorithm, AlgorithmBuilder, AlgorithmCollection, get_flag_buffer  # noqa: E402,F401
from ._core.buffer import GpuBuffer  # noqa: E402,F401
from ._core.comm import CommGroup  # noqa: E402,F401
from ._core.compiler import DslCompiler, NativeCodeCompiler  # noqa: E402,F401

if _os.environ.get("MSCCLPP_HOME") is None:
    _os.environ["MSCCLPP_HOME"] = _os.path.abspath(_os.path.dirname(__file__))

# Names that live in the compiled runtime; resolved on first access so that the pure-Python parts (the DSL,
# the plan interpreter) import on a machine where the runtime has not been built.
_NATIVE_NAMES = (
    "Device", "DeviceType", "Communicator", "Connection", "connect_nvls_collective", "EndpointConfig", "EndpointConfigIb",
    "IbMode", "ErrorCode", "Fifo", "Semaphore", "Host2DeviceSemaphore", "Host2HostSemaphore", "ProxyService", "RegisteredMemory",
    "PortChannel", "MemoryChannel", "MemoryDevice2DeviceSemaphore", "TcpBootstrap", "Transport", "TransportFlags", "DataType",
    "Executor", "ExecutionPlan", "PacketType", "RawGpuBuffer", "ReduceOp", "env", "is_bulk_supported", "is_nvls_supported",
    "SwitchChannel", "NvlsConnection", "BaseMemoryChannel", "BasePortChannel", "Context", "Endpoint", "Bootstrap", "SymmetricHeap",
    "CollectiveRequest", "CollectiveBufferMode", "AlgorithmType", "CommResult", "Error", "BaseError", "CudaError", "CuError",
    "SysError", "IbError", "npkit", "numa", "GpuBufferGranularity",
)

__all__ = [
    "SymmetricMemory", "Algorithm", "AlgorithmBuilder", "AlgorithmCollection", "CommGroup", "GpuBuffer", "DslCompiler",
    "NativeCodeCompiler", "compile", "compile_native", "get_flag_buffer", "get_include", "get_lib", "version", "__version__",
    "alloc_shared_physical_cuda", "deprecated", *_NATIVE_NAMES,
]


def native():
    """The compiled runtime module (raises if it has not been built)."""
    return _native_loader.load()


def deprecated(new_cls):
    """Decorator for a kept-for-compatibility name: calling the decorated class or function warns and builds `new_cls`
    instead (same helper as the reference's package: python/mscclpp/__init__.py:119-131)."""
    import functools
    import warnings

    def decorator(old_cls):
        @functools.wraps(old_cls)
        def wrapper(*args, **kwargs):
            warnings.warn(f"{old_cls.__name__} is deprecated, use {new_cls.__name__} instead.", DeprecationWarning, stacklevel=2)
            return new_cls(*args, **kwargs)

        return wrapper

    return decorator


def alloc_shared_physical_cuda(nbytes: int, granularity=None):
    """Zeroed physical (VMM) device memory of at least `nbytes`, shareable with peers and bindable to NVLink multicast.
    Returns the owning `RawGpuBuffer` (`.data()` is the device pointer, `.bytes()` the rounded size); the memory is
    freed when the object is dropped. (The name is exported by the reference's package as well: python/mscclpp/__init__.py:93.)"""
    n = _native_loader.load()
    return n.RawGpuBuffer(int(nbytes)) if granularity is None else n.RawGpuBuffer(int(nbytes), granularity)


def __getattr__(name):
    if name in _NATIVE_NAMES:
        value = getattr(_native_loader.load(), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def get_include() -> str:
    """Directory of the C++ headers (`#include <mscclpp/...>`)."""
    return _os.path.join(_os.path.dirname(__file__), "csrc", "include")


def get_lib() -> str:
    """Directory of the built shared libraries."""
    return _os.path.join(_os.path.dirname(__file__), "lib")


compile = DslCompiler()
compile_native = NativeCodeCompiler()
