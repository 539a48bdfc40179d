"""mscclpp_b200: a Blackwell-native (sm_100a) GPU-driven communication stack with the capabilities,
public API and execution-plan format of MSCCL++, written from scratch around a symmetric
NVSwitch heap, with collectives fused into the compute that produces or consumes them."""
from ._core import native as _native_loader
from ._core.symm import SymmetricMemory, tensor_from_pointer, torch_dtype_to_native  # noqa: F401

__version__ = "0.9.0+b200.1"


def native():
    """The compiled runtime module (raises if it has not been built)."""
    return _native_loader.load()
