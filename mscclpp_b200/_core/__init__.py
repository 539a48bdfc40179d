from .algorithm import Algorithm, AlgorithmBuilder, AlgorithmCollection, get_flag_buffer  # noqa: F401
from .buffer import GpuBuffer  # noqa: F401
from .comm import CommGroup  # noqa: F401
from .compiler import DslCompiler, NativeCodeCompiler  # noqa: F401

__all__ = ["Algorithm", "AlgorithmBuilder", "AlgorithmCollection", "get_flag_buffer", "GpuBuffer", "CommGroup", "DslCompiler",
           "NativeCodeCompiler"]
