"""Python face of the algorithm framework: `Algorithm`, `AlgorithmBuilder`, `AlgorithmCollection`,
`get_flag_buffer` (reference: python/mscclpp/_core/algorithm.py:28-281)."""
from __future__ import annotations

from functools import cached_property
from typing import Callable, Dict, Optional, Tuple

from . import native as _loader

__all__ = ["Algorithm", "AlgorithmBuilder", "AlgorithmCollection", "get_flag_buffer"]


def _n():
    return _loader.load()


class Algorithm:
    """A collective algorithm: either an execution plan (DSL) or a native kernel launcher."""

    class Constraint:
        def __init__(self, world_size: int = 0, n_ranks_per_node: int = 0):
            self._constraint = _n().Algorithm.Constraint(world_size, n_ranks_per_node)

        @property
        def world_size(self) -> int:
            return self._constraint.world_size

        @property
        def n_ranks_per_node(self) -> int:
            return self._constraint.n_ranks_per_node

    def __init__(self, id: Optional[str] = None, execution_plan=None, native_handle=None, tags: Optional[Dict[str, int]] = None,
                 constraint: Optional["Algorithm.Constraint"] = None):
        if execution_plan is not None:
            self._algorithm = _n().DslAlgorithm(
                id or execution_plan.name, execution_plan, tags=tags or {},
                constraint=constraint._constraint if constraint is not None else _n().Algorithm.Constraint())
        elif native_handle is not None:
            self._algorithm = native_handle
        else:
            raise ValueError("give an execution plan or a native handle")

    @classmethod
    def create_from_native_handle(cls, handle) -> "Algorithm":
        return cls(native_handle=handle)

    @classmethod
    def create_from_native_capsule(cls, obj) -> "Algorithm":
        return cls(native_handle=_n().Algorithm.from_native_capsule(obj))

    @classmethod
    def from_callable(cls, name: str, collective: str, kernel: Callable, init: Optional[Callable] = None,
                      min_message_size: int = 0, max_message_size: int = 2**64 - 1, buffer_mode=None,
                      tags: Optional[Dict[str, int]] = None, constraint: Optional["Algorithm.Constraint"] = None) -> "Algorithm":
        """Native algorithm whose launch function is a Python callable
        ``kernel(input_ptr, output_ptr, input_bytes, output_bytes, dtype, op, stream, n_blocks, n_threads, symmetric, extras)``."""
        n = _n()
        handle = n.NativeAlgorithm(name, collective, init, kernel, min_message_size, max_message_size,
                                   buffer_mode if buffer_mode is not None else n.CollectiveBufferMode.ANY, tags or {},
                                   constraint._constraint if constraint is not None else n.Algorithm.Constraint())
        return cls(native_handle=handle)

    @cached_property
    def name(self) -> str:
        return self._algorithm.name

    @cached_property
    def collective(self) -> str:
        return self._algorithm.collective

    @property
    def message_size_range(self) -> Tuple[int, int]:
        return tuple(self._algorithm.message_range)

    def set_message_size_range(self, min_message_size: int, max_message_size: int):
        self._algorithm.set_message_size_range(min_message_size, max_message_size)

    @cached_property
    def tags(self) -> Dict[str, int]:
        return dict(self._algorithm.tags)

    @cached_property
    def buffer_mode(self):
        return self._algorithm.buffer_mode

    def is_dsl_algorithm(self) -> bool:
        return self._algorithm.type == _n().AlgorithmType.DSL

    def is_native_algorithm(self) -> bool:
        return self._algorithm.type == _n().AlgorithmType.NATIVE

    def execute(self, comm, input_buffer: int, output_buffer: int, input_size: int, output_size: int, dtype, op=None, stream: int = 0,
                executor=None, nblocks: int = 0, nthreads_per_block: int = 0, symmetric_memory: bool = False,
                extras: Optional[Dict[str, int]] = None, accum_dtype=None) -> int:
        """Run the collective on `stream`; returns 0 on success (the numeric value of `CommResult`)."""
        n = _n()
        return self._algorithm.execute(comm, int(input_buffer), int(output_buffer), input_size, output_size, dtype,
                                       op if op is not None else n.ReduceOp.NOP, int(stream), executor, nblocks, nthreads_per_block,
                                       symmetric_memory, dict(extras) if extras else {},
                                       accum_dtype if accum_dtype is not None else n.DataType.auto)

    def reset(self):
        self._algorithm.reset()


class AlgorithmBuilder:
    def __init__(self, algorithm_builder):
        self._algorithm_builder = algorithm_builder

    def build(self) -> Algorithm:
        return Algorithm.create_from_native_handle(self._algorithm_builder.build())


class AlgorithmCollection:
    def __init__(self, native_collection=None):
        self._native_collection = native_collection if native_collection is not None else _n().AlgorithmCollection()
        self._refresh()

    def _refresh(self):
        self._algorithms = [Algorithm.create_from_native_handle(a) for a in self._native_collection.get_all_algorithms()]

    def __iter__(self):
        return iter(self._algorithms)

    def __len__(self):
        return len(self._algorithms)

    def __getitem__(self, index: int) -> Algorithm:
        return self._algorithms[index]

    def get_by_collective(self, collective: str):
        return [a for a in self._algorithms if a.collective == collective]

    def get_by_name(self, name: str) -> Optional[Algorithm]:
        for a in self._algorithms:
            if a.name == name:
                return a
        return None

    def register_algorithm(self, collective: str, algo_name: str, algorithm: Algorithm):
        self._native_collection.register_algorithm(collective, algo_name, algorithm._algorithm)
        self._refresh()

    def select(self, request) -> Optional[Algorithm]:
        """Run the selectors on a `CollectiveRequest`; None when nothing fits."""
        h = self._native_collection.select_algorithm(request)
        return Algorithm.create_from_native_handle(h) if h is not None else None


def get_flag_buffer():
    """The process-wide flag buffer (128 x uint32, initialised to 1) as a torch uint8 view plus its size in bytes."""
    ptr, nbytes = _n().get_flag_buffer()
    return ptr, nbytes
