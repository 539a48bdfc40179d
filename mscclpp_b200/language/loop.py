"""LoopIterationContext: ops issued inside it run as a pipeline over `num_chunks` chunks in units
of `unit` bytes (the executor iterates ceil(num_chunks * chunk_bytes / unit) times)."""
from __future__ import annotations

from . import ir
from ._context import get_program


class LoopIterationContext:
    def __init__(self, unit: int, num_chunks: int):
        self.unit = unit
        self.num_chunks = num_chunks
        self._ops = []

    def __enter__(self):
        get_program().set_loop_context(self)
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        prog = get_program()
        prog.set_loop_context(None)
        pipelines = {}
        for rank, tb, op in self._ops:
            key = (rank, tb)
            if key not in pipelines:
                pipelines[key] = ir.make_pipeline(self.unit, self.num_chunks)
            pipelines[key].body.append(op)
        for (rank, tb), pipe in pipelines.items():
            prog.add_operation(rank, tb, pipe)

    def add_operation(self, rank: int, tb: int, op) -> None:
        self._ops.append((rank, tb, op))
