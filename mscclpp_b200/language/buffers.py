"""Buffers are sliced with `buf[a:b]` into Chunks; `Buffer(rank, size)` grows the rank's scratch."""
from __future__ import annotations

from ._context import get_program
from .types import BufferType, Chunk


class BaseBuffer:
    def __init__(self, rank: int, buffer_type: BufferType, offset: int, size: int):
        self.rank = rank
        self.buffer_type = buffer_type
        self.offset = offset
        self.size = offset + size  # exclusive end, in chunks

    def __getitem__(self, key) -> Chunk:
        if not isinstance(key, slice):
            raise TypeError(f"Buffer indices must be slices, not {type(key).__name__}")
        if key.step is not None and key.step != 1:
            raise ValueError(f"Buffer slicing does not support step != 1 (got step={key.step})")
        length = self.size - self.offset
        start = 0 if key.start is None else key.start
        stop = length if key.stop is None else key.stop
        if start < 0 or stop < 0:
            raise ValueError(f"Buffer slicing does not support negative indices (got start={key.start}, stop={key.stop})")
        if start > stop:
            raise ValueError(f"Buffer slice start ({start}) must be <= stop ({stop})")
        if self.offset + stop > self.size:
            raise RuntimeError(f"Index range from {self.offset + start} - {self.offset + stop} is out of bounds for buffer "
                               f"{self.buffer_type}. Buffer size: {self.size}")
        return Chunk(self.rank, self.buffer_type, self.offset + start, stop - start)


class Buffer(BaseBuffer):
    """A fresh scratch region of `size` chunks on `rank`."""

    def __init__(self, rank: int, size: int):
        prog = get_program()
        if rank >= prog.num_ranks:
            raise RuntimeError(f"Rank {rank} is out of bounds. Number of ranks: {prog.num_ranks}")
        gpu = prog.gpus[rank]
        super().__init__(rank, BufferType.scratch, gpu.scratch_chunks, size)
        gpu.scratch_chunks += size
