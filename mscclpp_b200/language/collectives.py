"""Collective descriptors: how many chunks each rank's input and output buffers hold.

With `f = chunk_factor` and `n = num_ranks`: AllGather f -> n*f, AllReduce n*f -> n*f, ReduceScatter n*f -> f,
AllToAll n*f -> n*f, SendRecv f -> f (reference: python/mscclpp/language/collectives.py:36-281)."""
from __future__ import annotations

from .buffers import BaseBuffer
from .types import BufferType


class Collective:
    name = "custom"

    def __init__(self, num_ranks: int, chunk_factor: int, inplace: bool):
        self.num_ranks = num_ranks
        self.chunk_factor = chunk_factor
        self.inplace = inplace
        self.name = type(self).name

    def buffer_sizes(self):
        """(input chunks, output chunks) of one rank."""
        raise NotImplementedError

    def init_buffers(self):
        sizes_in, sizes_out = self.buffer_sizes()
        return [{BufferType.input: BaseBuffer(r, BufferType.input, 0, sizes_in),
                 BufferType.output: BaseBuffer(r, BufferType.output, 0, sizes_out)} for r in range(self.num_ranks)]

    def check(self, prog):
        pass


class TestCollective(Collective):
    name = "test"
    __test__ = False  # not a pytest class

    def __init__(self, num_ranks: int, input_size: int, output_size: int):
        super().__init__(num_ranks, 1, False)
        self.input_size = input_size
        self.output_size = output_size

    def buffer_sizes(self):
        return self.input_size, self.output_size


class AllGather(Collective):
    name = "allgather"

    def buffer_sizes(self):
        return self.chunk_factor, self.num_ranks * self.chunk_factor


class AllReduce(Collective):
    name = "allreduce"

    def buffer_sizes(self):
        return self.num_ranks * self.chunk_factor, self.num_ranks * self.chunk_factor


class ReduceScatter(Collective):
    name = "reducescatter"

    def buffer_sizes(self):
        return self.num_ranks * self.chunk_factor, self.chunk_factor


class AllToAll(Collective):
    name = "alltoall"

    def buffer_sizes(self):
        return self.num_ranks * self.chunk_factor, self.num_ranks * self.chunk_factor


class SendRecv(Collective):
    name = "sendrecv"

    def buffer_sizes(self):
        return self.chunk_factor, self.chunk_factor
