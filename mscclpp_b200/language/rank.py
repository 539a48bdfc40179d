"""Rank-local operations (copy, packet pack/unpack, reduce, barrier) and device semaphores.
API of the reference's python/mscclpp/language/rank.py."""
from __future__ import annotations

from typing import List, Optional

from . import ir
from ._context import get_program
from .buffers import BaseBuffer, Buffer  # noqa: F401  (re-exported: reference users import them from here)
from .ir import Operand, TbgInfo
from .thread_block_group import ThreadBlockGroup
from .types import BufferType, Chunk, ReduceOperationType, SyncType


def _tb_targets(tb: Optional[int], tb_group: Optional[ThreadBlockGroup]):
    """[(tb id, TbgInfo or None)] an op is issued on."""
    if tb is not None:
        return [(tb, None)]
    if tb_group is not None:
        return [(t, TbgInfo(tb_group.get_internal_id(t), tb_group.numtb())) for t in tb_group.tb_list]
    raise RuntimeError("Either 'tb' (thread block ID) or 'tb_group' (ThreadBlockGroup) must be provided, but both are None.")


def _local(chunk: Chunk) -> Operand:
    return Operand(chunk.buffer, chunk.index, chunk.size)


class Rank:
    def __init__(self, rank: int):
        self.rank = rank
        if rank >= get_program().num_ranks:
            raise RuntimeError(f"Rank {rank} is out of bounds. Number of ranks: {get_program().num_ranks}")

    def get_input_buffer(self) -> BaseBuffer:
        return get_program().buffers[self.rank][BufferType.input]

    def get_output_buffer(self) -> BaseBuffer:
        return get_program().buffers[self.rank][BufferType.output]

    def _copy(self, dst_chunk: Chunk, src_chunk: Chunk, tb, tb_group, from_packet=False, to_packet=False):
        if dst_chunk.rank != self.rank or src_chunk.rank != self.rank:
            raise RuntimeError(f"Inconsistent ranks: dst {dst_chunk.rank}, src {src_chunk.rank}, self {self.rank}. They must match.")
        if dst_chunk.size != src_chunk.size:
            raise RuntimeError(f"Inconsistent chunk sizes: dst {dst_chunk.size}, src {src_chunk.size}. They must match.")
        if from_packet and src_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Source chunk must be of type scratch.")
        if to_packet and dst_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Destination chunk must be of type scratch.")
        for tb_id, tbg in _tb_targets(tb, tb_group):
            op = ir.make_copy(_local(src_chunk), _local(dst_chunk), tbg, from_packet, to_packet)
            get_program().add_operation(self.rank, tb_id, op)

    def copy(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._copy(dst_chunk, src_chunk, tb, tb_group)

    def unpack_packets(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._copy(dst_chunk, src_chunk, tb, tb_group, from_packet=True)

    def copy_packets(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._copy(dst_chunk, src_chunk, tb, tb_group, to_packet=True)

    def reduce(self, src_chunk: Chunk, other_chunks: List[Chunk], tb: int = None, tb_group: ThreadBlockGroup = None,
               dst_chunk: Chunk = None, reduce_op: ReduceOperationType = ReduceOperationType.sum, packet: bool = False):
        if dst_chunk is None:
            dst_chunk = src_chunk
        if dst_chunk.rank != self.rank or src_chunk.rank != self.rank:
            raise RuntimeError(f"Inconsistent ranks: dst {dst_chunk.rank}, src {src_chunk.rank}, self {self.rank}. They must match.")
        if dst_chunk.size != src_chunk.size:
            raise RuntimeError(f"Inconsistent chunk sizes: dst {dst_chunk.size}, src {src_chunk.size}. They must match.")
        if len(other_chunks) == 0:
            raise RuntimeError("Other chunk empty.")
        for chunk in other_chunks:
            if chunk.rank != self.rank:
                raise RuntimeError(f"Other chunk rank {chunk.rank} does not match current rank {self.rank}.")
            if chunk.size != src_chunk.size:
                raise RuntimeError(f"Inconsistent chunk sizes: other {chunk.size}, src {src_chunk.size}. They must match.")
            if packet and chunk.buffer != BufferType.scratch:
                raise RuntimeError("Other chunk must be of type scratch.")
        for tb_id, tbg in _tb_targets(tb, tb_group):
            op = ir.make_reduce([_local(src_chunk)] + [_local(c) for c in other_chunks], [_local(dst_chunk)],
                                reduce_op=reduce_op, tbg=tbg, packet=packet)
            get_program().add_operation(self.rank, tb_id, op)

    def barrier(self, tb_list: List[int]):
        if len(tb_list) == 0:
            raise RuntimeError("Barrier requires at least thread block.")
        prog = get_program()
        if len(tb_list) == 1:
            prog.add_operation(self.rank, tb_list[0], ir.make_sync())
            return
        op = ir.make_barrier(prog.gpus[self.rank].barrier_id(tb_list), tb_list)
        for tb in tb_list:
            prog.add_operation(self.rank, tb, op)


class Semaphore:
    """Counting semaphore shared by the thread blocks of one rank."""

    def __init__(self, rank: int, initial_value: int):
        prog = get_program()
        if rank >= prog.num_ranks:
            raise RuntimeError(f"Source rank {rank} is out of bounds. Number of ranks: {prog.num_ranks}")
        self.id = prog.next_semaphore_id(rank)
        self.rank = rank
        self.initial_value = initial_value
        prog.gpus[rank].semaphores.append(initial_value)

    def acquire(self, tb: int, data_sync: SyncType = SyncType.both):
        get_program().add_operation(self.rank, tb, ir.make_sem(True, [self.id], data_sync))

    def release(self, tb: int, data_sync: SyncType = SyncType.both):
        get_program().add_operation(self.rank, tb, ir.make_sem(False, [self.id], data_sync))
