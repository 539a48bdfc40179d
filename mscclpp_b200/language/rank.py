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
    raise RuntimeError("no thread block given: pass tb=<id> or tb_group=<ThreadBlockGroup>")


def _local(chunk: Chunk) -> Operand:
    return Operand(chunk.buffer, chunk.index, chunk.size)


class Rank:
    def __init__(self, rank: int):
        self.rank = rank
        if rank >= get_program().num_ranks:
            raise RuntimeError(f"rank {rank} does not exist in a program of {get_program().num_ranks} ranks")

    def get_input_buffer(self) -> BaseBuffer:
        return get_program().buffers[self.rank][BufferType.input]

    def get_output_buffer(self) -> BaseBuffer:
        return get_program().buffers[self.rank][BufferType.output]

    def _check_local_pair(self, dst_chunk: Chunk, src_chunk: Chunk):
        """Both chunks live on this rank and cover the same number of chunks."""
        for name, chunk in (("destination", dst_chunk), ("source", src_chunk)):
            if chunk.rank != self.rank:
                raise RuntimeError(f"{name} chunk belongs to rank {chunk.rank}, the operation runs on rank {self.rank}")
        if dst_chunk.size != src_chunk.size:
            raise RuntimeError(f"destination covers {dst_chunk.size} chunks, source {src_chunk.size}: sizes must be equal")

    def _copy(self, dst_chunk: Chunk, src_chunk: Chunk, tb, tb_group, from_packet=False, to_packet=False):
        self._check_local_pair(dst_chunk, src_chunk)
        if from_packet and src_chunk.buffer != BufferType.scratch:
            raise RuntimeError("packets are unpacked from the scratch buffer: the source chunk is elsewhere")
        if to_packet and dst_chunk.buffer != BufferType.scratch:
            raise RuntimeError("packets are written into the scratch buffer: the destination chunk is elsewhere")
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
        self._check_local_pair(dst_chunk, src_chunk)
        if not other_chunks:
            raise RuntimeError("reduce needs at least one chunk besides the source")
        for chunk in other_chunks:
            if chunk.rank != self.rank:
                raise RuntimeError(f"reduce on rank {self.rank} was given a chunk of rank {chunk.rank}")
            if chunk.size != src_chunk.size:
                raise RuntimeError(f"reduce operands differ in size: {chunk.size} vs {src_chunk.size} chunks")
            if packet and chunk.buffer != BufferType.scratch:
                raise RuntimeError("a packet reduce reads its other operands from the scratch buffer")
        for tb_id, tbg in _tb_targets(tb, tb_group):
            op = ir.make_reduce([_local(src_chunk)] + [_local(c) for c in other_chunks], [_local(dst_chunk)],
                                reduce_op=reduce_op, tbg=tbg, packet=packet)
            get_program().add_operation(self.rank, tb_id, op)

    def barrier(self, tb_list: List[int]):
        if len(tb_list) == 0:
            raise RuntimeError("a barrier needs at least one thread block")
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
            raise RuntimeError(f"semaphore on rank {rank}: the program has {prog.num_ranks} ranks")
        self.id = prog.next_semaphore_id(rank)
        self.rank = rank
        self.initial_value = initial_value
        prog.gpus[rank].semaphores.append(initial_value)

    def acquire(self, tb: int, data_sync: SyncType = SyncType.both):
        get_program().add_operation(self.rank, tb, ir.make_sem(True, [self.id], data_sync))

    def release(self, tb: int, data_sync: SyncType = SyncType.both):
        get_program().add_operation(self.rank, tb, ir.make_sem(False, [self.id], data_sync))
