"""Channels of the DSL: MemoryChannel (thread-copy over peer-mapped memory), PortChannel (host-proxy
driven) and SwitchChannel (NVSwitch multimem). API of the reference's python/mscclpp/language/channel.py."""
from __future__ import annotations

from typing import List

from . import ir
from ._context import get_program
from .ir import Operand
from .rank import _local, _tb_targets
from .thread_block_group import ThreadBlockGroup
from .types import BufferType, ChannelType, Chunk, RankGroup, ReduceOperationType, SyncType


def _check_rank(rank: int, what: str):
    n = get_program().num_ranks
    if rank >= n:
        raise RuntimeError(f"{what} rank {rank} is out of bounds. Number of ranks: {n}")


class _PeerChannel:
    """What memory and port channels share: an id on the source rank, signalling, remote operand set-up."""

    channel_type = ChannelType.none

    def __init__(self, dst_rank: int, src_rank: int):
        _check_rank(src_rank, "Source")
        _check_rank(dst_rank, "Destination")
        self.dst_rank = dst_rank
        self.src_rank = src_rank
        self.channel_id = get_program().gpus[src_rank].add_peer_channel(self.channel_type, dst_rank)

    # -- helpers
    def _slot(self, tb: int) -> List[int]:
        return [get_program().gpus[self.src_rank].tb(tb).channel_slot(self.channel_type, self.channel_id)]

    def _remote(self, tb: int, chunk: Chunk) -> Operand:
        slot = get_program().gpus[self.src_rank].remote_buffer_slot(tb, chunk.rank, chunk.buffer, self.channel_type)
        return Operand(chunk.buffer, chunk.index, chunk.size, slot)

    def _check_pair(self, dst_chunk: Chunk, src_chunk: Chunk):
        if src_chunk.rank != self.src_rank:
            raise RuntimeError(f"Source chunk rank {src_chunk.rank} does not match current channel source rank {self.src_rank}.")
        if dst_chunk.rank != self.dst_rank:
            raise RuntimeError(f"Dst chunk rank {dst_chunk.rank} does not match current channel dst rank {self.dst_rank}.")
        if dst_chunk.size != src_chunk.size:
            raise RuntimeError(f"Destination chunk size {dst_chunk.size} does not match source chunk size {src_chunk.size}.")

    def _emit_put(self, dst_chunk: Chunk, src_chunk: Chunk, tb, tb_group, **flags):
        for tb_id, tbg in _tb_targets(tb, tb_group):
            remote = self._remote(tb_id, dst_chunk)
            op = ir.make_put([_local(src_chunk)], [remote], self._slot(tb_id), self.channel_type, tbg, **flags)
            get_program().add_operation(self.src_rank, tb_id, op)


class MemoryChannel(_PeerChannel):
    channel_type = ChannelType.memory

    def signal(self, tb: int, data_sync: SyncType = SyncType.both, relaxed: bool = False):
        prog = get_program()
        prog.add_operation(self.src_rank, tb, ir.make_signal(self._slot(tb), self.channel_type, data_sync, relaxed))
        prog.register_signal(self.src_rank, self.dst_rank, self.channel_type)

    def wait(self, tb: int, data_sync: SyncType = SyncType.both, relaxed: bool = False):
        prog = get_program()
        prog.add_operation(self.src_rank, tb, ir.make_wait(self._slot(tb), self.channel_type, data_sync, relaxed))
        prog.register_wait(self.src_rank, self.dst_rank, self.channel_type)

    def get(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        """Copy the peer's `src_chunk` into the local `dst_chunk`."""
        if dst_chunk.rank != self.src_rank:
            raise RuntimeError(f"Source chunk rank {dst_chunk.rank} does not match current channel source rank {self.src_rank}.")
        if src_chunk.rank != self.dst_rank:
            raise RuntimeError(f"Dst chunk rank {src_chunk.rank} does not match current channel dst rank {self.dst_rank}.")
        for tb_id, tbg in _tb_targets(tb, tb_group):
            remote = self._remote(tb_id, src_chunk)
            op = ir.make_get([remote], [_local(dst_chunk)], self._slot(tb_id), self.channel_type, tbg)
            get_program().add_operation(self.src_rank, tb_id, op)

    def put(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._check_pair(dst_chunk, src_chunk)
        self._emit_put(dst_chunk, src_chunk, tb, tb_group)

    def put_packets(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._check_pair(dst_chunk, src_chunk)
        if dst_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Destination chunk must be of type scratch.")
        self._emit_put(dst_chunk, src_chunk, tb, tb_group, to_packet=True)

    def read_put_packets(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._check_pair(dst_chunk, src_chunk)
        if src_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Source chunk must be of type scratch.")
        if dst_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Destination chunk must be of type scratch.")
        self._emit_put(dst_chunk, src_chunk, tb, tb_group, from_packet=True, to_packet=True)

    def reduce(self, local_src_chunk: Chunk, remote_src_chunks: List[Chunk], tb: int = None,
               tb_group: ThreadBlockGroup = None, local_dst_chunk: Chunk = None,
               reduce_op: ReduceOperationType = ReduceOperationType.sum):
        """local_dst = local_src (op) the peer's chunks, read through the channel."""
        if local_dst_chunk is None:
            local_dst_chunk = local_src_chunk
        if local_src_chunk.rank != self.src_rank:
            raise RuntimeError(f"Destination chunk rank {local_src_chunk.rank} does not match current channel source rank {self.src_rank}.")
        if local_src_chunk.size != local_dst_chunk.size:
            raise RuntimeError(f"Source chunk size {local_src_chunk.size} does not match destination chunk size {local_dst_chunk.size}.")
        for chunk in remote_src_chunks:
            if chunk.rank != self.dst_rank:
                raise RuntimeError(f"Source chunk rank {chunk.rank} does not match current channel dst rank {self.dst_rank}.")
            if chunk.size != local_src_chunk.size:
                raise RuntimeError(f"Source chunk size {chunk.size} does not match local source chunk size {local_src_chunk.size}.")
        for tb_id, tbg in _tb_targets(tb, tb_group):
            remotes = [self._remote(tb_id, c) for c in remote_src_chunks]
            op = ir.make_reduce([_local(local_src_chunk)], [_local(local_dst_chunk)], remote_src=remotes,
                                channel_ids=self._slot(tb_id), channel_type=self.channel_type, reduce_op=reduce_op, tbg=tbg)
            get_program().add_operation(self.src_rank, tb_id, op)


class PortChannel(_PeerChannel):
    channel_type = ChannelType.port

    def signal(self, tb: int, data_sync: SyncType = SyncType.both):
        prog = get_program()
        prog.add_operation(self.src_rank, tb, ir.make_signal(self._slot(tb), self.channel_type, data_sync))
        prog.register_signal(self.src_rank, self.dst_rank, self.channel_type)

    def wait(self, tb: int, data_sync: SyncType = SyncType.both):
        prog = get_program()
        prog.add_operation(self.src_rank, tb, ir.make_wait(self._slot(tb), self.channel_type, data_sync))
        prog.register_wait(self.src_rank, self.dst_rank, self.channel_type)

    def flush(self, tb: int, data_sync: SyncType = SyncType.both):
        get_program().add_operation(self.src_rank, tb, ir.make_flush(self._slot(tb), self.channel_type, data_sync))

    def put(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int):
        self._check_pair(dst_chunk, src_chunk)
        self._emit_put(dst_chunk, src_chunk, tb, None)

    def put_with_signal(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int):
        self._check_pair(dst_chunk, src_chunk)
        self._emit_put(dst_chunk, src_chunk, tb, None, with_signal=True)
        get_program().register_signal(self.src_rank, self.dst_rank, self.channel_type)

    def put_with_signal_and_flush(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int):
        self._check_pair(dst_chunk, src_chunk)
        self._emit_put(dst_chunk, src_chunk, tb, None, with_signal_and_flush=True)
        get_program().register_signal(self.src_rank, self.dst_rank, self.channel_type)

    def put_packets(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int):
        self._check_pair(dst_chunk, src_chunk)
        if dst_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Destination chunk must be of type scratch.")
        self._emit_put(dst_chunk, src_chunk, tb, None, to_packet=True)

    def read_put_packets(self, dst_chunk: Chunk, src_chunk: Chunk, tb: int = None, tb_group: ThreadBlockGroup = None):
        self._check_pair(dst_chunk, src_chunk)
        if src_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Source chunk must be of type scratch.")
        if dst_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Destination chunk must be of type scratch.")
        self._emit_put(dst_chunk, src_chunk, tb, tb_group, from_packet=True, to_packet=True)


class SwitchChannel:
    """One multicast group over `rank_list`, bound to every member's input, output or scratch buffer."""

    channel_type = ChannelType.switch

    def __init__(self, rank_list: List[int], buffer_type: BufferType):
        prog = get_program()
        if not all(r < prog.num_ranks for r in rank_list):
            raise RuntimeError(f"One or more ranks in {rank_list} are out of bounds. Number of ranks: {prog.num_ranks}")
        self.buffer_type = buffer_type
        self.rank_group = RankGroup(len(rank_list), list(rank_list))
        self.channel_ids = {r: prog.gpus[r].add_switch_channel(buffer_type, self.rank_group) for r in rank_list}

    def at_rank(self, rank: int) -> "SwitchChannel.SwitchChannelRankView":
        if rank not in self.rank_group.ranks:
            raise RuntimeError(f"Rank {rank} is not part of this SwitchChannel's rank group.")
        return SwitchChannel.SwitchChannelRankView(self, rank)

    def _slot(self, rank: int, tb: int) -> List[int]:
        return [get_program().gpus[rank].tb(tb).channel_slot(self.channel_type, self.channel_ids[rank])]

    def _check_extent(self, buffer_offset: int, size: int):
        prog = get_program()
        for r in self.rank_group.ranks:
            have = prog.gpus[r].scratch_chunks if self.buffer_type == BufferType.scratch else prog.buffers[r][self.buffer_type].size
            if have < buffer_offset + size:
                raise RuntimeError(f"Buffer size {have} is smaller than required size {buffer_offset + size} for rank {r}.")

    def reduce(self, rank, buffer_offset, size, dst_chunk: Chunk, tb, reduce_op=ReduceOperationType.sum):
        """dst_chunk (local on `rank`) = reduction over the group of [buffer_offset, +size) of the bound buffer."""
        if dst_chunk.rank not in self.rank_group.ranks:
            raise RuntimeError(f"Destination chunk rank {dst_chunk.rank} is not part of the rank group {self.rank_group.ranks}.")
        if dst_chunk.size != size:
            raise RuntimeError(f"Destination chunk size {dst_chunk.size} does not match the required size {size}.")
        self._check_extent(buffer_offset, size)
        op = ir.make_group_load_reduce(self.buffer_type, buffer_offset, size, dst_chunk, self._slot(rank, tb),
                                       self.channel_type, reduce_op)
        get_program().add_operation(rank, tb, op)

    def broadcast(self, rank, src_chunk: Chunk, buffer_offset, size, tb):
        """Store src_chunk (local on `rank`) into [buffer_offset, +size) of every member's bound buffer."""
        if src_chunk.rank not in self.rank_group.ranks:
            raise RuntimeError(f"Source chunk rank {src_chunk.rank} is not part of the rank group {self.rank_group.ranks}.")
        if src_chunk.size != size:
            raise RuntimeError(f"Source chunk size {src_chunk.size} does not match the required size {size}.")
        self._check_extent(buffer_offset, size)
        op = ir.make_group_store(src_chunk, self.buffer_type, buffer_offset, size, self._slot(rank, tb), self.channel_type)
        get_program().add_operation(rank, tb, op)

    def broadcast_packets(self, rank, src_chunk: Chunk, buffer_offset, size, tb):
        if src_chunk.rank not in self.rank_group.ranks:
            raise RuntimeError(f"Source chunk rank {src_chunk.rank} is not part of the rank group {self.rank_group.ranks}.")
        if src_chunk.buffer != BufferType.scratch:
            raise RuntimeError("Source chunk must be of type scratch.")
        if self.buffer_type != BufferType.scratch:
            raise RuntimeError("Switch channel buffer must be of type scratch.")
        if src_chunk.size != size:
            raise RuntimeError(f"Source chunk size {src_chunk.size} does not match the required size {size}.")
        self._check_extent(buffer_offset, size)
        op = ir.make_group_store(src_chunk, self.buffer_type, buffer_offset, size, self._slot(rank, tb), self.channel_type,
                                 use_packet=True)
        get_program().add_operation(rank, tb, op)

    class SwitchChannelRankView:
        def __init__(self, channel: "SwitchChannel", rank: int):
            self._channel = channel
            self._rank = rank

        def reduce(self, buffer_offset, size, dst_chunk: Chunk, tb, reduce_op=ReduceOperationType.sum):
            return self._channel.reduce(self._rank, buffer_offset, size, dst_chunk, tb, reduce_op)

        def broadcast(self, src_chunk: Chunk, buffer_offset, size, tb):
            return self._channel.broadcast(self._rank, src_chunk, buffer_offset, size, tb)

        def broadcast_packets(self, src_chunk: Chunk, buffer_offset, size, tb):
            return self._channel.broadcast_packets(self._rank, src_chunk, buffer_offset, size, tb)
