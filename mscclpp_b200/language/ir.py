"""Operation IR of the DSL and its JSON form.

One `Op` class covers every instruction; `family` selects which fields are meaningful. The passes
in `passes.py` (fusion, sync insertion, dependency sync, instance replication) are plain functions
over lists of `Op`. The emitted dictionaries follow the plan format the executor parses (op names
of src/core/executor/execution_plan.cc:25-89; operand shapes of
python/mscclpp/language/internal/operations.py `to_dict` methods).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import List, Optional, Set

from .types import BufferType, ChannelType, Chunk, Instruction, ReduceOperationType, SyncType

_op_ids = itertools.count(1)


@dataclass
class Operand:
    """Local operand when buffer_id is None, remote operand (buffer named by a thread-block-local
    remote-buffer index) otherwise."""

    type: BufferType
    index: int
    size: int
    buffer_id: Optional[int] = None

    def same_span(self, other: "Operand") -> bool:
        return (self.type, self.index, self.size, self.buffer_id) == (other.type, other.index, other.size, other.buffer_id)

    def to_dict(self):
        if self.buffer_id is None:
            return {"type": self.type.value, "index": self.index, "size": self.size}
        return {"buffer_id": self.buffer_id, "index": self.index, "size": self.size}


@dataclass
class TbgInfo:
    tb_id: int
    tbg_size: int

    def to_dict(self):
        return {"tb_id": self.tb_id, "tbg_size": self.tbg_size}


SYNCING_FAMILIES = ("sem", "signal", "wait", "flush")


@dataclass
class Op:
    name: Instruction
    family: str
    uid: int = field(default_factory=lambda: next(_op_ids))
    # data movement
    src: List[Operand] = field(default_factory=list)        # local sources
    dst: List[Operand] = field(default_factory=list)        # local destinations
    pkt_dst: List[Operand] = field(default_factory=list)    # reduce: extra local packet destination
    remote_src: List[Operand] = field(default_factory=list)
    remote_dst: List[Operand] = field(default_factory=list)
    channel_ids: object = None          # list (data ops) or set (signal/wait/flush)
    put_channel_ids: List[int] = field(default_factory=list)
    channel_type: ChannelType = ChannelType.none
    tbg: Optional[TbgInfo] = None
    reduce_op: ReduceOperationType = ReduceOperationType.sum
    packet: bool = False
    # synchronisation
    data_sync: SyncType = SyncType.none
    semaphore_ids: List[int] = field(default_factory=list)
    barrier_id: int = 0
    barrier_tbs: tuple = ()
    # switch ops
    buffer_type: Optional[BufferType] = None
    buffer_offset: int = 0
    size: int = 0
    chunk: Optional[Chunk] = None
    src_index: List[int] = field(default_factory=list)
    dst_index: List[int] = field(default_factory=list)
    # pipeline
    unit_size: int = 0
    num_chunks: int = 0
    body: List["Op"] = field(default_factory=list)

    @property
    def is_syncing(self) -> bool:
        return self.family in SYNCING_FAMILIES

    # ------------------------------------------------------------------ pipeline helpers
    def pipeline_sync(self) -> SyncType:
        """Which barriers the first/last inner op of a pipeline already implies."""
        result = SyncType.none
        if self.body:
            result |= _edge_sync(self.body[0], SyncType.before)
            result |= _edge_sync(self.body[-1], SyncType.after)
        return result

    # ------------------------------------------------------------------ JSON
    def to_dict(self) -> dict:
        f = self.family
        out = {"name": self.name.value}
        if f == "sync":
            return out
        if f == "copy":
            out["src_buff"] = [c.to_dict() for c in self.src]
            out["dst_buff"] = [c.to_dict() for c in self.dst]
        elif f == "sem":
            out["semaphore_ids"] = list(self.semaphore_ids)
        elif f in ("signal", "wait", "flush"):
            out["channel_ids"] = list(self.channel_ids)
            out["channel_type"] = self.channel_type.value
        elif f == "barrier":
            out["barrier_id"] = self.barrier_id
            out["num_threadblocks"] = len(self.barrier_tbs)
        elif f == "get":
            out["src_buff"] = [c.to_dict() for c in self.remote_src]
            out["dst_buff"] = [c.to_dict() for c in self.dst]
            out["channel_ids"] = self.channel_ids
            out["channel_type"] = self.channel_type.value
        elif f == "put":
            out["src_buff"] = [c.to_dict() for c in self.src]
            out["dst_buff"] = [c.to_dict() for c in self.remote_dst]
            if self.channel_type == ChannelType.port:
                out["channel_ids"] = self.channel_ids
            out["channel_type"] = self.channel_type.value
        elif f == "reduce":
            out["src_buff"] = [c.to_dict() for c in self.src] + [c.to_dict() for c in self.remote_src]
            out["dst_buff"] = [c.to_dict() for c in self.dst] + [c.to_dict() for c in self.pkt_dst] + \
                [c.to_dict() for c in self.remote_dst]
            if self.channel_type != ChannelType.none:
                out["channel_type"] = self.channel_type.value
            out["reduce_op"] = self.reduce_op.value
        elif f == "gload":
            out["buffer_type"] = self.buffer_type.value
            out["buffer_offset"] = self.buffer_offset
            out["size"] = self.size
            out["dst_chunk"] = self.chunk.to_dict()
            out["channel_ids"] = self.channel_ids
            out["channel_type"] = self.channel_type.value
            out["reduce_op"] = self.reduce_op.value
            return out
        elif f == "gstore":
            out["src_buff"] = [self.chunk.to_dict()]
            out["dst_buff"] = [{"switch_channel_id": self.channel_ids[0], "index": self.buffer_offset, "size": self.size}]
            out["channel_type"] = self.channel_type.value
            return out
        elif f == "glres":
            out["src_buff"] = [{"switch_channel_id": self.channel_ids[i], "index": self.src_index[i], "size": self.size}
                               for i in range(len(self.src_index))]
            # The plan format as produced by the reference writes the *source* index into dst_buff too
            # (python/mscclpp/language/internal/operations.py:976-980); in-place switch allreduce, the
            # only user, has equal indices. Kept for plan compatibility.
            out["dst_buff"] = [{"switch_channel_id": self.channel_ids[i], "index": self.src_index[i], "size": self.size}
                               for i in range(len(self.dst_index))]
            out["channel_type"] = self.channel_type.value
            out["reduce_op"] = self.reduce_op.value
            return out
        elif f == "pipeline":
            out["iter_context"] = {"unit_size": self.unit_size, "num_chunks": self.num_chunks}
            out["ops"] = [o.to_dict() for o in self.body]
            return out
        if self.tbg is not None and f in ("copy", "get", "put", "reduce"):
            out["tbg_info"] = self.tbg.to_dict()
        return out


def _edge_sync(op: Op, flag: SyncType) -> SyncType:
    result = SyncType.none
    if op.family in ("sync", "barrier"):
        result |= SyncType.before
    if op.is_syncing:
        result |= flag & op.data_sync
    return result


# ---------------------------------------------------------------------- constructors
def make_sync() -> Op:
    return Op(Instruction.nop, "sync")


def make_copy(src: Operand, dst: Operand, tbg=None, from_packet=False, to_packet=False) -> Op:
    if from_packet and to_packet:
        raise RuntimeError("Copy Operation from Packet to Packet is not Supported.")
    name = Instruction.unpack_packet if from_packet else (Instruction.copy_packet if to_packet else Instruction.copy)
    return Op(name, "copy", src=[src], dst=[dst], tbg=tbg)


def make_sem(acquire: bool, ids: List[int], data_sync: SyncType) -> Op:
    return Op(Instruction.sem_acquire if acquire else Instruction.sem_release, "sem", semaphore_ids=list(ids),
              data_sync=data_sync)


def make_signal(ids, channel_type, data_sync=SyncType.none, relaxed=False) -> Op:
    return Op(Instruction.relaxed_signal if relaxed else Instruction.signal, "signal", channel_ids=set(ids),
              channel_type=channel_type, data_sync=data_sync)


def make_wait(ids, channel_type, data_sync=SyncType.none, relaxed=False) -> Op:
    return Op(Instruction.relaxed_wait if relaxed else Instruction.wait, "wait", channel_ids=set(ids),
              channel_type=channel_type, data_sync=data_sync)


def make_flush(ids, channel_type, data_sync=SyncType.none) -> Op:
    return Op(Instruction.flush, "flush", channel_ids=set(ids), channel_type=channel_type, data_sync=data_sync)


def make_barrier(barrier_id: int, tb_list) -> Op:
    return Op(Instruction.barrier, "barrier", barrier_id=barrier_id, barrier_tbs=tuple(tb_list))


def make_get(remote_src: List[Operand], dst: List[Operand], channel_ids, channel_type, tbg=None) -> Op:
    return Op(Instruction.get, "get", remote_src=remote_src, dst=dst, channel_ids=list(channel_ids),
              channel_type=channel_type, tbg=tbg)


def make_put(src: List[Operand], remote_dst: List[Operand], channel_ids, channel_type, tbg=None, from_packet=False,
             to_packet=False, with_signal=False, with_signal_and_flush=False) -> Op:
    if from_packet and to_packet:
        name = Instruction.read_put_packet
    elif to_packet:
        name = Instruction.put_packet
    elif from_packet:
        raise RuntimeError("Put Operation from Packet is not Supported.")
    elif with_signal_and_flush:
        name = Instruction.put_with_signal_and_flush
    elif with_signal:
        name = Instruction.put_with_signal
    else:
        name = Instruction.put
    op = Op(name, "put", src=src, remote_dst=remote_dst, channel_ids=list(channel_ids), channel_type=channel_type, tbg=tbg)
    op.packet = to_packet
    return op


def reduce_name(has_remote_src: bool, has_remote_dst: bool, packet: bool, has_pkt_dst: bool) -> Instruction:
    if not has_remote_src and not has_remote_dst:
        if packet:
            return Instruction.reduce_copy_packet if has_pkt_dst else Instruction.reduce_packet
        return Instruction.reduce
    if not has_remote_src:
        if packet:
            return Instruction.reduce_copy_send_packet if has_pkt_dst else Instruction.reduce_send_packet
        return Instruction.reduce_send
    if not packet:
        return Instruction.read_reduce if not has_remote_dst else Instruction.read_reduce_send
    raise RuntimeError("Reduce Operation invalid parameters.")


def make_reduce(src, dst, pkt_dst=None, remote_src=None, remote_dst=None, channel_ids=None, put_channel_ids=None,
                channel_type=ChannelType.none, reduce_op=ReduceOperationType.sum, tbg=None, packet=False) -> Op:
    pkt_dst = list(pkt_dst or [])
    remote_src = list(remote_src or [])
    remote_dst = list(remote_dst or [])
    name = reduce_name(bool(remote_src), bool(remote_dst), packet, bool(pkt_dst))
    return Op(name, "reduce", src=list(src), dst=list(dst), pkt_dst=pkt_dst, remote_src=remote_src, remote_dst=remote_dst,
              channel_ids=list(channel_ids or []), put_channel_ids=list(put_channel_ids or []), channel_type=channel_type,
              reduce_op=reduce_op, tbg=tbg, packet=packet)


def make_group_load_reduce(buffer_type, offset, size, dst_chunk, channel_ids, channel_type, reduce_op) -> Op:
    return Op(Instruction.group_load_reduce, "gload", buffer_type=buffer_type, buffer_offset=offset, size=size,
              chunk=dst_chunk, channel_ids=list(channel_ids), channel_type=channel_type, reduce_op=reduce_op)


def make_group_store(src_chunk, buffer_type, offset, size, channel_ids, channel_type, use_packet=False) -> Op:
    return Op(Instruction.group_store_packet if use_packet else Instruction.group_store, "gstore", chunk=src_chunk,
              buffer_type=buffer_type, buffer_offset=offset, size=size, channel_ids=list(channel_ids),
              channel_type=channel_type)


def make_glres(buffer_type, size, src_index, dst_index, channel_ids, channel_type, reduce_op) -> Op:
    return Op(Instruction.group_load_reduce_store, "glres", buffer_type=buffer_type, size=size, src_index=list(src_index),
              dst_index=list(dst_index), channel_ids=list(channel_ids), channel_type=channel_type, reduce_op=reduce_op)


def make_pipeline(unit_size: int, num_chunks: int) -> Op:
    return Op(Instruction.pipeline, "pipeline", unit_size=unit_size, num_chunks=num_chunks)
