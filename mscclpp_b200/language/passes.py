"""Post-processing passes over a thread block's op list.

  fuse()              greedy left-to-right instruction fusion
  insert_data_sync()  `nop` (block barrier) before/after ops that asked for one
  resolve_hazards()   `nop` where two ops of one thread block touch overlapping local chunks
  replicate_op()      per-instance rewrite of indices and ids

The observable behaviour (which ops fuse, where barriers land) is the execution-plan contract set by
the reference compiler (python/mscclpp/language/internal/operations.py `__add__` methods and
`add_data_sync`, internal/optimizer.py:8-31, internal/buffer_access.py:11-95), because plans must be
interchangeable; the implementation here is a rule table over one Op type.
"""
from __future__ import annotations

import bisect
import copy
from typing import Callable, List, Optional

from . import ir
from .ir import Op
from .types import BufferType, ChannelType, Instruction, SyncType

I = Instruction


# ====================================================================== fusion
def _next_forces_barrier(b: Op) -> bool:
    """True when op `b` starts with a block barrier anyway, so a trailing one on the previous op is redundant."""
    if b.is_syncing and b.data_sync.has(SyncType.before):
        return True
    if b.family == "pipeline" and b.pipeline_sync().has(SyncType.before):
        return True
    return b.family in ("sync", "barrier")


def _fuse_sync(a: Op, b: Op) -> Optional[Op]:
    if b.family == "sync":
        return ir.make_sync()
    if b.family == "barrier":
        return b
    if b.family == "pipeline" and b.pipeline_sync().has(SyncType.before):
        return b
    if b.is_syncing:
        b.data_sync = b.data_sync.without(SyncType.before)  # the explicit nop already covers it
    return None


def _fuse_syncing(a: Op, b: Op) -> Optional[Op]:
    """sem / signal / wait / flush: merge with a compatible twin, else drop a redundant trailing barrier."""
    merged = None
    if a.family == "sem" and b.family == "sem" and a.name == b.name:
        merged = ir.make_sem(a.name == I.sem_acquire, a.semaphore_ids + b.semaphore_ids, a.data_sync | b.data_sync)
    elif a.family == "signal" and b.family == "signal" and a.channel_type == b.channel_type and a.name == b.name \
            and not (a.channel_ids & b.channel_ids):
        merged = ir.make_signal(a.channel_ids | b.channel_ids, a.channel_type, a.data_sync | b.data_sync,
                                relaxed=a.name == I.relaxed_signal)
    elif a.family == "wait" and b.family == "wait" and a.name == b.name and a.channel_type == b.channel_type \
            and not (a.channel_ids & b.channel_ids):
        merged = ir.make_wait(a.channel_ids | b.channel_ids, a.channel_type, a.data_sync | b.data_sync,
                              relaxed=a.name == I.relaxed_wait)
    elif a.family == "flush" and b.family == "flush" and a.channel_type == b.channel_type:
        merged = ir.make_flush(a.channel_ids | b.channel_ids, a.channel_type, a.data_sync | b.data_sync)
    if merged is not None:
        return merged
    if _next_forces_barrier(b):
        a.data_sync = a.data_sync.without(SyncType.after)
    return None


def _fuse_barrier(a: Op, b: Op) -> Optional[Op]:
    if b.is_syncing:
        b.data_sync = b.data_sync.without(SyncType.before)
        return None
    if b.family == "sync":
        return a
    return None


def _same_tbg(a: Op, b: Op) -> bool:
    return a.tbg == b.tbg


def _fuse_get(a: Op, b: Op) -> Optional[Op]:
    if b.family == "get" and a.remote_src[0].size == b.remote_src[0].size and a.channel_type == b.channel_type \
            and _same_tbg(a, b):
        return ir.make_get(a.remote_src + b.remote_src, a.dst + b.dst, a.channel_ids + b.channel_ids, a.channel_type, a.tbg)
    return None


def _fuse_put(a: Op, b: Op) -> Optional[Op]:
    if b.family != "put" or a.name != b.name or a.channel_type != b.channel_type or not _same_tbg(a, b):
        return None
    if a.name in (I.put, I.put_packet, I.put_with_signal, I.put_with_signal_and_flush):
        if a.src[0].size != b.src[0].size:
            return None
        return ir.make_put(a.src + b.src, a.remote_dst + b.remote_dst, a.channel_ids + b.channel_ids, a.channel_type, a.tbg,
                           to_packet=a.name == I.put_packet, with_signal=a.name == I.put_with_signal,
                           with_signal_and_flush=a.name == I.put_with_signal_and_flush)
    if a.name == I.read_put_packet:
        if len(a.src) != len(b.src) or not all(x.same_span(y) for x, y in zip(a.src, b.src)):
            return None
        return ir.make_put(a.src, a.remote_dst + b.remote_dst, a.channel_ids + b.channel_ids, a.channel_type, a.tbg,
                           from_packet=True, to_packet=True)
    return None


def _fuse_reduce(a: Op, b: Op) -> Optional[Op]:
    if not _same_tbg(a, b):
        return None
    n = a.name
    if b.family == "reduce":
        if n in (I.reduce, I.reduce_packet, I.read_reduce) and n == b.name and a.src[0].same_span(b.src[0]) \
                and len(a.dst) == len(b.dst) and all(x.same_span(y) for x, y in zip(a.dst, b.dst)) \
                and a.channel_type == b.channel_type and a.reduce_op == b.reduce_op:
            return ir.make_reduce(a.src + b.src[1:], a.dst, remote_src=a.remote_src + b.remote_src,
                                  channel_ids=a.channel_ids + b.channel_ids, channel_type=a.channel_type,
                                  reduce_op=a.reduce_op, tbg=a.tbg, packet=a.packet)
        return None
    if b.family == "put" and b.channel_type == ChannelType.memory:
        plain = n in (I.reduce, I.reduce_send, I.read_reduce, I.read_reduce_send) and b.name == I.put \
            and a.dst[0].same_span(b.src[0])
        pkt = n in (I.reduce_packet, I.reduce_send_packet) and b.name == I.put_packet and a.dst[0].same_span(b.src[0])
        cpkt = n in (I.reduce_copy_packet, I.reduce_copy_send_packet) and (
            (b.name == I.put_packet and a.dst[0].same_span(b.src[0]))
            or (b.name == I.read_put_packet and a.pkt_dst[0].same_span(b.src[0])))
        if plain or pkt or cpkt:
            return ir.make_reduce(a.src, a.dst, pkt_dst=a.pkt_dst if cpkt else None, remote_src=a.remote_src,
                                  remote_dst=a.remote_dst + b.remote_dst, channel_ids=a.channel_ids,
                                  put_channel_ids=a.put_channel_ids + b.channel_ids, channel_type=b.channel_type,
                                  reduce_op=a.reduce_op, tbg=a.tbg, packet=a.packet)
        return None
    if b.family == "copy" and n == I.reduce_packet and b.name == I.copy_packet and a.dst[0].same_span(b.src[0]):
        return ir.make_reduce(a.src, a.dst, pkt_dst=b.dst, remote_src=a.remote_src, remote_dst=a.remote_dst,
                              channel_ids=a.channel_ids, put_channel_ids=a.put_channel_ids, channel_type=a.channel_type,
                              reduce_op=a.reduce_op, tbg=a.tbg, packet=a.packet)
    return None


def _fuse_gload(a: Op, b: Op) -> Optional[Op]:
    if b.family == "gstore" and b.name == I.group_store and a.buffer_type == b.buffer_type and a.size == b.size \
            and a.chunk == b.chunk and a.channel_ids == b.channel_ids and a.channel_type == b.channel_type:
        return ir.make_glres(a.buffer_type, a.size, [a.buffer_offset], [b.buffer_offset], a.channel_ids, a.channel_type,
                             a.reduce_op)
    return None


def _fuse_pipeline(a: Op, b: Op) -> Optional[Op]:
    ends_with_barrier = a.pipeline_sync().has(SyncType.after)
    if ends_with_barrier and b.is_syncing:
        b.data_sync = b.data_sync.without(SyncType.before)
        return None
    if ends_with_barrier and b.family == "sync":
        return a
    return None


_FUSERS: dict = {
    "sync": _fuse_sync, "sem": _fuse_syncing, "signal": _fuse_syncing, "wait": _fuse_syncing, "flush": _fuse_syncing,
    "barrier": _fuse_barrier, "get": _fuse_get, "put": _fuse_put, "reduce": _fuse_reduce, "gload": _fuse_gload,
    "pipeline": _fuse_pipeline,
}


def try_fuse(a: Op, b: Op) -> Optional[Op]:
    """a followed by b as one op, or None. May relax a's/b's data_sync when a barrier is provably redundant."""
    fn = _FUSERS.get(a.family)
    return fn(a, b) if fn else None


def fuse(ops: List[Op]) -> List[Op]:
    out: List[Op] = []
    i = 0
    while i < len(ops):
        cur = ops[i]
        if cur.family == "pipeline":
            cur.body = fuse(cur.body)
        j = i + 1
        while j < len(ops):
            merged = try_fuse(cur, ops[j])
            if merged is None:
                break
            cur = merged
            j += 1
        out.append(cur)
        i = j
    return out


# ====================================================================== explicit barriers
def insert_data_sync(ops: List[Op]) -> List[Op]:
    out: List[Op] = []
    for op in ops:
        if op.family == "pipeline":
            op.body = insert_data_sync(op.body)
        if op.is_syncing and op.data_sync in (SyncType.before, SyncType.both):
            out.append(ir.make_sync())
        out.append(op)
        if op.is_syncing and op.data_sync in (SyncType.after, SyncType.both):
            out.append(ir.make_sync())
    return out


# ====================================================================== hazard tracking
def local_accesses(op: Op):
    """(buffer type, first chunk, last chunk, is_write) for every local chunk range the op touches that
    needs ordering against other ops of the same thread block. Packet reads order themselves through
    their flags, so they are left out (as the reference does)."""
    f, n = op.family, op.name
    acc = []
    if f == "copy":
        if n != I.unpack_packet:
            acc += [(c.type, c.index, c.index + c.size - 1, False) for c in op.src]
        if n != I.copy_packet:
            acc += [(c.type, c.index, c.index + c.size - 1, True) for c in op.dst]
    elif f == "get":
        acc += [(c.type, c.index, c.index + c.size - 1, True) for c in op.dst]
    elif f == "put":
        if n != I.read_put_packet:
            acc += [(c.type, c.index, c.index + c.size - 1, False) for c in op.src]
    elif f == "reduce":
        for i, c in enumerate(op.src):
            if not op.packet or i != 0:
                acc.append((c.type, c.index, c.index + c.size - 1, False))
        acc += [(c.type, c.index, c.index + c.size - 1, True) for c in op.dst]
    elif f == "pipeline":
        for inner in op.body:
            acc += local_accesses(inner)
    return acc


class _HazardTracker:
    """Per buffer type: disjoint [start, end] ranges, each tagged with the op that touched it last and
    whether that touch was a write."""

    def __init__(self):
        self.ranges = {t: [] for t in (BufferType.input, BufferType.output, BufferType.scratch)}

    def clear(self):
        for lst in self.ranges.values():
            lst.clear()

    def touch(self, uid: int, btype: BufferType, start: int, end: int, write: bool) -> bool:
        """Record an access; True when it conflicts with an earlier op (which also resets the tracker)."""
        lst = self.ranges[btype]
        conflict = False
        while lst:
            # first range whose end reaches `start`; ranges are disjoint, so ends are sorted too
            idx = bisect.bisect_left([r[1] for r in lst], start)
            if idx >= len(lst):
                break
            s, e, owner, w = lst[idx]
            if not (start <= e and s <= end):
                break
            if owner != uid and (write or w):
                self.clear()
                conflict = True
                break
            del lst[idx]
            if e > end:
                bisect.insort(lst, (end + 1, e, owner, w))
            if s < start:
                bisect.insort(lst, (s, start - 1, owner, w))
        bisect.insort(self.ranges[btype], (start, end, uid, write))
        return conflict


def resolve_hazards(ops: List[Op]) -> List[Op]:
    tracker = _HazardTracker()
    out: List[Op] = []
    for op in ops:
        if op.family in ("sync", "barrier"):
            tracker.clear()
        else:
            if op.family == "pipeline":
                op.body = resolve_hazards(op.body)
            added = False
            for btype, start, end, write in local_accesses(op):
                if tracker.touch(op.uid, btype, start, end, write) and not added:
                    out.append(ir.make_sync())
                    added = True
        out.append(op)
    return out


# ====================================================================== instance replication
def replicate_op(op: Op, instance: int, instances: int, shift_index: Callable[[int, int], int]) -> None:
    """Rewrite `op` (already a private copy) for replica `instance`. shift_index(index, size) maps a chunk index."""
    for lst in (op.src, op.dst, op.remote_src, op.remote_dst):
        for c in lst:
            c.index = shift_index(c.index, c.size)
    if op.family in ("gload", "gstore"):
        op.buffer_offset = shift_index(op.buffer_offset, op.size)
        op.chunk = copy.copy(op.chunk)
        op.chunk.index = shift_index(op.chunk.index, op.size)
    if op.family == "glres":
        op.src_index = [shift_index(i, op.size) for i in op.src_index]
        op.dst_index = [shift_index(i, op.size) for i in op.dst_index]
    if op.family == "sem":
        op.semaphore_ids = [i * instances + instance for i in op.semaphore_ids]
    if op.family == "barrier":
        op.barrier_id = op.barrier_id * instances + instance
    for inner in op.body:
        replicate_op(inner, instance, instances, shift_index)
