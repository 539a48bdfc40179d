"""Enumerations and small value types of the DSL.

Names and string values are the execution-plan format's vocabulary (they appear verbatim in the
JSON), so they match the reference (python/mscclpp/language/internal/types.py:64-123).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import List


class _BitEnum(Enum):
    """Enum whose members combine like bit masks through a class-level `_bits` table."""

    def _combine(self, other, fn):
        if not isinstance(other, type(self)):
            return NotImplemented
        bits = type(self)._bits()
        inv = {v: k for k, v in bits.items()}
        return inv[fn(bits[self], bits[other])]

    def __or__(self, other):
        return self._combine(other, lambda a, b: a | b)

    def __and__(self, other):
        return self._combine(other, lambda a, b: a & b)

    def __xor__(self, other):
        return self._combine(other, lambda a, b: a ^ b)

    def __str__(self):
        return self.value


class SyncType(_BitEnum):
    """Where a synchronising op needs a block-wide barrier relative to itself."""

    none = "none"
    before = "before"
    after = "after"
    both = "both"

    @classmethod
    def _bits(cls):
        return {cls.none: 0, cls.before: 1, cls.after: 2, cls.both: 3}

    def has(self, flag: "SyncType") -> bool:
        return (self & flag) == flag

    def without(self, flag: "SyncType") -> "SyncType":
        return self ^ (flag & self)


class ReduceOperationType(Enum):
    sum = "sum"
    min = "min"
    max = "max"

    def __str__(self):
        return self.value


class BufferType(Enum):
    input = "i"
    output = "o"
    scratch = "s"

    def __str__(self):
        return self.value

    def __lt__(self, other):
        return self.value < other.value


class Instruction(Enum):
    start = "start"
    nop = "nop"
    copy = "copy"
    copy_packet = "cpkt"
    unpack_packet = "upkt"
    reduce = "re"
    reduce_packet = "repkt"
    reduce_copy_packet = "recpkt"
    sem_acquire = "sem_acquire"
    sem_release = "sem_release"
    signal = "signal"
    wait = "wait"
    relaxed_signal = "rlxsignal"
    relaxed_wait = "rlxwait"
    barrier = "barrier"
    flush = "flush"
    get = "get"
    put = "put"
    put_packet = "ppkt"
    read_put_packet = "rppkt"
    put_with_signal = "pws"
    put_with_signal_and_flush = "pwsf"
    reduce_send = "res"
    reduce_send_packet = "respkt"
    reduce_copy_send_packet = "recspkt"
    read_reduce = "rre"
    read_reduce_send = "rres"
    group_store = "gstore"
    group_store_packet = "gstorepkt"
    group_load_reduce = "glre"
    group_load_reduce_store = "glres"
    pipeline = "pipeline"

    def __str__(self):
        return self.value


class ChannelType(Enum):
    port = "port"
    memory = "memory"
    switch = "switch"
    none = "none"

    def __str__(self):
        return self.value


class ReplicationPolicy(Enum):
    interleaved = "interleaved"
    none = "none"

    def __str__(self):
        return self.value


@dataclass
class Chunk:
    """A run of `size` chunks starting at `index` in one buffer of one rank."""

    rank: int
    buffer: BufferType
    index: int
    size: int

    def __hash__(self):
        return hash((self.rank, self.buffer, self.index, self.size))

    def to_dict(self):
        return {"rank": self.rank, "type": self.buffer.value, "index": self.index, "size": self.size}


@dataclass
class RankGroup:
    size: int
    ranks: List[int]

    def to_dict(self):
        return {"size": self.size, "ranks": self.ranks}
