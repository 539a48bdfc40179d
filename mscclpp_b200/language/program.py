"""CollectiveProgram: the container a DSL algorithm is written into and the source of the JSON plan.

Public surface follows the reference (python/mscclpp/language/program.py:44-284). Differences that are
deliberate: post-processing runs exactly once per program (to_json() can be called repeatedly and
yields the same plan), id counters are per program instead of process-global, and the `none`
replication policy works.
"""
from __future__ import annotations

import json
from collections import defaultdict
from typing import List, Optional

from . import _context
from .collectives import Collective
from .state import RankState
from .types import BufferType, ChannelType, ReplicationPolicy
from .utils import AlgoSpec


class CollectiveProgram:
    def __init__(self, name: str, collective: Collective, num_ranks: int, instances: int = 1, protocol: str = "Simple",
                 instr_fusion: bool = True, auto_sync: bool = True,
                 replication_policy: ReplicationPolicy = ReplicationPolicy.interleaved, reuse_resources: bool = False,
                 num_threads_per_block: int = 1024, use_double_scratch_buffer: bool = False, buffer_alignment: int = 16,
                 min_message_size: int = 0, max_message_size: int = 2**64 - 1):
        assert protocol in ("Simple", "LL"), f"Given protocol: {protocol}. Must be either Simple, LL"
        self.name = name
        self.collective = collective
        self.num_ranks = num_ranks
        self.instances = instances
        self.protocol = protocol
        self.instr_fusion = instr_fusion
        self.auto_sync = auto_sync
        self.replication_policy = replication_policy
        self.reuse_resources = reuse_resources
        self.num_threads_per_block = num_threads_per_block
        self.use_double_scratch_buffer = use_double_scratch_buffer
        self.buffer_alignment = buffer_alignment
        self.min_message_size = min_message_size
        self.max_message_size = max_message_size
        self.buffers = collective.init_buffers()
        self.gpus: List[RankState] = [
            RankState(r, self.buffers[r][BufferType.input].size, self.buffers[r][BufferType.output].size)
            for r in range(num_ranks)
        ]
        self.loop_context = None
        self._signals = defaultdict(int)
        self._waits = defaultdict(int)
        self._semaphore_counts = defaultdict(int)
        self._post_processed = False

    @classmethod
    def from_spec(cls, spec: AlgoSpec) -> "CollectiveProgram":
        return cls(spec.name, spec.collective, spec.world_size, instances=spec.instances, protocol=spec.protocol,
                   instr_fusion=spec.instr_fusion, auto_sync=spec.auto_sync, replication_policy=spec.replication_policy,
                   reuse_resources=spec.reuse_resources, num_threads_per_block=spec.num_threads_per_block,
                   use_double_scratch_buffer=spec.use_double_scratch_buffer, buffer_alignment=spec.buffer_alignment,
                   min_message_size=spec.min_message_size, max_message_size=spec.max_message_size)

    def __enter__(self):
        _context.set_program(self)
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        _context.set_program(None)

    # ------------------------------------------------------------------ used by channels / ranks
    def add_operation(self, rank: int, tb: int, op) -> None:
        if self._post_processed:
            raise RuntimeError("the program has already been compiled; create a new CollectiveProgram")
        if self.loop_context is not None:
            self.loop_context.add_operation(rank, tb, op)
        else:
            self.gpus[rank].tb(tb).ops.append(op)

    def register_signal(self, src_rank: int, dst_rank: int, channel_type: ChannelType) -> None:
        self._signals[(src_rank, dst_rank, channel_type)] += 1

    def register_wait(self, src_rank: int, dst_rank: int, channel_type: ChannelType) -> None:
        self._waits[(src_rank, dst_rank, channel_type)] += 1

    def next_semaphore_id(self, rank: int) -> int:
        sid = self._semaphore_counts[rank]
        self._semaphore_counts[rank] += 1
        return sid

    def set_loop_context(self, loop_context) -> None:
        if self.loop_context is not None and loop_context is not None:
            raise RuntimeError("Nested Pipelines are not Supported.")
        self.loop_context = loop_context

    # ------------------------------------------------------------------ compile
    def validate_signal_wait_pairing(self) -> None:
        """Every signal rank a sends to rank b over one channel type needs a wait on b for a."""
        keys = set(self._signals) | {(dst, src, t) for (src, dst, t) in self._waits}
        for src, dst, t in keys:
            signals = self._signals.get((src, dst, t), 0)
            waits = self._waits.get((dst, src, t), 0)
            if signals != waits:
                raise RuntimeError(
                    f"Signal/Wait mismatch on {t}: rank {src} issues {signals} signal(s) to rank {dst}, but rank {dst} "
                    f"performs {waits} wait(s) for rank {src}. Every signal must be matched by a corresponding wait "
                    f"on the peer rank over a channel of the same type.")

    def post_process_operations(self) -> None:
        if self._post_processed:
            return
        self.validate_signal_wait_pairing()
        for gpu in self.gpus:
            gpu.post_process(self.instr_fusion, self.auto_sync, self.instances, self.replication_policy)
        self._post_processed = True

    def to_dict(self) -> dict:
        self.post_process_operations()
        return {
            "name": self.name,
            "collective": self.collective.name,
            "protocol": self.protocol,
            "inplace": self.collective.inplace,
            "reuse_resources": self.reuse_resources,
            "gpus": [gpu.to_dict() for gpu in self.gpus],
            "num_threads_per_block": self.num_threads_per_block,
            "use_double_scratch_buffer": self.use_double_scratch_buffer,
            "buffer_alignment": self.buffer_alignment,
            "min_message_size": self.min_message_size,
            "max_message_size": self.max_message_size,
        }

    def to_json(self, indent: Optional[int] = 2, **kwargs) -> str:
        return json.dumps(self.to_dict(), indent=indent, **kwargs)
