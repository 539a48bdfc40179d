"""AlgoSpec: everything a compiler entry point needs to know to build one plan."""
from __future__ import annotations

from dataclasses import dataclass, field

from .types import ReplicationPolicy

__all__ = ["AlgoSpec", "ReplicationPolicy"]


@dataclass(frozen=True)
class AlgoSpec:
    name: str
    collective: object
    nranks_per_node: int
    world_size: int
    in_place: bool
    instances: int
    protocol: str
    instr_fusion: bool = True
    auto_sync: bool = True
    replication_policy: ReplicationPolicy = ReplicationPolicy.interleaved
    reuse_resources: bool = False
    num_threads_per_block: int = 1024
    use_double_scratch_buffer: bool = False
    buffer_alignment: int = 16
    min_message_size: int = 0
    max_message_size: int = 2**64 - 1
    tags: dict = field(default_factory=dict)
