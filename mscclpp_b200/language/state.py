"""Per-rank bookkeeping of a program under construction: thread blocks, channel tables, remote
buffer tables, semaphores; and their JSON form (the `gpus[]` entries of a plan)."""
from __future__ import annotations

import copy
from typing import Dict, List

from . import passes
from .ir import Op
from .types import BufferType, ChannelType, RankGroup, ReplicationPolicy

_CHANNEL_ACCESS_ORDER = {ChannelType.memory: 0, ChannelType.port: 1, ChannelType.switch: 2}


class ThreadBlockState:
    def __init__(self, tb_id: int):
        self.id = tb_id
        self.ops: List[Op] = []
        # channel type -> list of rank-level channel ids, in first-use order
        self.channels: Dict[ChannelType, List[int]] = {}
        # access channel type -> list of rank-level remote-buffer ids, in first-use order
        self.remote_refs: Dict[ChannelType, List[int]] = {}

    def channel_slot(self, channel_type: ChannelType, channel_id: int) -> int:
        ids = self.channels.setdefault(channel_type, [])
        if channel_id not in ids:
            ids.append(channel_id)
        return ids.index(channel_id)

    def remote_slot(self, access: ChannelType, remote_buffer_id: int) -> int:
        ids = self.remote_refs.setdefault(access, [])
        if remote_buffer_id not in ids:
            ids.append(remote_buffer_id)
        return ids.index(remote_buffer_id)

    def to_dict(self) -> dict:
        return {
            "id": self.id,
            "ops": [op.to_dict() for op in self.ops],
            "channels": [{"channel_type": t.value, "channel_ids": ids} for t, ids in self.channels.items() if ids],
            "remote_buffer_refs": [{"access_channel_type": t.value, "remote_buffer_ids": ids}
                                   for t, ids in self.remote_refs.items()],
        }


class RankState:
    def __init__(self, rank: int, input_chunks: int, output_chunks: int):
        self.id = rank
        self.input_chunks = input_chunks
        self.output_chunks = output_chunks
        self.scratch_chunks = 0
        self.threadblocks: List[ThreadBlockState] = []
        self.connected: Dict[ChannelType, List[int]] = {}    # memory/port: peer rank per channel id
        self.switch_channels: List[dict] = []                 # {"buffer_type", "rank_group"}
        self.remote_buffers: Dict[tuple, dict] = {}           # (remote rank, buffer type) -> {"id", "access"}
        self.semaphores: List[int] = []
        self.barriers: Dict[tuple, int] = {}

    # ------------------------------------------------------------------ building
    def tb(self, tb_id: int) -> ThreadBlockState:
        while len(self.threadblocks) <= tb_id:
            self.threadblocks.append(ThreadBlockState(len(self.threadblocks)))
        return self.threadblocks[tb_id]

    def add_peer_channel(self, channel_type: ChannelType, dst_rank: int) -> int:
        peers = self.connected.setdefault(channel_type, [])
        peers.append(dst_rank)
        return len(peers) - 1

    def add_switch_channel(self, buffer_type: BufferType, rank_group: RankGroup) -> int:
        self.switch_channels.append({"buffer_type": buffer_type, "rank_group": rank_group})
        return len(self.switch_channels) - 1

    def remote_buffer_slot(self, tb_id: int, remote_rank: int, buffer_type: BufferType, access: ChannelType) -> int:
        key = (remote_rank, buffer_type)
        entry = self.remote_buffers.get(key)
        if entry is None:
            entry = {"id": len(self.remote_buffers), "rank": remote_rank, "type": buffer_type, "access": []}
            self.remote_buffers[key] = entry
        if access not in entry["access"]:
            entry["access"].append(access)
        return self.tb(tb_id).remote_slot(access, entry["id"])

    def barrier_id(self, tb_list) -> int:
        key = tuple(tb_list)
        if key not in self.barriers:
            self.barriers[key] = len(self.barriers)
        return self.barriers[key]

    # ------------------------------------------------------------------ passes
    def post_process(self, instr_fusion: bool, auto_sync: bool, instances: int, policy: ReplicationPolicy) -> None:
        for tb in self.threadblocks:
            if instr_fusion:
                tb.ops = passes.fuse(tb.ops)
            tb.ops = passes.insert_data_sync(tb.ops)
            if auto_sync:
                tb.ops = passes.resolve_hazards(tb.ops)
        self._replicate(instances, policy)

    def _replicate(self, instances: int, policy: ReplicationPolicy) -> None:
        self.input_chunks *= instances
        self.output_chunks *= instances
        self.scratch_chunks *= instances
        for t in list(self.connected):
            self.connected[t] = [peer for peer in self.connected[t] for _ in range(instances)]
        self.switch_channels = [ch for ch in self.switch_channels for _ in range(instances)]
        self.semaphores = [s for s in self.semaphores for _ in range(instances)]
        replicated: List[ThreadBlockState] = []
        for tb in self.threadblocks:
            for inst in range(instances):
                clone = copy.deepcopy(tb)
                clone.id = tb.id * instances + inst
                for t in clone.channels:
                    clone.channels[t] = [cid * instances + inst for cid in clone.channels[t]]
                if policy == ReplicationPolicy.interleaved:
                    shift = lambda index, size, inst=inst: index * instances + inst * size  # noqa: E731
                else:
                    shift = lambda index, size: index  # noqa: E731
                for op in clone.ops:
                    passes.replicate_op(op, inst, instances, shift)
                replicated.append(clone)
        self.threadblocks = replicated

    # ------------------------------------------------------------------ JSON
    def to_dict(self) -> dict:
        channels = [{"channel_type": t.value, "connected_to": peers} for t, peers in self.connected.items()]
        channels += [{"channel_type": ChannelType.switch.value, "buffer_type": ch["buffer_type"].value,
                      "rank_groups": [ch["rank_group"].to_dict()]} for ch in self.switch_channels]
        remote = [{"rank": e["rank"], "type": e["type"].value,
                   "access_channel_types": [a.value for a in sorted(e["access"], key=_CHANNEL_ACCESS_ORDER.get)]}
                  for e in self.remote_buffers.values()]
        return {
            "id": self.id,
            "input_chunks": self.input_chunks,
            "output_chunks": self.output_chunks,
            "scratch_chunks": self.scratch_chunks,
            "threadblocks": [tb.to_dict() for tb in self.threadblocks],
            "channels": channels,
            "remote_buffers": remote,
            "semaphores": [{"init_value": v} for v in self.semaphores],
        }
