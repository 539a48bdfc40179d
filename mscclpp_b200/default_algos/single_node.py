"""Single-node algorithms written in the DSL. Each function takes an AlgoSpec and returns the
CollectiveProgram (call .to_json() for the plan). They double as the library's DSL examples and as
the CPU-verifiable reference for the native kernels of the same shape."""
from __future__ import annotations

from ..language.channel import MemoryChannel, SwitchChannel
from ..language.collectives import AllGather, AllReduce, AllToAll, ReduceScatter
from ..language.program import CollectiveProgram
from ..language.rank import Buffer, Rank
from ..language.types import BufferType, SyncType
from ..language.utils import AlgoSpec


def make_spec(name: str, collective, world_size: int, protocol: str = "Simple", instances: int = 1, in_place: bool = True,
              **kwargs) -> AlgoSpec:
    return AlgoSpec(name=name, collective=collective, nranks_per_node=world_size, world_size=world_size, in_place=in_place,
                    instances=instances, protocol=protocol, **kwargs)


def _peers(rank: int, n: int):
    return [(rank + i) % n for i in range(1, n)]


def allreduce_allpairs(spec: AlgoSpec) -> CollectiveProgram:
    """Two-shot, zero-copy, in place: rank r reduces chunk r by reading it from every peer's input,
    then writes the result back into every peer's input. One thread block per peer pair would waste
    SMs on NVSwitch, so all peers of a rank share one thread block per instance."""
    n = spec.world_size
    prog = CollectiveProgram.from_spec(spec)
    with prog:
        chan = {(src, dst): MemoryChannel(dst, src) for src in range(n) for dst in range(n) if src != dst}
        # everybody's input is ready
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.none, relaxed=True)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after, relaxed=True)
        for r in range(n):
            mine = Rank(r).get_input_buffer()[r:r + 1]
            for p in _peers(r, n):
                chan[(r, p)].reduce(mine, [Rank(p).get_input_buffer()[r:r + 1]], tb=0)
            for p in _peers(r, n):
                chan[(r, p)].put(Rank(p).get_input_buffer()[r:r + 1], mine, tb=0)
        # results have landed everywhere
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.before)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after)
    return prog


def allreduce_allpairs_packet(spec: AlgoSpec) -> CollectiveProgram:
    """One-shot LL: every rank sends its whole input to every peer's scratch as packets, then reduces
    its input with the n-1 packet streams. No signals; flags travel with the data."""
    n = spec.world_size
    prog = CollectiveProgram.from_spec(spec)
    with prog:
        scratch = [Buffer(r, n * n) for r in range(n)]  # slot [src * n + chunk]
        chan = {(src, dst): MemoryChannel(dst, src) for src in range(n) for dst in range(n) if src != dst}
        for r in range(n):
            inp = Rank(r).get_input_buffer()
            for p in _peers(r, n):
                chan[(r, p)].put_packets(scratch[p][r * n:(r + 1) * n], inp[0:n], tb=0)
        for r in range(n):
            rank = Rank(r)
            inp = rank.get_input_buffer()
            rank.reduce(inp[0:n], [scratch[r][p * n:(p + 1) * n] for p in _peers(r, n)], tb=0, packet=True)
    return prog


def allgather_allpairs(spec: AlgoSpec) -> CollectiveProgram:
    """Every rank puts its input chunk into slot `rank` of every peer's output."""
    n = spec.world_size
    prog = CollectiveProgram.from_spec(spec)
    with prog:
        chan = {(src, dst): MemoryChannel(dst, src) for src in range(n) for dst in range(n) if src != dst}
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.none, relaxed=True)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after, relaxed=True)
        for r in range(n):
            rank = Rank(r)
            src = rank.get_input_buffer()[0:1] if not spec.in_place else rank.get_output_buffer()[r:r + 1]
            if not spec.in_place:
                rank.copy(rank.get_output_buffer()[r:r + 1], src, tb=0)
            for p in _peers(r, n):
                chan[(r, p)].put(Rank(p).get_output_buffer()[r:r + 1], src, tb=0)
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.before)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after)
    return prog


def reducescatter_allpairs(spec: AlgoSpec) -> CollectiveProgram:
    """Rank r reads chunk r of every peer's input and leaves the sum in its output."""
    n = spec.world_size
    prog = CollectiveProgram.from_spec(spec)
    with prog:
        chan = {(src, dst): MemoryChannel(dst, src) for src in range(n) for dst in range(n) if src != dst}
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.none, relaxed=True)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after, relaxed=True)
        for r in range(n):
            rank = Rank(r)
            mine = rank.get_input_buffer()[r:r + 1]
            out = rank.get_output_buffer()[0:1]
            for p in _peers(r, n):
                chan[(r, p)].reduce(mine, [Rank(p).get_input_buffer()[r:r + 1]], tb=0, local_dst_chunk=out)
        # nobody may overwrite its input before every peer has read it
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.before)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after)
    return prog


def alltoall_allpairs(spec: AlgoSpec) -> CollectiveProgram:
    """Chunk p of rank r's input lands in chunk r of rank p's output."""
    n = spec.world_size
    prog = CollectiveProgram.from_spec(spec)
    with prog:
        chan = {(src, dst): MemoryChannel(dst, src) for src in range(n) for dst in range(n) if src != dst}
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.none, relaxed=True)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after, relaxed=True)
        for r in range(n):
            rank = Rank(r)
            rank.copy(rank.get_output_buffer()[r:r + 1], rank.get_input_buffer()[r:r + 1], tb=0)
            for p in _peers(r, n):
                chan[(r, p)].put(Rank(p).get_output_buffer()[r:r + 1], rank.get_input_buffer()[p:p + 1], tb=0)
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.before)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after)
    return prog


def allreduce_nvls(spec: AlgoSpec) -> CollectiveProgram:
    """In-place allreduce through the NVSwitch: rank r multimem-load-reduces chunk r and multimem-stores
    it back; peer barriers before and after."""
    n = spec.world_size
    prog = CollectiveProgram.from_spec(spec)
    with prog:
        switch = SwitchChannel(list(range(n)), BufferType.input)
        chan = {(src, dst): MemoryChannel(dst, src) for src in range(n) for dst in range(n) if src != dst}
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.none, relaxed=True)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after, relaxed=True)
        for r in range(n):
            mine = Rank(r).get_input_buffer()[r:r + 1]
            switch.at_rank(r).reduce(buffer_offset=r, size=1, dst_chunk=mine, tb=0)
            switch.at_rank(r).broadcast(src_chunk=mine, buffer_offset=r, size=1, tb=0)
        for r in range(n):
            for p in _peers(r, n):
                chan[(r, p)].signal(tb=0, data_sync=SyncType.before)
            for p in _peers(r, n):
                chan[(r, p)].wait(tb=0, data_sync=SyncType.after)
    return prog


ALGORITHMS = {
    "allreduce_allpairs": (allreduce_allpairs, AllReduce, "Simple"),
    "allreduce_allpairs_packet": (allreduce_allpairs_packet, AllReduce, "LL"),
    "allreduce_nvls": (allreduce_nvls, AllReduce, "Simple"),
    "allgather_allpairs": (allgather_allpairs, AllGather, "Simple"),
    "reducescatter_allpairs": (reducescatter_allpairs, ReduceScatter, "Simple"),
    "alltoall_allpairs": (alltoall_allpairs, AllToAll, "Simple"),
}


def build(name: str, world_size: int, instances: int = 1, in_place: bool = True, **kwargs) -> CollectiveProgram:
    fn, coll, protocol = ALGORITHMS[name]
    if name in ("alltoall_allpairs", "reducescatter_allpairs"):
        in_place = False
    collective = coll(world_size, 1, in_place)
    spec = make_spec(name, collective, world_size, protocol=protocol, instances=instances, in_place=in_place, **kwargs)
    return fn(spec)
