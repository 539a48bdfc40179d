"""Hierarchical multi-node collectives in the DSL, LL (packet) protocol.

Ranks are numbered node-major: rank = node * G + g with G GPUs per node. GPUs of one node talk through
memory channels (NVLink), GPUs with the same local index g on different nodes through port channels (a NIC
driven by the host proxy). All three programs carry data as LL packets in scratch buffers, so no separate
signal/wait pairs are needed: a consumer that unpacks or reduces packets waits for their flags.

The reference ships the same three algorithms (python/mscclpp/default_algos/allreduce_multi_nodes.py:16-221,
allgather_multi_nodes.py:13-200, reducescatter_multi_nodes.py:14-190).
"""
from __future__ import annotations

from ..language.channel import MemoryChannel, PortChannel
from ..language.collectives import AllGather, AllReduce, ReduceScatter
from ..language.program import CollectiveProgram
from ..language.rank import Buffer, Rank
from ..language.thread_block_group import ThreadBlockGroup
from ..language.utils import AlgoSpec

__all__ = ["allreduce_multi_nodes", "allgather_multi_nodes", "reducescatter_multi_nodes"]


class _Topology:
    """Node-major rank arithmetic plus the two channel families."""

    def __init__(self, spec: AlgoSpec):
        if spec.world_size % spec.nranks_per_node != 0:
            raise ValueError("world_size must be divisible by nranks_per_node")
        if spec.protocol != "LL":
            raise ValueError("the multi-node default algorithms use protocol='LL'")
        self.G = spec.nranks_per_node
        self.N = spec.world_size // spec.nranks_per_node
        self.world = spec.world_size

    def rank(self, node: int, g: int) -> int:
        return node * self.G + g

    def split(self, rank: int):
        return divmod(rank, self.G)

    def local_peers(self, rank: int):
        node, g = self.split(rank)
        return [self.rank(node, (g + i) % self.G) for i in range(1, self.G)]

    def remote_peers(self, rank: int):
        node, g = self.split(rank)
        return [self.rank((node + i) % self.N, g) for i in range(1, self.N)]

    def open_channels(self):
        """Call inside the program context. (src, dst) -> channel that src uses to reach dst."""
        self.mem = {}
        self.port = {}
        for src in range(self.world):
            for dst in self.local_peers(src):
                self.mem[(src, dst)] = MemoryChannel(dst, src)
            for dst in self.remote_peers(src):
                self.port[(src, dst)] = PortChannel(dst, src)


def _peer_groups(G: int, size: int, first_tb: int = 1):
    """One thread-block group per local peer slot plus one group over all of them."""
    groups = [ThreadBlockGroup(tb_list=list(range(first_tb + i * size, first_tb + (i + 1) * size))) for i in range(G - 1)]
    everyone = ThreadBlockGroup(tb_list=list(range(first_tb, first_tb + (G - 1) * size)))
    return groups, everyone


def _slot_of(peer_g: int, my_g: int) -> int:
    """Index of local peer `peer_g` among the G-1 peers of `my_g`."""
    return peer_g if peer_g < my_g else peer_g - 1


def allreduce_multi_nodes(spec: AlgoSpec, thread_block_group_size: int = 1) -> CollectiveProgram:
    """In-place allreduce over N nodes x G GPUs.

    The input is cut into G sections of N chunks; section g belongs to the GPUs with local index g.
      1. inside the node: send every peer its section as packets, reduce my section over the G-1 arrivals;
      2. across nodes: send my node-reduced section to the N-1 GPUs with my local index, reduce again;
      3. inside the node: forward the finished section to the local peers, unpack the G-1 finished sections
         that arrive.
    Scratch layout per rank (in chunks): [0, W) arrivals of step 1, [W, W + N*N) arrivals of step 2 and my own
    packed section, then the arrivals of step 3."""
    if not isinstance(spec.collective, AllReduce):
        raise ValueError("allreduce_multi_nodes requires an AllReduce collective")
    if thread_block_group_size <= 0:
        raise ValueError("thread_block_group_size must be positive")
    topo = _Topology(spec)
    G, N, W = topo.G, topo.N, topo.world
    sect = N                       # chunks per section
    stage2 = W                     # first chunk of the step-2 area
    stage3 = W + sect * N          # first chunk of the step-3 area
    with CollectiveProgram.from_spec(spec) as prog:
        topo.open_channels()
        scratch = [Buffer(r, 2 * W + sect * N) for r in range(W)]
        groups, everyone = _peer_groups(G, thread_block_group_size)
        all_tbs = list(range(1 + (G - 1) * thread_block_group_size))
        for me in range(W):
            node, g = topo.split(me)
            rank = Rank(me)
            inp = rank.get_input_buffer()
            mine = inp[g * sect:(g + 1) * sect]
            # 1. intra-node scatter + reduce
            for p in range(G):
                if p == g:
                    continue
                peer = topo.rank(node, p)
                topo.mem[(me, peer)].put_packets(scratch[peer][g * sect:(g + 1) * sect], inp[p * sect:(p + 1) * sect],
                                                 tb_group=groups[_slot_of(p, g)])
            rank.reduce(mine, [scratch[me][p * sect:(p + 1) * sect] for p in range(G) if p != g], tb_group=everyone, packet=True)
            rank.copy_packets(scratch[me][g * sect:(g + 1) * sect], mine, tb_group=everyone)
            rank.barrier(tb_list=all_tbs)
            # 2. inter-node exchange + reduce (thread block 0 talks to the proxy)
            for other in range(N):
                if other == node:
                    continue
                peer = topo.rank(other, g)
                topo.port[(me, peer)].put_packets(scratch[peer][stage2 + node * sect:stage2 + (node + 1) * sect],
                                                  scratch[me][g * sect:(g + 1) * sect], tb=0)
            if N > 1:
                rank.reduce(mine, [scratch[me][stage2 + o * sect:stage2 + (o + 1) * sect] for o in range(N) if o != node],
                            tb_group=everyone, packet=True)
            rank.copy_packets(scratch[me][stage2 + node * sect:stage2 + (node + 1) * sect], mine, tb_group=everyone)
            # 3. intra-node broadcast of the finished section
            for p in range(G):
                if p == g:
                    continue
                peer = topo.rank(node, p)
                topo.mem[(me, peer)].read_put_packets(scratch[peer][stage3 + g * sect:stage3 + (g + 1) * sect],
                                                      scratch[me][stage2 + node * sect:stage2 + (node + 1) * sect],
                                                      tb_group=groups[_slot_of(p, g)])
            for p in range(G):
                if p == g:
                    continue
                rank.unpack_packets(inp[p * sect:(p + 1) * sect], scratch[me][stage3 + p * sect:stage3 + (p + 1) * sect],
                                    tb_group=groups[_slot_of(p, g)])
    return prog


def allgather_multi_nodes(spec: AlgoSpec) -> CollectiveProgram:
    """Allgather over N nodes x G GPUs (chunk_factor 1).

      1. my chunk goes as packets to the G-1 local peers and, through the NIC, to the N-1 GPUs with my local
         index;
      2. every chunk that arrived from another node is forwarded, still as packets, to the G-1 local peers;
      3. all arrivals are unpacked into the output.
    Scratch layout per rank (in chunks): [0, G) local arrivals by sender's local index, [G, G+N) my packed chunk
    at [G + my node] and remote arrivals by sender's node, [G+N, G+N+G*N) forwarded chunks by (node, local)."""
    if not isinstance(spec.collective, AllGather):
        raise ValueError("allgather_multi_nodes requires an AllGather collective")
    if spec.collective.chunk_factor != 1:
        raise ValueError("allgather_multi_nodes requires chunk_factor=1")
    if spec.in_place != spec.collective.inplace:
        raise ValueError("spec.in_place must match spec.collective.inplace")
    topo = _Topology(spec)
    G, N, W = topo.G, topo.N, topo.world
    remote0 = G
    fwd0 = G + N
    with CollectiveProgram.from_spec(spec) as prog:
        topo.open_channels()
        scratch = [Buffer(r, G + N + G * N) for r in range(W)]
        for me in range(W):
            node, g = topo.split(me)
            rank = Rank(me)
            out = rank.get_output_buffer()
            if spec.in_place:
                src = out[me:me + 1]
            else:
                src = rank.get_input_buffer()[0:1]
                rank.copy(out[me:me + 1], src, tb=0)
            # 1. my chunk to local peers (one thread block per peer) and to the other nodes (thread block 0)
            for p in range(G):
                if p != g:
                    topo.mem[(me, topo.rank(node, p))].put_packets(scratch[topo.rank(node, p)][g:g + 1], src, tb=1 + _slot_of(p, g))
            if N > 1:
                rank.copy_packets(scratch[me][remote0 + node:remote0 + node + 1], src, tb=0)
                for other in range(N):
                    if other != node:
                        peer = topo.rank(other, g)
                        topo.port[(me, peer)].read_put_packets(scratch[peer][remote0 + node:remote0 + node + 1],
                                                               scratch[me][remote0 + node:remote0 + node + 1], tb=0)
        for me in range(W):
            node, g = topo.split(me)
            rank = Rank(me)
            out = rank.get_output_buffer()
            # 2. forward remote arrivals to local peers
            for other in range(N):
                if other == node:
                    continue
                for p in range(G):
                    if p != g:
                        peer = topo.rank(node, p)
                        topo.mem[(me, peer)].read_put_packets(scratch[peer][fwd0 + other * G + g:fwd0 + other * G + g + 1],
                                                              scratch[me][remote0 + other:remote0 + other + 1], tb=1 + _slot_of(p, g))
            # 3. unpack everything
            for p in range(G):
                if p != g:
                    rank.unpack_packets(out[topo.rank(node, p):topo.rank(node, p) + 1], scratch[me][p:p + 1], tb=1 + _slot_of(p, g))
            for other in range(N):
                if other == node:
                    continue
                rank.unpack_packets(out[topo.rank(other, g):topo.rank(other, g) + 1], scratch[me][remote0 + other:remote0 + other + 1], tb=0)
                for p in range(G):
                    if p != g:
                        rank.unpack_packets(out[topo.rank(other, p):topo.rank(other, p) + 1],
                                            scratch[me][fwd0 + other * G + p:fwd0 + other * G + p + 1], tb=1 + _slot_of(p, g))
    return prog


def reducescatter_multi_nodes(spec: AlgoSpec, thread_block_group_size: int = 1) -> CollectiveProgram:
    """In-place reduce-scatter over N nodes x G GPUs (chunk_factor 1): rank r ends with chunk r reduced over all
    ranks, in input[r].

      1. inside the node: for every node m, chunk (m, p) goes as packets to local peer p, who reduces the G
         contributions of its node into its own copy of chunk (m, g);
      2. across nodes: the node-reduced chunk (m, g) goes through the NIC to its owner, rank (m, g), who reduces
         the N-1 arrivals into input[r].
    Scratch layout per rank (in chunks): [0, G*N) step-1 arrivals by (sender's local index, node of the chunk),
    [G*N, G*N + N) my packed partial sums by destination node, then N step-2 arrivals by sender's node."""
    if not isinstance(spec.collective, ReduceScatter):
        raise ValueError("reducescatter_multi_nodes requires a ReduceScatter collective")
    if spec.collective.chunk_factor != 1:
        raise ValueError("reducescatter_multi_nodes requires chunk_factor=1")
    if not spec.in_place or not spec.collective.inplace:
        raise ValueError("reducescatter_multi_nodes requires in-place buffers")
    if thread_block_group_size <= 0:
        raise ValueError("thread_block_group_size must be positive")
    topo = _Topology(spec)
    G, N, W = topo.G, topo.N, topo.world
    packed0 = G * N
    arrive0 = G * N + N
    with CollectiveProgram.from_spec(spec) as prog:
        topo.open_channels()
        scratch = [Buffer(r, G * N + 2 * N) for r in range(W)]
        groups, everyone = _peer_groups(G, thread_block_group_size)
        all_tbs = list(range(1 + (G - 1) * thread_block_group_size))
        for me in range(W):
            node, g = topo.split(me)
            inp = Rank(me).get_input_buffer()
            for p in range(G):
                if p == g:
                    continue
                peer = topo.rank(node, p)
                for m in range(N):
                    c = topo.rank(m, p)
                    topo.mem[(me, peer)].put_packets(scratch[peer][g * N + m:g * N + m + 1], inp[c:c + 1], tb_group=groups[_slot_of(p, g)])
        for me in range(W):
            node, g = topo.split(me)
            rank = Rank(me)
            inp = rank.get_input_buffer()
            for m in range(N):
                c = topo.rank(m, g)
                if G > 1:
                    rank.reduce(inp[c:c + 1], [scratch[me][p * N + m:p * N + m + 1] for p in range(G) if p != g], tb_group=everyone,
                                packet=True)
                if m != node:
                    rank.copy_packets(scratch[me][packed0 + m:packed0 + m + 1], inp[c:c + 1], tb_group=everyone)
            if N > 1:
                rank.barrier(tb_list=all_tbs)
                for m in range(N):
                    if m == node:
                        continue
                    owner = topo.rank(m, g)
                    topo.port[(me, owner)].read_put_packets(scratch[owner][arrive0 + node:arrive0 + node + 1],
                                                            scratch[me][packed0 + m:packed0 + m + 1], tb=0)
                rank.reduce(inp[me:me + 1], [scratch[me][arrive0 + o:arrive0 + o + 1] for o in range(N) if o != node],
                            tb_group=everyone, packet=True)
    return prog
