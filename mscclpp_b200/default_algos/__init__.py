"""Algorithms written in the DSL that ship with the library: single-node all-pairs / NVLS programs and the
hierarchical multi-node ones that `python -m mscclpp_b200 --install` turns into default plans."""
from .multi_node import allgather_multi_nodes, allreduce_multi_nodes, reducescatter_multi_nodes  # noqa: F401
from .single_node import (  # noqa: F401
    ALGORITHMS,
    allgather_allpairs,
    allreduce_allpairs,
    allreduce_allpairs_packet,
    allreduce_nvls,
    alltoall_allpairs,
    build,
    make_spec,
    reducescatter_allpairs,
)

__all__ = ["allgather_multi_nodes", "allreduce_multi_nodes", "reducescatter_multi_nodes", "default_algo_configs", "build", "ALGORITHMS"]


def default_algo_configs():
    """The plans installed by `python -m mscclpp_b200 --install` (same names, ranges and tags as the reference's
    list, python/mscclpp/__main__.py:13-98, plus single-node 8-GPU plans that the B200 executor can run)."""
    from ..language.collectives import AllReduce
    from ..language.utils import AlgoSpec

    configs = []
    for nodes in (2, 4):
        world = 8 * nodes
        for lo, hi, tbg, label in ((1 << 10, 64 << 10, 1, "1K_64K"), (128 << 10, 2 << 20, 4, "128K_2M")):
            name = f"allreduce_{nodes}nodes_{label}"
            configs.append({
                "filename": name + ".json",
                "function": allreduce_multi_nodes,
                "spec": AlgoSpec(name=name, collective=AllReduce(world, 1, True), nranks_per_node=8, world_size=world, in_place=True,
                                 instances=1, protocol="LL", auto_sync=False, num_threads_per_block=1024, reuse_resources=True,
                                 use_double_scratch_buffer=True, min_message_size=lo, max_message_size=hi, tags={"default": 1}),
                "additional_kwargs": {"thread_block_group_size": tbg},
            })
    return configs
