"""CPU-only: the hierarchical multi-node DSL algorithms produce plans that the numpy interpreter executes
correctly, for several (nodes, GPUs per node) shapes, and the installer writes the default plans."""
import json

import numpy as np
import pytest

from mscclpp_b200.default_algos import allgather_multi_nodes, allreduce_multi_nodes, default_algo_configs, reducescatter_multi_nodes
from mscclpp_b200.language.collectives import AllGather, AllReduce, ReduceScatter
from mscclpp_b200.language.interpreter import PlanInterpreter, validate_plan
from mscclpp_b200.language.utils import AlgoSpec

SHAPES = [(2, 2), (2, 4), (3, 2), (4, 2), (1, 4)]


def _spec(name, collective, nodes, gpus, in_place=True, **kw):
    return AlgoSpec(name=name, collective=collective, nranks_per_node=gpus, world_size=nodes * gpus, in_place=in_place, instances=1,
                    protocol="LL", auto_sync=False, num_threads_per_block=1024, reuse_resources=True, use_double_scratch_buffer=True,
                    **kw)


@pytest.mark.parametrize("nodes,gpus", SHAPES)
@pytest.mark.parametrize("tbg", [1, 2])
def test_allreduce_multi_nodes(nodes, gpus, tbg):
    w = nodes * gpus
    plan = allreduce_multi_nodes(_spec("ar_mn", AllReduce(w, 1, True), nodes, gpus), thread_block_group_size=tbg).to_dict()
    validate_plan(plan)
    elems = w * nodes * 24
    data = [np.random.default_rng(r).uniform(-1, 1, elems).astype(np.float32) for r in range(w)]
    expect = np.sum(np.stack(data), axis=0)
    out = PlanInterpreter(plan).run([d.copy() for d in data])
    for r in range(w):
        np.testing.assert_allclose(out[r], expect, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("nodes,gpus", SHAPES)
@pytest.mark.parametrize("in_place", [True, False])
def test_allgather_multi_nodes(nodes, gpus, in_place):
    w = nodes * gpus
    plan = allgather_multi_nodes(_spec("ag_mn", AllGather(w, 1, in_place), nodes, gpus, in_place=in_place)).to_dict()
    validate_plan(plan)
    per = 48
    expect = np.concatenate([np.arange(per, dtype=np.int32) + 1000 * r for r in range(w)])
    outs = [np.zeros(w * per, dtype=np.int32) for _ in range(w)]
    if in_place:
        for r in range(w):
            outs[r][r * per:(r + 1) * per] = expect[r * per:(r + 1) * per]
        ins = [o[r * per:(r + 1) * per] for r, o in enumerate(outs)]
    else:
        ins = [expect[r * per:(r + 1) * per].copy() for r in range(w)]
    PlanInterpreter(plan).run(ins, outs)
    for r in range(w):
        np.testing.assert_array_equal(outs[r], expect)


@pytest.mark.parametrize("nodes,gpus", SHAPES)
@pytest.mark.parametrize("tbg", [1, 2])
def test_reducescatter_multi_nodes(nodes, gpus, tbg):
    w = nodes * gpus
    plan = reducescatter_multi_nodes(_spec("rs_mn", ReduceScatter(w, 1, True), nodes, gpus), thread_block_group_size=tbg).to_dict()
    validate_plan(plan)
    per = 40
    data = [np.random.default_rng(10 + r).uniform(-1, 1, w * per).astype(np.float32) for r in range(w)]
    total = np.sum(np.stack(data), axis=0)
    bufs = [d.copy() for d in data]
    outs = [b[r * per:(r + 1) * per] for r, b in enumerate(bufs)]
    PlanInterpreter(plan).run(bufs, outs)
    for r in range(w):
        np.testing.assert_allclose(bufs[r][r * per:(r + 1) * per], total[r * per:(r + 1) * per], rtol=1e-5, atol=1e-5)


def test_bad_specs_are_rejected():
    with pytest.raises(ValueError):
        allreduce_multi_nodes(_spec("x", AllGather(4, 1, True), 2, 2))
    with pytest.raises(ValueError):
        reducescatter_multi_nodes(_spec("x", ReduceScatter(4, 1, False), 2, 2, in_place=False))
    with pytest.raises(ValueError):
        allreduce_multi_nodes(_spec("x", AllReduce(4, 1, True), 2, 2), thread_block_group_size=0)


def test_install_writes_default_plans(tmp_path, monkeypatch):
    from mscclpp_b200.__main__ import create_default_plans

    written = create_default_plans(tmp_path / "default", verbose=False)
    assert len(written) == len(default_algo_configs()) == 4
    plan = json.loads(written[0].read_text())
    assert plan["name"] == "allreduce_2nodes_1K_64K"
    assert plan["min_message_size"] == 1 << 10 and plan["max_message_size"] == 64 << 10
    assert len(plan["gpus"]) == 16
