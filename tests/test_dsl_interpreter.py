"""CPU-only: DSL programs compile to plans that the numpy interpreter executes correctly."""
import json

import numpy as np
import pytest

from mscclpp_b200.default_algos import single_node
from mscclpp_b200.language.interpreter import Deadlock, PlanError, PlanInterpreter, validate_plan


def _inputs(n, elems, dtype, seed=0):
    out = []
    for r in range(n):
        rng = np.random.default_rng(seed + r)
        out.append(rng.uniform(-1, 1, size=elems).astype(dtype))
    return out


def test_allpairs_allreduce_8_ranks_fp16_1mib():
    """8-rank all-pairs allreduce (sum, fp16, 1 MiB per rank), inputs Uniform[-1,1] seeded by rank,
    checked against the fp32-accumulated sum cast to fp16."""
    n, elems = 8, (1 << 20) // 2
    plan = single_node.build("allreduce_allpairs", n).to_json()
    validate_plan(plan)
    data = _inputs(n, elems, np.float16)
    expect = np.sum(np.stack([d.astype(np.float32) for d in data]), axis=0).astype(np.float16)
    out = PlanInterpreter(plan).run([d.copy() for d in data])
    for r in range(n):
        np.testing.assert_allclose(out[r].astype(np.float32), expect.astype(np.float32), atol=1e-2, rtol=0)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("instances", [1, 2])
@pytest.mark.parametrize("algo", ["allreduce_allpairs", "allreduce_allpairs_packet", "allreduce_nvls"])
def test_allreduce_algorithms(n, instances, algo):
    plan = single_node.build(algo, n, instances=instances).to_dict()
    validate_plan(plan)
    elems = 8 * n * instances * 12
    data = _inputs(n, elems, np.float32, seed=3)
    expect = np.sum(np.stack(data), axis=0)
    out = PlanInterpreter(plan).run([d.copy() for d in data])
    for r in range(n):
        np.testing.assert_allclose(out[r], expect, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n", [2, 8])
def test_allgather_reducescatter_alltoall(n):
    per = 64
    # allgather, in place: rank r's contribution sits in slot r of its output
    plan = single_node.build("allgather_allpairs", n, in_place=True).to_dict()
    bufs = [np.zeros(n * per, dtype=np.int32) for _ in range(n)]
    for r in range(n):
        bufs[r][r * per:(r + 1) * per] = np.arange(per) + 1000 * r
    ins = [b[r * per:(r + 1) * per] for r, b in enumerate(bufs)]
    PlanInterpreter(plan).run(ins, bufs)
    expect = np.concatenate([np.arange(per) + 1000 * r for r in range(n)])
    for r in range(n):
        np.testing.assert_array_equal(bufs[r], expect)
    # reduce-scatter
    plan = single_node.build("reducescatter_allpairs", n).to_dict()
    data = _inputs(n, n * per, np.float32, seed=5)
    outs = [np.zeros(per, dtype=np.float32) for _ in range(n)]
    PlanInterpreter(plan).run([d.copy() for d in data], outs)
    total = np.sum(np.stack(data), axis=0)
    for r in range(n):
        np.testing.assert_allclose(outs[r], total[r * per:(r + 1) * per], rtol=1e-5, atol=1e-5)
    # all-to-all
    plan = single_node.build("alltoall_allpairs", n).to_dict()
    data = [np.arange(n * per, dtype=np.int32) + 100000 * r for r in range(n)]
    outs = [np.zeros(n * per, dtype=np.int32) for _ in range(n)]
    PlanInterpreter(plan).run(data, outs)
    for r in range(n):
        for p in range(n):
            np.testing.assert_array_equal(outs[r][p * per:(p + 1) * per], data[p][r * per:(r + 1) * per])


def test_uneven_message_size_uses_aligned_split():
    n = 4
    plan = single_node.build("allreduce_allpairs", n).to_dict()
    elems = (16 * 7) // 4  # 7 alignment units over 4 chunks: chunk sizes 2,2,2,1 units
    data = _inputs(n, elems, np.float32, seed=9)
    out = PlanInterpreter(plan).run([d.copy() for d in data])
    np.testing.assert_allclose(out[2], np.sum(np.stack(data), axis=0), rtol=1e-5, atol=1e-5)


def test_validator_rejects_bad_plans():
    plan = single_node.build("allreduce_allpairs", 2).to_dict()
    bad = json.loads(json.dumps(plan))
    bad["gpus"][0]["threadblocks"][0]["ops"].append({"name": "frobnicate"})
    with pytest.raises(PlanError):
        validate_plan(bad)
    bad = json.loads(json.dumps(plan))
    for op in bad["gpus"][0]["threadblocks"][0]["ops"]:
        if op["name"] in ("rres", "rre", "put"):
            op["src_buff"][0]["index"] = 99
            break
    with pytest.raises(PlanError):
        validate_plan(bad)
    # drop a wait: signals no longer pair up
    bad = json.loads(json.dumps(plan))
    ops = bad["gpus"][1]["threadblocks"][0]["ops"]
    idx = max(i for i, op in enumerate(ops) if op["name"] == "wait")
    del ops[idx]
    with pytest.raises(PlanError):
        validate_plan(bad)


def test_missing_signal_is_a_deadlock_not_a_hang():
    plan = single_node.build("allreduce_allpairs", 2).to_dict()
    ops = plan["gpus"][0]["threadblocks"][0]["ops"]
    idx = next(i for i, op in enumerate(ops) if op["name"] in ("signal", "rlxsignal"))
    del ops[idx]
    data = _inputs(2, 64, np.float32)
    with pytest.raises(Deadlock):
        PlanInterpreter(plan).run(data)
