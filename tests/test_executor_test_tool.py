"""The plan runner's host-side parts (sizes, buffer shapes, expected results) and, on a GPU, one emulated run."""
import json

import numpy as np
import pytest

from mscclpp_b200.benchmark import executor_test as et


def test_parse_size():
    assert et.parse_size("4096") == 4096
    assert et.parse_size("32K") == 32 << 10
    assert et.parse_size("1m") == 1 << 20
    assert et.parse_size("2GB") == 2 << 30
    with pytest.raises(ValueError):
        et.parse_size("12X")


def test_buffer_elems():
    assert et.buffer_elems("allreduce", 4096, 8, 2, True) == (2048, 2048)
    assert et.buffer_elems("allgather", 4096, 8, 4, False) == (128, 1024)
    assert et.buffer_elems("allgather", 4096, 8, 4, True) == (1024, 1024)
    assert et.buffer_elems("reducescatter", 4096, 4, 4, False) == (1024, 256)
    assert et.buffer_elems("alltoall", 4100, 8, 4, False) == (1024, 1024)  # rounded down to a multiple of the world size
    with pytest.raises(ValueError):
        et.buffer_elems("allreduce", 8, 8, 4, True)


def test_expected_outputs_follow_the_plan():
    from mscclpp_b200.default_algos import single_node

    world, per = 4, 64
    plan = single_node.build("allreduce_allpairs", world).to_json()
    assert json.loads(plan)["collective"] == "allreduce"
    ins = et.make_inputs(world, world * per, np.int32)
    assert not np.array_equal(ins[0], ins[1])  # every rank its own data
    out = et.expected_outputs(plan, ins, world * per, in_place=True)
    total = sum(a.astype(np.int64) for a in ins).astype(np.int32)
    assert all(et.matches(o, total) for o in out)
    assert not et.matches(out[0] + 1, total)
    rs = single_node.build("reducescatter_allpairs", world).to_json()
    out = et.expected_outputs(rs, ins, per, in_place=False)
    assert all(et.matches(out[r], total[r * per:(r + 1) * per]) for r in range(world))
    fl = et.make_inputs(2, 16, np.float16)
    assert et.matches(fl[0], fl[0] + np.float16(1e-3)) and not et.matches(fl[0], fl[0] + np.float16(0.5))


@pytest.mark.gpu
def test_emulated_run_on_one_gpu(tmp_path, capsys):
    from mscclpp_b200.default_algos import single_node

    path = tmp_path / "rs.json"
    path.write_text(single_node.build("reducescatter_allpairs", 4).to_json())
    rc = et.main(["-path", str(path), "--size", "64K", "--dtype", "float32", "--emulate", "--n_iters", "4", "--n_graph_iters", "2"])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["correct"] and line["world"] == 4 and line["us_per_execution"] > 0
    path2 = tmp_path / "ar.json"
    path2.write_text(single_node.build("allreduce_allpairs", 2).to_json())
    rc = et.main(["-path", str(path2), "--size", "32K", "--dtype", "float16", "--emulate", "--in_place"])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["correct"] and line["us_per_execution"] is None
