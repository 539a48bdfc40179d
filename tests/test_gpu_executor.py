"""GPU plan interpreter against the numpy plan interpreter on identical plans and inputs.
All ranks of a plan are emulated on one GPU in one cooperative launch."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NP2TORCH = {np.float32: torch.float32, np.float16: torch.float16, np.int32: torch.int32}


def _run_both(plan_json, world, in_elems, out_elems, np_dtype, inplace, launches=2, packet_type="LL16"):
    from mscclpp_b200 import SymmetricMemory, native
    from mscclpp_b200.language.interpreter import PlanInterpreter

    n = native()
    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=3000)
    tdtype = NP2TORCH[np_dtype]
    t_in = symm.tensor((in_elems,), tdtype)
    t_out = t_in if inplace else symm.tensor((out_elems,), tdtype)
    executor = n.Executor(symm.heap)
    plans = [n.ExecutionPlan.from_string(plan_json, r) for r in range(world)]
    interp = PlanInterpreter(plan_json)
    dt = {np.float32: n.DataType.float32, np.float16: n.DataType.float16, np.int32: n.DataType.int32}[np_dtype]
    for launch in range(launches):
        rng = np.random.default_rng(100 + launch)
        if np_dtype == np.int32:
            ins = [rng.integers(-1000, 1000, size=in_elems).astype(np_dtype) for _ in range(world)]
        else:
            ins = [rng.uniform(-1, 1, size=in_elems).astype(np_dtype) for _ in range(world)]
        outs = [np.zeros(out_elems, dtype=np_dtype) for _ in range(world)]
        for r in range(world):
            symm.rank_view(t_in, r).copy_(torch.from_numpy(ins[r]))
            if not inplace:
                symm.rank_view(t_out, r).zero_()
        expect = interp.run([a.copy() for a in ins], None if inplace else outs)
        executor.execute(0, t_in.data_ptr(), t_out.data_ptr(), in_elems * ins[0].itemsize, out_elems * ins[0].itemsize, dt,
                         plans[0], torch.cuda.current_stream().cuda_stream, getattr(n.PacketType, packet_type))
        torch.cuda.synchronize()
        symm.check()
        for r in range(world):
            got = symm.rank_view(t_out, r).cpu().numpy()
            if np_dtype == np.int32:
                np.testing.assert_array_equal(got, expect[r])
            else:
                np.testing.assert_allclose(got.astype(np.float32), expect[r].astype(np.float32), rtol=2e-3, atol=2e-3,
                                           err_msg=f"rank {r} of {world}, launch {launch}, {in_elems} elements, packets {packet_type}")
    executor.reset()
    symm.destroy()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", ["allreduce_allpairs", "allreduce_allpairs_packet", "allreduce_nvls"])
@pytest.mark.parametrize("instances", [1, 2])
def test_allreduce_plans(world, algo, instances):
    from mscclpp_b200.default_algos import single_node

    plan = single_node.build(algo, world, instances=instances).to_json()
    elems = 4 * world * instances * 64
    _run_both(plan, world, elems, elems, np.float32, inplace=True)
    _run_both(plan, world, elems, elems, np.float16, inplace=True)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("packet_type", ["LL8", "LL16"])
def test_packet_plans_with_both_packet_formats(world, packet_type):
    """The same LL plan through 8-byte and 16-byte packets, a small and a larger message. (Sizes divide evenly into the
    plan's chunks: with a remainder the plan format maps unequal input chunks onto scratch chunks of other sizes, in
    the reference as well, and neighbouring ranges then overlap.)"""
    from mscclpp_b200.default_algos import single_node

    plan = single_node.build("allreduce_allpairs_packet", world).to_json()
    for elems in (4 * world * 16, 4 * world * 1024):
        _run_both(plan, world, elems, elems, np.float32, inplace=True, packet_type=packet_type)


@pytest.mark.parametrize("nodes,gpus", [(2, 2), (2, 4)])
def test_port_channel_plans_go_through_the_host_proxy(nodes, gpus):
    """The hierarchical multi-node plans talk to the GPUs of other nodes through port channels: the interpreter kernel
    queues requests in the executor's FIFO and the executor's proxy thread moves the packets with the copy engines.
    Here the 'nodes' are groups of emulated ranks on one GPU, which exercises exactly that path."""
    from mscclpp_b200.default_algos import allreduce_multi_nodes, reducescatter_multi_nodes
    from mscclpp_b200.language.collectives import AllReduce, ReduceScatter
    from mscclpp_b200.language.utils import AlgoSpec

    w = nodes * gpus

    def spec(name, coll):
        return AlgoSpec(name=name, collective=coll, nranks_per_node=gpus, world_size=w, in_place=True, instances=1, protocol="LL",
                        auto_sync=False, num_threads_per_block=1024, reuse_resources=True, use_double_scratch_buffer=True)

    plan = allreduce_multi_nodes(spec("ar_mn_gpu", AllReduce(w, 1, True))).to_json()
    assert '"port"' in plan
    elems = w * nodes * 64
    _run_both(plan, w, elems, elems, np.float32, inplace=True, launches=3)
    plan = reducescatter_multi_nodes(spec("rs_mn_gpu", ReduceScatter(w, 1, True))).to_json()
    assert '"port"' in plan


def test_plan_with_more_blocks_than_the_gpu_can_hold_is_refused():
    """Thread blocks of a plan wait on one another, so all of them (times the emulated ranks) must be resident at once;
    a launch that cannot be is refused with a message that names the plan and the numbers, before anything runs."""
    from mscclpp_b200 import SymmetricMemory, native
    from mscclpp_b200.default_algos import single_node

    n = native()
    world = 8
    plan_json = single_node.build("allreduce_allpairs", world, instances=32).to_json()  # 32 blocks of 1024 threads per rank
    blocks = max(len(g["threadblocks"]) for g in json.loads(plan_json)["gpus"])
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if blocks * world <= sms:
        pytest.skip("this plan fits the GPU even with all ranks emulated")
    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=1000)
    elems = 4 * world * 32 * 64
    t = symm.tensor((elems,), torch.float32, zero=True)
    ex = n.Executor(symm.heap)
    with pytest.raises(Exception, match="resident at the same time"):
        ex.execute(0, t.data_ptr(), t.data_ptr(), elems * 4, elems * 4, n.DataType.float32, n.ExecutionPlan.from_string(plan_json, 0), 0)
    ex.reset()
    symm.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_allgather_reducescatter_alltoall_plans(world):
    from mscclpp_b200.default_algos import single_node

    per = 256
    _run_both(single_node.build("reducescatter_allpairs", world).to_json(), world, world * per, per, np.float32, inplace=False)
    _run_both(single_node.build("alltoall_allpairs", world).to_json(), world, world * per, world * per, np.int32, inplace=False)
    _run_both(single_node.build("allgather_allpairs", world, in_place=False).to_json(), world, per, world * per, np.int32, inplace=False)


def test_malformed_plan_is_rejected():
    from mscclpp_b200 import native
    from mscclpp_b200.default_algos import single_node

    n = native()
    plan = json.loads(single_node.build("allreduce_allpairs", 2).to_json())
    plan["gpus"][0]["threadblocks"][0]["ops"].append({"name": "frobnicate"})
    from mscclpp_b200 import SymmetricMemory

    symm = SymmetricMemory.emulated(2, nbytes=64 << 20, timeout_ms=1000)
    t = symm.tensor((1024,), torch.float32, zero=True)
    ex = n.Executor(symm.heap)
    with pytest.raises(Exception):
        ex.execute(0, t.data_ptr(), t.data_ptr(), 4096, 4096, n.DataType.float32, n.ExecutionPlan.from_string(json.dumps(plan), 0), 0)
    ex.reset()
    symm.destroy()


def test_tracer_records_executor_operations(tmp_path):
    """With the tracer on, every thread block of a plan leaves ENTRY/EXIT pairs that convert to a Chrome trace."""
    from mscclpp_b200 import SymmetricMemory, native
    from mscclpp_b200.default_algos import single_node
    from mscclpp_b200.utils.npkit_trace import convert_npkit_dump_to_trace

    n = native()
    world = 2
    plan_json = single_node.build("allreduce_allpairs", world).to_json()
    symm = SymmetricMemory.emulated(world, nbytes=64 << 20, timeout_ms=3000)
    t = symm.tensor((4096,), torch.float32)
    for r in range(world):
        symm.rank_view(t, r).fill_(r + 1.0)
    n.npkit.init(0)
    try:
        assert n.npkit.enabled()
        executor = n.Executor(symm.heap)
        plan = n.ExecutionPlan.from_string(plan_json, 0)
        executor.execute(0, t.data_ptr(), t.data_ptr(), t.numel() * 4, t.numel() * 4, n.DataType.float32, plan,
                         torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        symm.check()
        assert bool((symm.rank_view(t, 1) == 3.0).all().item())
        n.npkit.dump(str(tmp_path))
    finally:
        n.npkit.shutdown()
    assert not n.npkit.enabled()
    files = sorted(os.listdir(tmp_path))
    assert any(f.startswith("gpu_events_rank_0_buf_") for f in files) and "gpu_time_sync_rank_0" in files
    trace = json.loads(open(convert_npkit_dump_to_trace(str(tmp_path), str(tmp_path / "out"))).read())["traceEvents"]
    slices = [e for e in trace if e["ph"] == "X"]
    assert slices and all(e["dur"] >= 0 for e in slices)
    assert {"EXECUTOR_OP_SIGNAL", "EXECUTOR_OP_WAIT"} & {e["name"] for e in slices} or any("EXECUTOR_OP" in e["name"] for e in slices)
    executor.reset()
    symm.destroy()


def test_guard_bands_around_executor_buffers(monkeypatch):
    """With MSCCLPP_EXECUTOR_CANARY=1 the executor's scratch sits between two bands of 0xA5 on every rank. A correct plan
    leaves them alone (a packet plan writes its scratch from every peer, up to the last byte); a byte written just past
    the scratch is found by check_canaries() and again reported by reset(), which still returns the buffers."""
    from mscclpp_b200 import SymmetricMemory, native
    from mscclpp_b200._core.symm import tensor_from_pointer
    from mscclpp_b200.default_algos import single_node

    monkeypatch.setenv("MSCCLPP_EXECUTOR_CANARY", "1")
    n = native()
    world = 4
    symm = SymmetricMemory.emulated(world, nbytes=64 << 20, timeout_ms=3000)
    elems = 4 * world * 256
    t = symm.tensor((elems,), torch.float32)
    for r in range(world):
        symm.rank_view(t, r).fill_(r + 1.0)
    executor = n.Executor(symm.heap)
    assert executor.check_canaries() == 0  # nothing allocated yet
    plan = n.ExecutionPlan.from_string(single_node.build("allreduce_allpairs_packet", world).to_json(), 0)
    for _ in range(3):
        executor.execute(0, t.data_ptr(), t.data_ptr(), elems * 4, elems * 4, n.DataType.float32, plan,
                         torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    symm.check()
    regions = executor.canary_regions()
    assert len(regions) == 2 * world and all(nbytes == 256 for _, _, nbytes in regions)
    assert executor.check_canaries() == len(regions)

    label, address, nbytes = next(r for r in regions if "/scratch/back" in r[0] and r[0].endswith("rank 2"))
    band = tensor_from_pointer(address, (nbytes,), torch.uint8, t.device)
    assert bool((band == 0xA5).all().item())
    band[3] = 0
    torch.cuda.synchronize()
    with pytest.raises(Exception, match="guard band .*scratch/back/rank 2.*first at byte 3"):
        executor.check_canaries()
    free_before = symm.heap.bytes_free() if hasattr(symm.heap, "bytes_free") else None
    with pytest.raises(Exception, match="guard band"):
        executor.reset()
    if free_before is not None:
        assert symm.heap.bytes_free() > free_before  # the buffers went back to the heap all the same
    assert executor.canary_regions() == []
    symm.destroy()
