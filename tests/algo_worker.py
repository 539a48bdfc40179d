"""Multi-process GPU check of the algorithm framework: every default algorithm and the default selector, run
through the public Python API on a real symmetric heap (one rank per GPU), with heap and non-heap buffers."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import mscclpp_b200 as mp  # noqa: E402
from mscclpp_b200.ext import AlgorithmCollectionBuilder  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n = mp.native()
    symm = mp.SymmetricMemory.from_env(nbytes=1 << 30, enable_nvls=os.environ.get("MSCCLPP_TEST_NVLS", "1") == "1", timeout_ms=5000)
    executor = n.Executor(symm.heap)
    coll = AlgorithmCollectionBuilder().build_default_algorithms(symm)
    names = sorted(a.name for a in coll)
    failures = []

    def report(name, ok, **extra):
        if not ok:
            failures.append(name)
        if rank == 0:
            print(json.dumps({"check": name, "ok": bool(ok), **extra}), flush=True)

    report("registered", {"default_allreduce_packet", "default_allreduce_rsag_zero_copy", "default_allgather_fullmesh2",
                          "default_reducescatter_zero_copy"} <= set(names), names=names)
    stream = torch.cuda.current_stream().cuda_stream

    def reference(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        return torch.stack([p.float() for p in parts]).sum(0)

    numel = 1 << 18  # 512 KiB of bf16: inside the packet algorithms' range too
    heap_in, heap_out = symm.tensor((numel,), torch.bfloat16), symm.tensor((numel,), torch.bfloat16)
    user_in, user_out = torch.empty(numel, dtype=torch.bfloat16, device=dev), torch.empty(numel, dtype=torch.bfloat16, device=dev)
    for algo in coll.get_by_collective("allreduce"):
        for where, (tin, tout) in {"heap": (heap_in, heap_out), "user": (user_in, user_out)}.items():
            g = torch.Generator(device=dev).manual_seed(rank + 11)
            tin.copy_(torch.randn(numel, generator=g, device=dev).to(torch.bfloat16))
            expect = reference(tin).to(torch.bfloat16).float()
            tout.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            rc = algo.execute(None, tin.data_ptr(), tout.data_ptr(), numel * 2, numel * 2, n.DataType.bfloat16, n.ReduceOp.SUM, stream,
                              executor, symmetric_memory=(where == "heap"))
            torch.cuda.synchronize()
            symm.check()
            zero_copy = algo.name.endswith("zero_copy")
            if zero_copy and where == "user":
                report(f"{algo.name}/{where}/refuses", rc == int(n.CommResult.InvalidUsage), rc=rc)
                continue
            err = (tout.float() - expect).abs().max().item()
            report(f"{algo.name}/{where}", rc == 0 and err <= 6e-2 * max(1.0, expect.abs().max().item()), rc=rc, err=err)

    # selector: size and placement decide
    def pick(nbytes, symmetric):
        req = n.CollectiveRequest()
        req.world_size, req.n_ranks_per_node, req.rank = world, world, rank
        req.collective, req.message_size, req.symmetric_memory = "allreduce", nbytes, symmetric
        req.dtype, req.op = n.DataType.bfloat16, n.ReduceOp.SUM
        a = coll.select(req)
        return a.name if a else None

    small = pick(1024, True)
    report("select/small", small in ("default_allreduce_nvls_packet", "default_allreduce_packet"), got=small)
    big_sym = pick(64 << 20, True)
    report("select/large_symmetric", big_sym in ("default_allreduce_nvls_zero_copy", "default_allreduce_rsag_zero_copy"), got=big_sym)
    big_user = pick(64 << 20, False)
    report("select/large_user", big_user is not None and "zero_copy" not in big_user, got=big_user)

    # odd size (not a multiple of 16 bytes) beyond the packet range goes through padded staging
    odd = (3 << 20) + 3
    t = torch.ones(odd, dtype=torch.float32, device=dev) * (rank + 1)
    req_algo = pick(odd * 4, False)
    algo = coll.get_by_name(req_algo)
    rc = algo.execute(None, t.data_ptr(), t.data_ptr(), odd * 4, odd * 4, n.DataType.float32, n.ReduceOp.SUM, stream, executor)
    torch.cuda.synchronize()
    report("odd_size_in_place", rc == 0 and bool((t == world * (world + 1) / 2).all().item()), algo=req_algo)

    # allgather and reduce-scatter on user buffers
    per = 1 << 16
    src = torch.arange(per, device=dev, dtype=torch.float32) + rank * per
    dst = torch.zeros(world * per, device=dev, dtype=torch.float32)
    ag = coll.get_by_name("default_allgather_fullmesh2")
    rc = ag.execute(None, src.data_ptr(), dst.data_ptr(), per * 4, world * per * 4, n.DataType.float32, n.ReduceOp.NOP, stream, executor)
    torch.cuda.synchronize()
    report("allgather/user", rc == 0 and bool(torch.equal(dst, torch.arange(world * per, device=dev, dtype=torch.float32))))
    inp = torch.ones(world * per, device=dev, dtype=torch.float32) * (rank + 1)
    out = torch.zeros(per, device=dev, dtype=torch.float32)
    rs = coll.get_by_name("default_reducescatter_zero_copy")
    rc = rs.execute(None, inp.data_ptr(), out.data_ptr(), world * per * 4, per * 4, n.DataType.float32, n.ReduceOp.SUM, stream, executor)
    torch.cuda.synchronize()
    report("reducescatter/user", rc == 0 and bool((out == world * (world + 1) / 2).all().item()))

    # all-to-all: chunk p of my input becomes chunk `rank` of rank p's output
    a2a = coll.get_by_name("default_alltoall")
    send = (torch.arange(world * per, device=dev, dtype=torch.float32) + 1000000 * rank)
    recv = torch.zeros(world * per, device=dev, dtype=torch.float32)
    rc = a2a.execute(None, send.data_ptr(), recv.data_ptr(), world * per * 4, world * per * 4, n.DataType.uint8, n.ReduceOp.NOP, stream, executor)
    torch.cuda.synchronize()
    want = torch.cat([torch.arange(rank * per, (rank + 1) * per, device=dev, dtype=torch.float32) + 1000000 * p for p in range(world)])
    report("alltoall/user", rc == 0 and bool(torch.equal(recv, want)))

    # broadcast from the last rank, odd size (padded through staging)
    bc = coll.get_by_name("default_broadcast")
    nb = 100003
    buf = torch.full((nb,), float(rank), device=dev, dtype=torch.float16)
    rc = bc.execute(None, buf.data_ptr(), buf.data_ptr(), nb * 2, nb * 2, n.DataType.uint8, n.ReduceOp.NOP, stream, executor,
                    extras={"root": world - 1})
    torch.cuda.synchronize()
    report("broadcast/user_odd_size", rc == 0 and bool((buf == world - 1).all().item()))

    # a DSL algorithm compiled at run time runs through the same interface
    from mscclpp_b200.default_algos import allreduce_allpairs, make_spec
    from mscclpp_b200.language.collectives import AllReduce

    dsl = mp.compile(allreduce_allpairs, make_spec("dsl_allpairs", AllReduce(world, 1, True), world), rank)
    g = torch.Generator(device=dev).manual_seed(rank + 5)
    heap_in.copy_(torch.randn(numel, generator=g, device=dev).to(torch.bfloat16))
    expect = reference(heap_in).to(torch.bfloat16).float()
    torch.cuda.synchronize()
    dist.barrier()
    rc = dsl.execute(None, heap_in.data_ptr(), heap_in.data_ptr(), numel * 2, numel * 2, n.DataType.bfloat16, n.ReduceOp.SUM, stream, executor)
    torch.cuda.synchronize()
    symm.check()
    err = (heap_in.float() - expect).abs().max().item()
    report("dsl_algorithm", rc == 0 and err <= 6e-2 * max(1.0, expect.abs().max().item()), err=err)

    # the same plan on ORDINARY tensors (outside the heap), large enough for zero copy: every rank maps every rank's buffer
    # once, the plan runs on the tensors themselves, and a second call on the same tensors finds the mappings again
    big = 1 << 20  # 2 MiB of bf16
    user = torch.empty(big, dtype=torch.bfloat16, device=dev)
    before = executor.zero_copy_launches()
    for rep in range(2):
        g = torch.Generator(device=dev).manual_seed(rank * 3 + rep)
        user.copy_(torch.randn(big, generator=g, device=dev).to(torch.bfloat16))
        expect = reference(user).to(torch.bfloat16).float()
        torch.cuda.synchronize()
        dist.barrier()
        rc = dsl.execute(None, user.data_ptr(), user.data_ptr(), big * 2, big * 2, n.DataType.bfloat16, n.ReduceOp.SUM, stream, executor)
        torch.cuda.synchronize()
        symm.check()
        err = (user.float() - expect).abs().max().item()
        report(f"dsl_algorithm/user_buffer_zero_copy/{rep}", rc == 0 and err <= 6e-2 * max(1.0, expect.abs().max().item()), err=err)
    report("dsl_algorithm/zero_copy_taken", executor.zero_copy_launches() == before + 2, launches=executor.zero_copy_launches() - before)
    # a small message on an ordinary tensor is staged (two short copies cost less than a mapping)
    small_t = torch.ones(4096, dtype=torch.bfloat16, device=dev)
    before = executor.zero_copy_launches()
    rc = dsl.execute(None, small_t.data_ptr(), small_t.data_ptr(), 8192, 8192, n.DataType.bfloat16, n.ReduceOp.SUM, stream, executor)
    torch.cuda.synchronize()
    report("dsl_algorithm/small_user_buffer_staged", rc == 0 and executor.zero_copy_launches() == before and bool((small_t == world).all().item()))

    torch.cuda.synchronize()
    dist.barrier()
    executor.reset()
    symm.destroy()
    dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({"summary": "algo_worker", "ok": not failures, "failures": failures}), flush=True)
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
