"""A native algorithm compiled at run time (`compile_native`) and used from PyTorch.

    python -m torch.distributed.run --nproc-per-node 2 examples/torch-integration/customized_allgather.py
"""
import os

import torch
import torch.distributed as dist

import mscclpp_b200 as mp


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    symm = mp.SymmetricMemory.from_env(nbytes=256 << 20)
    here = os.path.dirname(os.path.abspath(__file__))
    module = mp.compile_native("customized_allgather", os.path.join(here, "..", "customized-collective-algorithm", "customized_allgather.cu"))
    algo = mp.Algorithm.create_from_native_capsule(module.create_allgather(symm.heap))
    n = 1 << 20
    mine = torch.full((n,), float(rank), device="cuda", dtype=torch.float32)
    out = symm.tensor((world * n,), torch.float32)
    dist.barrier()
    rc = algo.execute(None, mine.data_ptr(), out.data_ptr(), n * 4, world * n * 4, mp.DataType.float32, stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    symm.check()
    expect = torch.arange(world, device="cuda", dtype=torch.float32).repeat_interleave(n)
    ok = rc == 0 and torch.equal(out, expect)
    if rank == 0:
        print("customized allgather:", "correct" if ok else "WRONG")
    dist.barrier()
    symm.destroy()
    dist.destroy_process_group()
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
