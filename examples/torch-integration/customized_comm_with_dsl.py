"""An algorithm written in the DSL, compiled to an execution plan at run time and executed on torch tensors.

    python -m torch.distributed.run --nproc-per-node 8 examples/torch-integration/customized_comm_with_dsl.py
"""
import os

import torch
import torch.distributed as dist

import mscclpp_b200 as mp
from mscclpp_b200.language.channel import MemoryChannel
from mscclpp_b200.language.collectives import AllReduce
from mscclpp_b200.language.program import CollectiveProgram
from mscclpp_b200.language.rank import Buffer, Rank
from mscclpp_b200.language.utils import AlgoSpec


def one_shot_packets(spec: AlgoSpec) -> CollectiveProgram:
    """Every rank sends its whole input to every peer as LL packets and reduces what arrives: one step, no signals."""
    n = spec.world_size
    with CollectiveProgram.from_spec(spec) as prog:
        scratch = [Buffer(r, n * n) for r in range(n)]
        chan = {(s, d): MemoryChannel(d, s) for s in range(n) for d in range(n) if s != d}
        for r in range(n):
            inp = Rank(r).get_input_buffer()
            for p in range(n):
                if p != r:
                    chan[(r, p)].put_packets(scratch[p][r * n:(r + 1) * n], inp[0:n], tb=0)
        for r in range(n):
            rank = Rank(r)
            rank.reduce(rank.get_input_buffer()[0:n], [scratch[r][p * n:(p + 1) * n] for p in range(n) if p != r], tb=0, packet=True)
    return prog


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    symm = mp.SymmetricMemory.from_env(nbytes=512 << 20)
    executor = mp.native().Executor(symm.heap)
    spec = AlgoSpec(name="one_shot_packets", collective=AllReduce(world, 1, True), nranks_per_node=world, world_size=world, in_place=True,
                    instances=1, protocol="LL", num_threads_per_block=1024, max_message_size=1 << 20)
    algo = mp.compile(one_shot_packets, spec, rank)  # cached under MSCCLPP_CACHE_DIR
    t = torch.full((64 * 1024,), float(rank + 1), device="cuda", dtype=torch.float32)  # an ordinary torch tensor: staged by the executor
    dist.barrier()
    rc = algo.execute(None, t.data_ptr(), t.data_ptr(), t.numel() * 4, t.numel() * 4, mp.DataType.float32, mp.ReduceOp.SUM,
                      torch.cuda.current_stream().cuda_stream, executor)
    torch.cuda.synchronize()
    symm.check()
    ok = rc == 0 and bool((t == world * (world + 1) / 2).all().item())
    if rank == 0:
        print("DSL allreduce:", "correct" if ok else "WRONG")
    dist.barrier()
    executor.reset()
    symm.destroy()
    dist.destroy_process_group()
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
