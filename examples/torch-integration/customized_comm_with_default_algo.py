"""Default algorithms called on torch tensors through the algorithm collection, on torch streams.

    python -m torch.distributed.run --nproc-per-node 8 examples/torch-integration/customized_comm_with_default_algo.py
"""
import os

import torch
import torch.distributed as dist

import mscclpp_b200 as mp
from mscclpp_b200.ext import AlgorithmCollectionBuilder


class CustomizedComm:
    """All-reduce on top of the default algorithm collection: the selector picks packets for small messages, the
    NVSwitch (multimem) two-shot kernel for large symmetric buffers and a staged path for ordinary torch tensors."""

    def __init__(self, heap_bytes: int = 1 << 30):
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.symm = mp.SymmetricMemory.from_env(nbytes=heap_bytes)
        n = mp.native()
        self.executor = n.Executor(self.symm.heap)
        self.collection = AlgorithmCollectionBuilder().build_default_algorithms(self.symm)

    def all_reduce(self, tensor: torch.Tensor, stream: torch.cuda.Stream = None):
        n = mp.native()
        nbytes = tensor.numel() * tensor.element_size()
        req = n.CollectiveRequest()
        req.world_size, req.n_ranks_per_node, req.rank = self.world, self.world, self.rank
        req.collective, req.message_size = "allreduce", nbytes
        req.input_buffer = req.output_buffer = tensor.data_ptr()
        req.dtype, req.op = mp.torch_dtype_to_native(tensor.dtype), n.ReduceOp.SUM
        req.symmetric_memory = self.symm.contains(tensor)
        algo = self.collection.select(req)
        assert algo is not None, "no algorithm for this request"
        st = (stream or torch.cuda.current_stream()).cuda_stream
        rc = algo.execute(None, tensor.data_ptr(), tensor.data_ptr(), nbytes, nbytes, req.dtype, n.ReduceOp.SUM, st, self.executor,
                          symmetric_memory=req.symmetric_memory)
        assert rc == 0, f"{algo.name} failed with {rc}"
        return algo.name

    def close(self):
        torch.cuda.synchronize()
        self.executor.reset()
        self.symm.destroy()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    comm = CustomizedComm()
    ok = True
    for numel, symmetric in ((1024, False), (1 << 20, False), (16 << 20, True)):
        t = comm.symm.tensor((numel,), torch.bfloat16) if symmetric else torch.empty(numel, dtype=torch.bfloat16, device="cuda")
        t.fill_(rank + 1)
        dist.barrier()
        name = comm.all_reduce(t)
        torch.cuda.synchronize()
        comm.symm.check()
        good = bool((t.float() == world * (world + 1) / 2).all().item())
        ok &= good
        if rank == 0:
            print(f"{numel:>9} elements ({'symmetric' if symmetric else 'torch'} memory) -> {name}: {'correct' if good else 'WRONG'}")
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
