"""Plain torch.distributed code (backend "nccl") running on this library through the NCCL-API shim.

    LD_PRELOAD=$(python -c "import mscclpp_b200, os; print(os.path.join(mscclpp_b200.get_lib(), 'libmscclpp_b200_nccl.so'))") \
    MSCCLPP_NCCL_LIB_PATH=<path to a real libnccl.so.2, for the collectives the shim passes through> \
        python -m torch.distributed.run --nproc-per-node 8 examples/torch-integration/dsl_with_nccl_api.py

Plans installed with `python -m mscclpp_b200 --install` (or any JSON plan dropped into <cache>/default/) are picked up by
the shim's algorithm collection and take precedence over the native kernels for the sizes they cover.
"""
import os

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    loaded = any("libmscclpp_b200_nccl" in line for line in open("/proc/self/maps"))
    x = torch.full((1 << 20,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
    dist.all_reduce(x)
    torch.cuda.synchronize()
    ok = bool((x.float() == world * (world + 1) / 2).all().item())
    if rank == 0:
        print(f"all_reduce through {'the shim' if loaded else 'stock NCCL (shim not preloaded)'}: {'correct' if ok else 'WRONG'}")
    dist.destroy_process_group()
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
