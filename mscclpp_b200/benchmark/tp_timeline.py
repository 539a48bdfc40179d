"""Per-CTA time line of the fused tensor-parallel layer (GEMM + allreduce + residual + RMSNorm in one launch).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m mscclpp_b200.benchmark.tp_timeline \
        [--tokens 8192] [--reducers 8,32,64] [--core 2] [--mode 1] [--nvls auto|on|off]

For every reducer count it prints the device time per step and, from one stamped launch on rank 0: when the GEMM CTAs
finished their tiles, how long reducer groups waited for row blocks, how long a row took (split into gather, residual
math and broadcast stores) and how much of the GEMM CTAs' time went into publishing row-block flags. This is the tool
that shows whether the reduction really runs under the matmul.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist


def _stats(v: torch.Tensor) -> str:
    v = v.double() / 1e3
    return f"{v.min().item():7.1f}/{v.median().item():7.1f}/{v.max().item():7.1f}"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--k-shard", type=int, default=1024)
    ap.add_argument("--reducers", default="8,32,64")
    ap.add_argument("--core", type=int, default=2, choices=(1, 2), help="1: one-SM 128x256 tiles, 2: 256x256 tiles on SM pairs")
    ap.add_argument("--mode", type=int, default=1, choices=(0, 1))
    ap.add_argument("--nvls", default="auto", choices=("auto", "on", "off"))
    ap.add_argument("--rows-per-unit", type=int, default=0)
    args = ap.parse_args()

    import mscclpp_b200 as mp
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    symm = mp.SymmetricMemory.from_env(nbytes=2 << 30)
    layer = RowParallelLinearNorm(symm, args.hidden, args.k_shard, max_tokens=args.tokens)
    x = torch.randn((args.tokens, args.k_shard), device="cuda").to(torch.bfloat16)
    layer.residual_in.normal_()
    nvls = bool(symm.nvls) and (world >= 8 if args.nvls == "auto" else args.nvls == "on")
    tl = torch.zeros((256, 16), dtype=torch.int64, device="cuda")

    for red in [int(r) for r in args.reducers.split(",")]:
        kw = dict(mode=args.mode, nvls=nvls, num_reducers=red, block_n=-1 if args.core == 2 else 256,
                  rows_per_unit=args.rows_per_unit)
        for _ in range(3):
            layer.forward_fused(x, **kw)
        torch.cuda.synchronize()
        dist.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            layer.forward_fused(x, **kw)
        end.record()
        torch.cuda.synchronize()
        us = torch.tensor([start.elapsed_time(end) / 5 * 1e3], device="cuda")
        dist.all_reduce(us, op=dist.ReduceOp.MAX)
        tl.zero_()
        dist.barrier()
        layer.forward_fused(x, timeline=tl, **kw)
        torch.cuda.synchronize()
        symm.check()
        t = tl.cpu()
        t = t[t[:, 0] > 0]
        n = t.shape[0]
        t0 = int(t[:, 0].min())
        gemm, ded = t[: n - red], t[n - red:]
        if rank == 0:
            print(f"== world {world} mode {args.mode} nvls {nvls} reducers {red} core {args.core}: {us.item():.1f} us/step "
                  f"(max over ranks), grid {n} CTAs; times in us as min/median/max")
            print(f"  GEMM CTAs: tiles done at {_stats(gemm[:, 1] - t0)}, left the kernel at {_stats(gemm[:, 2] - t0)}")
            print(f"             counting tiles {_stats(gemm[:, 11])}, of it in calls that published flags {_stats(gemm[:, 13])}, "
                  f"longest time between two tiles {_stats(gemm[:, 15])}")
            for name, part in (("joined after GEMM", gemm), ("dedicated reducers", ded)):
                if part.shape[0] == 0:
                    continue
                rows = max(1.0, part[:, 3].double().sum().item())
                print(f"  {name}: rows per group {part[:, 3].double().mean().item():.1f}, waited {_stats(part[:, 4])}, "
                      f"per row {part[:, 5].double().sum().item() / rows / 1e3:.1f} "
                      f"(gather {part[:, 8].double().sum().item() / rows / 1e3:.1f}, residual math "
                      f"{part[:, 9].double().sum().item() / rows / 1e3:.1f}, stores {part[:, 10].double().sum().item() / rows / 1e3:.1f})")
            if ded.shape[0]:
                print(f"  dedicated reducers: first row done at {_stats(ded[:, 6] - t0)}, left the kernel at {_stats(ded[:, 2] - t0)}")
            sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
