"""Worker for the NCCL-API shim test: plain torch.distributed code, run with the shim preloaded.

Every collective below is issued through torch's NCCL backend; with the shim in LD_PRELOAD the
allreduce / allgather / reducescatter calls land in this library and the rest goes to the real NCCL
named by MSCCLPP_NCCL_LIB_PATH.
"""
import json
import os
import sys

import torch
import torch.distributed as dist


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda")
    results = {}
    ok = True
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32):
        for n in (1, 257, 4096, 1 << 16, 1 << 20, (1 << 22) + 8):
            g = torch.Generator(device="cpu").manual_seed(1234 + n)
            full = torch.randint(-3, 4, (world, n), generator=g).to(dtype)
            x = full[rank].to(dev).clone()
            dist.all_reduce(x)
            want = full.to(torch.float32).sum(0)
            err = (x.float().cpu() - want).abs().max().item()
            good = err <= (0 if dtype in (torch.int32, torch.float32) else 0.51)
            ok &= good
            results[f"allreduce/{dtype}/{n}"] = err
    # min
    x = torch.full((1000,), float(rank + 1), device=dev)
    dist.all_reduce(x, op=dist.ReduceOp.MIN)
    ok &= bool((x == 1).all().item())
    # all_gather / reduce_scatter
    for n in (64, 1 << 14, 1 << 20):
        src = torch.arange(n, device=dev, dtype=torch.float32) + rank * 1000
        out = torch.empty(world * n, device=dev, dtype=torch.float32)
        dist.all_gather_into_tensor(out, src)
        want = torch.cat([torch.arange(n, dtype=torch.float32) + r * 1000 for r in range(world)])
        ok &= bool(torch.equal(out.cpu(), want))
        inp = (torch.arange(world * n, device=dev, dtype=torch.float32) % 17) * (rank + 1)
        rs = torch.empty(n, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(rs, inp)
        tot = sum(r + 1 for r in range(world))
        want = (torch.arange(world * n, dtype=torch.float32) % 17)[rank * n:(rank + 1) * n] * tot
        ok &= bool(torch.equal(rs.cpu(), want))
    # broadcast: native (root streams into every rank's buffer), any size, any root
    for n, root in ((100, world - 1), (1 << 20, 0), ((1 << 18) + 3, world // 2)):
        b = torch.full((n,), float(rank), device=dev, dtype=torch.float16)
        dist.broadcast(b, src=root)
        ok &= bool((b == root).all().item())
    # CUDA-graph capture of an allreduce
    y = torch.ones(1 << 16, device=dev, dtype=torch.bfloat16)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        dist.all_reduce(y)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    dist.barrier()
    loaded = [l.split()[-1] for l in open("/proc/self/maps") if "libmscclpp_b200_nccl" in l]
    if rank == 0:
        print(json.dumps({"ok": bool(ok), "shim_loaded": bool(loaded), "world": world, "max_err": max(results.values())}))
    dist.destroy_process_group()
    sys.exit(0 if ok and loaded else 1)


if __name__ == "__main__":
    main()
