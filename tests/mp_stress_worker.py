"""Stress test of the fused TP layer's cross-GPU flag protocol, one rank per GPU (launched by torch.distributed.run from
test_gpu_multi.py or by hand).

Every configuration runs STRESS_LAUNCHES (default 1000) launches back to back with no host synchronisation in between;
consecutive launches use different inputs and different token counts, so a reducer that read a row block before its
producer's stores had landed (a stale row of the previous launch, or a half-written one) changes that row's checksum.
After each launch a small kernel reduces every row of `out` and of the residual stream to one fp32 checksum; all
checksums are compared at the end with those of an fp32 PyTorch reference of the same inputs. All device waits are
bounded: a flag that never arrives ends the launch with an error status, which check() turns into an exception.

Prints one JSON line per rank-0 check; exit code 0 = all good."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mscclpp_b200 import SymmetricMemory  # noqa: E402
from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    launches = int(os.environ.get("STRESS_LAUNCHES", "1000"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    symm = SymmetricMemory.from_env(nbytes=1 << 30, enable_nvls=os.environ.get("MSCCLPP_TEST_NVLS", "1") == "1", timeout_ms=5000)
    failures = []

    def report(name, ok, **extra):
        if not ok:
            failures.append(name)
        if rank == 0:
            print(json.dumps({"check": name, "ok": bool(ok), **extra}), flush=True)

    hidden, k_shard, max_t = 4096, 512, 1024
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k_shard, max_tokens=max_t, seed=11)
    gen = torch.Generator(device=dev).manual_seed(5)
    layer.gamma.copy_((1 + 0.1 * torch.randn((hidden,), generator=gen, device=dev)).to(torch.bfloat16))

    # a pool of inputs with their fp32-reference checksums; consecutive launches take consecutive pool entries
    pool = []
    for i, tokens in enumerate((1024, 100, 512, 8, 1024, 333, 256, 1000)):
        g_all = torch.Generator(device=dev).manual_seed(900 + i)  # the residual is replicated: same seed on every rank
        residual = torch.randn((tokens, hidden), generator=g_all, device=dev).to(torch.bfloat16)
        g_mine = torch.Generator(device=dev).manual_seed(7000 + 31 * i + rank)
        x = torch.randn((tokens, k_shard), generator=g_mine, device=dev).to(torch.bfloat16)
        part = (x.float() @ layer.weight.float().t()).to(torch.bfloat16)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        h = (torch.stack([p.float() for p in parts]).sum(0).to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
        y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps) * layer.gamma.float()).to(torch.bfloat16).float()
        pool.append((x, residual, h.sum(-1), y.sum(-1)))

    sums_h = torch.zeros((launches, max_t), device=dev)
    sums_y = torch.zeros((launches, max_t), device=dev)
    configs = [(mode, nv, False) for mode in (0, 1, 3) for nv in ([False, True] if symm.nvls else [False])]
    configs.append((0, False, True))  # the conservative publication (system-scope fence + release stores) as well
    configs.append((1, symm.nvls, True))
    for mode, nv, sys_fence in configs:
        sums_h.zero_()
        sums_y.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        for it in range(launches):
            x, residual, _, _ = pool[it % len(pool)]
            t = x.shape[0]
            out, res = layer.forward_fused(x, residual, mode=mode, nvls=nv, sys_fence=sys_fence)
            torch.sum(res, dim=-1, dtype=torch.float32, out=sums_h[it, :t])
            torch.sum(out, dim=-1, dtype=torch.float32, out=sums_y[it, :t])
        torch.cuda.synchronize()
        symm.check()
        worst_h = worst_y = 0.0
        bad = 0
        for it in range(launches):
            _, _, ref_h, ref_y = pool[it % len(pool)]
            t = ref_h.shape[0]
            eh = (sums_h[it, :t] - ref_h).abs().max().item()
            ey = (sums_y[it, :t] - ref_y).abs().max().item()
            worst_h, worst_y = max(worst_h, eh), max(worst_y, ey)
            # a row of 4096 O(1) values: rounding moves its sum by a few tenths, a stale or torn row by tens
            bad += int(eh > 4.0 or ey > 6.0)
        report(f"tp_fused_stress/mode={mode}/nvls={nv}/sys_fence={sys_fence}/launches={launches}", bad == 0,
               bad_launches=bad, worst_h=worst_h, worst_y=worst_y)

    torch.cuda.synchronize()
    dist.barrier()
    symm.destroy()
    dist.destroy_process_group()
    if failures:
        print(json.dumps({"rank": rank, "failures": failures[:10]}), flush=True)
        sys.exit(1)


if __name__ == "__main__":
    main()
