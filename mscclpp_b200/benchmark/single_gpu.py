"""Single-GPU runs of the multi-rank kernels, for profiling: the ranks of a collective are emulated inside one
cooperative launch (gridDim.y = world) on one GPU, so the kernels can be captured with a profiler without a
multi-process job. Device-timed; numbers are NOT comparable to real multi-GPU runs (all "peers" share one HBM).

    python -m mscclpp_b200.benchmark.single_gpu tp-layer   --tokens 2048 --world 1
    python -m mscclpp_b200.benchmark.single_gpu tp-local   --tokens 2048 [--probe 128] [--two-sm 1] [--one-kernel 0]
    python -m mscclpp_b200.benchmark.single_gpu allreduce  --world 8 --mbytes 16
    python -m mscclpp_b200.benchmark.single_gpu moe        --world 8 --tokens 1024
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def _timed(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e3


def tp_layer(args):
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    world = args.world
    symm = SymmetricMemory.emulated(world, nbytes=(5 * args.tokens * args.hidden * 2) + (64 << 20), timeout_ms=5000)
    layer = RowParallelLinearNorm(symm, args.hidden, args.k, max_tokens=args.tokens)
    xs = [torch.randn((args.tokens, args.k), device="cuda").to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn((args.hidden, args.k), device="cuda") * 0.02).to(torch.bfloat16) for _ in range(world)]
    sms = torch.cuda.get_device_properties(0).multi_processor_count // world
    reducers = args.reducers or max(2, sms // 5)
    bn = -1 if args.two_sm else 0
    fn = lambda: layer.forward_fused(xs[0], mode=args.mode, nvls=False, block_n=bn if args.tokens >= 256 else 0, num_reducers=reducers,  # noqa: E731
                                     num_gemm_ctas=(sms - reducers) & ~1, emulated_inputs=list(zip(xs, ws)))
    us = _timed(fn, args.iters, args.warmup)
    symm.check()
    flops = 2.0 * args.tokens * args.k * args.hidden * world
    print(json.dumps({"tp_layer_emulated": {"world": world, "tokens": args.tokens, "hidden": args.hidden, "k": args.k, "mode": args.mode,
                                            "reducer_ctas": reducers, "two_sm": bool(args.two_sm), "us": round(us, 2),
                                            "tflops": round(flops / us / 1e6, 1)}}), flush=True)
    symm.destroy()


def tp_local(args):
    """The single-GPU layer (GEMM + residual + RMSNorm, world size 1) through its own kernel(s)."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    symm = SymmetricMemory.emulated(1, nbytes=(5 * args.tokens * args.hidden * 2) + (64 << 20), timeout_ms=5000)
    layer = RowParallelLinearNorm(symm, args.hidden, args.k, max_tokens=args.tokens)
    x = torch.randn((args.tokens, args.k), device="cuda").to(torch.bfloat16)
    layer.residual_in.normal_()
    fn = lambda: layer.forward_local(x, two_sm=bool(args.two_sm), one_kernel=bool(args.one_kernel), probe=args.probe)  # noqa: E731
    us = _timed(fn, args.iters, args.warmup)
    moved = args.tokens * args.hidden * 2 * 3 + (args.tokens + args.hidden) * args.k * 2
    print(json.dumps({"tp_local": {"tokens": args.tokens, "hidden": args.hidden, "k": args.k, "two_sm": bool(args.two_sm),
                                   "one_kernel": bool(args.one_kernel), "probe": args.probe, "us": round(us, 2),
                                   "tflops": round(2.0 * args.tokens * args.k * args.hidden / us / 1e6, 1),
                                   "algorithmic_gbs": round(moved / us / 1e3, 1)}}), flush=True)
    symm.destroy()


def allreduce(args):
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.ops import all_reduce

    world = args.world
    n = args.mbytes * (1 << 20) // 2
    symm = SymmetricMemory.emulated(world, nbytes=4 * n + (64 << 20), timeout_ms=5000)
    x = symm.tensor((n,), torch.bfloat16)
    y = symm.tensor((n,), torch.bfloat16)
    for r in range(world):
        symm.rank_view(x, r).fill_(r + 1)
    algo = args.algo
    us = _timed(lambda: all_reduce(symm, x, y, algo=algo), args.iters, args.warmup)
    symm.check()
    ok = bool((symm.rank_view(y, world - 1).float() == world * (world + 1) / 2).all().item())
    print(json.dumps({"allreduce_emulated": {"world": world, "bytes": n * 2, "algo": algo, "us": round(us, 2), "correct": ok,
                                             "hbm_gbs": round(n * 2 * world * 3 / us / 1e3, 1)}}), flush=True)
    symm.destroy()


def moe(args):
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.moe import ExpertParallelDispatcher

    world, T, H, K, E = args.world, args.tokens, args.hidden, 2, 64
    symm = SymmetricMemory.emulated(world, nbytes=10 * T * K * H * 2 + (64 << 20), timeout_ms=5000)
    disp = ExpertParallelDispatcher(symm, num_experts=E, hidden=H, max_tokens=T, topk=K, fp8=bool(args.fp8))
    for r in range(world):
        x = torch.randn((T, H), device="cuda").to(torch.bfloat16)
        idx = torch.topk(torch.rand((T, E), device="cuda"), K, dim=1).indices.to(torch.int32)
        wts = torch.full((T, K), 0.5, device="cuda")
        x_s, idx_s, w_s = disp.stage(r, x, idx, wts)
    blocks = max(1, 128 // world)
    us_d = _timed(lambda: disp.dispatch(x_s, idx_s, n_blocks=blocks), args.iters, args.warmup)
    _, _, slot_map = disp.dispatch(x_s, idx_s, n_blocks=blocks)
    us_c = _timed(lambda: disp.combine(idx_s, w_s, slot_map, n_blocks=blocks), args.iters, args.warmup)
    symm.check()
    print(json.dumps({"moe_emulated": {"world": world, "tokens_per_rank": T, "hidden": H, "fp8": bool(args.fp8), "dispatch_us": round(us_d, 2),
                                       "combine_us": round(us_c, 2)}}), flush=True)
    symm.destroy()


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("tp-layer", "tp-local", "allreduce", "moe"):
        s = sub.add_parser(name)
        s.add_argument("--world", type=int, default=1 if name.startswith("tp-") else 8)
        s.add_argument("--iters", type=int, default=10)
        s.add_argument("--warmup", type=int, default=3)
        s.add_argument("--tokens", type=int, default=2048 if name.startswith("tp-") else 1024)
        s.add_argument("--hidden", type=int, default=8192 if name.startswith("tp-") else 4096)
        if name.startswith("tp-"):
            s.add_argument("--k", type=int, default=1024)
            s.add_argument("--mode", type=int, default=1)
            s.add_argument("--reducers", type=int, default=0)
            s.add_argument("--two-sm", type=int, default=0)
        if name == "tp-local":
            s.add_argument("--one-kernel", type=int, default=1)
            s.add_argument("--probe", type=int, default=0, help="diagnostic bits of the kernel (0 in production)")
        if name == "allreduce":
            s.add_argument("--mbytes", type=int, default=16)
            s.add_argument("--algo", default="rsag_zero_copy")
        if name == "moe":
            s.add_argument("--fp8", type=int, default=0)
    args = p.parse_args(argv)
    {"tp-layer": tp_layer, "tp-local": tp_local, "allreduce": allreduce, "moe": moe}[args.cmd](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
