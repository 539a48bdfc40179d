"""tcgen05 GEMM benchmark on one GPU against cuBLAS (torch.matmul) for the same shape.

    python -m mscclpp_b200.benchmark.gemm --m 8192 --n 8192 --k 8192 [--block-n 256] [--iters 20]
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--n", type=int, default=8192)
    p.add_argument("--k", type=int, default=8192)
    p.add_argument("--block-n", type=int, default=0)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--no-cublas", action="store_true")
    p.add_argument("--two-sm", type=int, default=-1, help="1: 256x256 tiles on SM pairs, 0: one-SM tiles, -1: automatic")
    args = p.parse_args(argv)
    from mscclpp_b200.ops.gemm import gemm_bf16, pick_block_n

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn((args.m, args.k), generator=g, device=dev).to(torch.bfloat16)
    b = (torch.randn((args.n, args.k), generator=g, device=dev) * 0.05).to(torch.bfloat16)
    d = torch.empty((args.m, args.n), dtype=torch.bfloat16, device=dev)
    bn = args.block_n or pick_block_n(args.m, args.n)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / args.iters * 1e3

    two_sm = None if args.two_sm < 0 else bool(args.two_sm)
    us = timed(lambda: gemm_bf16(a, b, d, block_n=args.block_n, two_sm=two_sm))
    flops = 2.0 * args.m * args.n * args.k
    out = {"shape": [args.m, args.n, args.k], "block_n": bn, "two_sm": args.two_sm, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1)}
    ref = a.float() @ b.float().t() if args.m * args.n <= (1 << 26) else None
    if ref is not None:
        out["rel_err"] = ((d.float() - ref).abs().max() / ref.abs().max()).item()
    if not args.no_cublas:
        bt = b.t()
        cu = timed(lambda: torch.matmul(a, bt))
        out["cublas_us"] = round(cu, 2)
        out["cublas_tflops"] = round(flops / cu / 1e6, 1)
    print(json.dumps({"gemm": out}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
