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
    p.add_argument("--probes", action="store_true", help="also time the kernel with its loads, its MMAs or its stores dropped")
    p.add_argument("--band", type=int, default=0, help="row blocks per band of the tile order (0 default, -1 none)")
    p.add_argument("--clocks", action="store_true", help="run each variant for about a second more and report the median SM "
                   "clock and power nvidia-smi saw meanwhile")
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

    def sustained(fn):
        """(median SM MHz, median W) while fn runs back to back for ~1.2 s."""
        import subprocess
        import time

        proc = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-lms", "100", "-i", "0"],
                                stdout=subprocess.PIPE, text=True)
        t_end = time.time() + 1.2
        while time.time() < t_end:
            for _ in range(50):
                fn()
            torch.cuda.synchronize()
        proc.terminate()
        rows = [r.split(",") for r in proc.communicate()[0].strip().splitlines() if "," in r]
        rows = rows[3:] or rows  # the first samples predate the load
        mhz = sorted(float(r[0]) for r in rows)
        watts = sorted(float(r[1]) for r in rows)
        return [mhz[len(mhz) // 2], watts[len(watts) // 2]] if rows else None

    two_sm = None if args.two_sm < 0 else bool(args.two_sm)
    run = lambda probe=0: gemm_bf16(a, b, d, block_n=args.block_n, two_sm=two_sm, probe=probe, band=args.band)
    us = timed(run)
    flops = 2.0 * args.m * args.n * args.k
    out = {"shape": [args.m, args.n, args.k], "block_n": bn, "two_sm": args.two_sm, "band": args.band, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1)}
    ref = a.float() @ b.float().t() if args.m * args.n <= (1 << 26) else None
    if ref is not None:
        out["rel_err"] = ((d.float() - ref).abs().max() / ref.abs().max()).item()
    if args.probes:
        names = {1: "no_loads", 2: "no_mma", 4: "no_stores", 5: "mma_only", 6: "loads_only", 3: "stores_only", 13: "mma_no_epilogue",
                 7: "epilogue_no_stores"}
        out["probe_us"] = {name: round(timed(lambda bit=bit: run(bit)), 2) for bit, name in names.items()}
        if args.clocks:
            out["probe_mhz_w"] = {name: sustained(lambda bit=bit: run(bit)) for bit, name in names.items()}
    if args.clocks:
        out["mhz_w"] = sustained(run)
    if not args.no_cublas:
        bt = b.t()
        cu = timed(lambda: torch.matmul(a, bt))
        if args.clocks:
            out["cublas_mhz_w"] = sustained(lambda: torch.matmul(a, bt))
        out["cublas_us"] = round(cu, 2)
        out["cublas_tflops"] = round(flops / cu / 1e6, 1)
    print(json.dumps({"gemm": out}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
