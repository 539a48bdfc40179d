"""Sequence-parallel MLP benchmark: fused all-gather -> GEMM and GEMM -> reduce-scatter against the library
composition (NCCL all-gather + cuBLAS, cuBLAS + NCCL reduce-scatter) on the same shapes.

    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.sp_mlp --hidden 8192 --ffn 28672 --seq 8192

Reports microseconds (device-timed, max over ranks), achieved TFLOP/s per GPU and the fraction of the roofline
max(FLOPs / GEMM peak, NVLink bytes / link bandwidth).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from .common import Dist, time_eager

GEMM_PEAK_TFLOPS = 1420.0   # sustained cuBLAS bf16 on this part (measured), the roofline's compute side
LINK_GBS = 770.0            # measured peer copy bandwidth per direction


def run(args) -> dict:
    import mscclpp_b200 as mp
    from mscclpp_b200.parallel.sp_layer import SequenceParallelMLP, all_gather_gemm, gemm_reduce_scatter

    d = Dist()
    tp = d.world
    seq, hidden, ffn = args.seq, args.hidden, args.ffn
    f_shard = ffn // tp
    heap = 2 * (seq // tp) * hidden * 2 + 2 * seq * hidden * 2 + seq * f_shard * 2 + (512 << 20)
    symm = mp.SymmetricMemory.from_env(nbytes=heap)
    mlp = SequenceParallelMLP(symm, hidden=hidden, ffn=ffn, seq=seq, activation="gelu")
    g = torch.Generator(device=d.device).manual_seed(5 + d.rank)
    mlp.x_local.copy_(torch.randn(mlp.x_local.shape, generator=g, device=d.device).to(torch.bfloat16))
    out = {"config": {"seq": seq, "hidden": hidden, "ffn": ffn, "tp": tp, "dtype": "bf16", "nvls": bool(symm.nvls),
                      "l2": "operands of every step exceed the 126 MB L2"}}

    def roofline_us(flops, link_bytes):
        return max(flops / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e6

    # ---- all-gather -> GEMM
    flops_up = 2.0 * seq * hidden * f_shard
    ag_bytes = (tp - 1) / tp * seq * hidden * 2
    best = None
    for copiers in args.copiers:
        us = time_eager(d, lambda: all_gather_gemm(symm, mlp.x_local, mlp.x_full, mlp.w1, mlp.h, activation="gelu", num_copiers=copiers),
                        args.iters, args.warmup, check=symm.check) * 1e3
        if best is None or us < best[0]:
            best = (us, copiers)
    x_full = torch.empty((seq, hidden), dtype=torch.bfloat16, device=d.device)
    w1_t = mlp.w1.t()

    def base_up():
        if tp > 1:
            dist.all_gather_into_tensor(x_full, mlp.x_local)
        else:
            x_full.copy_(mlp.x_local)
        return torch.nn.functional.gelu(torch.matmul(x_full, w1_t), approximate="tanh")

    base_us = time_eager(d, base_up, args.iters, args.warmup) * 1e3
    # numerics of the fused path against the composition
    ref = base_up().float()
    all_gather_gemm(symm, mlp.x_local, mlp.x_full, mlp.w1, mlp.h, activation="gelu", num_copiers=best[1])
    torch.cuda.synchronize()
    err_up = (mlp.h.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-9)
    roof = roofline_us(flops_up, ag_bytes)
    out["all_gather_gemm"] = {"us": round(best[0], 2), "copier_ctas": best[1], "tflops_per_gpu": round(flops_up / best[0] / 1e6, 1),
                              "roofline_us": round(roof, 2), "frac_of_roofline": round(roof / best[0], 3),
                              "nccl_cublas_us": round(base_us, 2), "speedup": round(base_us / best[0], 3), "rel_err": err_up}
    del ref

    # ---- GEMM -> reduce-scatter
    flops_down = 2.0 * seq * f_shard * hidden
    rs_bytes = (tp - 1) / tp * seq * hidden * 2
    best = None
    for reducers in args.reducers:
        us = time_eager(d, lambda: gemm_reduce_scatter(symm, mlp.h, mlp.w2, mlp.partial, mlp.y_local, num_reducers=reducers),
                        args.iters, args.warmup, check=symm.check) * 1e3
        if best is None or us < best[0]:
            best = (us, reducers)
    w2_t = mlp.w2.t()
    y_base = torch.empty((seq // tp, hidden), dtype=torch.bfloat16, device=d.device)

    def base_down():
        p = torch.matmul(mlp.h, w2_t)
        if tp > 1:
            dist.reduce_scatter_tensor(y_base, p)
        else:
            y_base.copy_(p)
        return y_base

    base_us = time_eager(d, base_down, args.iters, args.warmup) * 1e3
    ref = base_down().float()
    gemm_reduce_scatter(symm, mlp.h, mlp.w2, mlp.partial, mlp.y_local, num_reducers=best[1])
    torch.cuda.synchronize()
    err_down = (mlp.y_local.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-9)
    roof = roofline_us(flops_down, rs_bytes)
    out["gemm_reduce_scatter"] = {"us": round(best[0], 2), "reducer_ctas": best[1], "tflops_per_gpu": round(flops_down / best[0] / 1e6, 1),
                                  "roofline_us": round(roof, 2), "frac_of_roofline": round(roof / best[0], 3),
                                  "cublas_nccl_us": round(base_us, 2), "speedup": round(base_us / best[0], 3), "rel_err": err_down}

    # ---- both halves back to back
    cop, red = out["all_gather_gemm"]["copier_ctas"], out["gemm_reduce_scatter"]["reducer_ctas"]
    mlp_us = time_eager(d, lambda: mlp.forward(num_copiers=cop, num_reducers=red), args.iters, args.warmup, check=symm.check) * 1e3

    def base_mlp():
        if tp > 1:
            dist.all_gather_into_tensor(x_full, mlp.x_local)
        else:
            x_full.copy_(mlp.x_local)
        hh = torch.nn.functional.gelu(torch.matmul(x_full, w1_t), approximate="tanh")
        p = torch.matmul(hh, w2_t)
        if tp > 1:
            dist.reduce_scatter_tensor(y_base, p)
        return y_base

    base_us = time_eager(d, base_mlp, args.iters, args.warmup) * 1e3
    out["mlp"] = {"us": round(mlp_us, 2), "nccl_cublas_us": round(base_us, 2), "speedup": round(base_us / mlp_us, 3),
                  "tflops_per_gpu": round((flops_up + flops_down) / mlp_us / 1e6, 1)}
    # ---- gated form (SwiGLU): all-gather -> GEMM over interleaved gate / up weights, silu(gate) * up in the epilogue
    if args.gated:
        del mlp
        symm.destroy()
        f_g = args.gated_ffn // tp
        heap = 2 * (seq // tp) * hidden * 2 + 2 * seq * hidden * 2 + seq * f_g * 2 + (512 << 20)
        symm = mp.SymmetricMemory.from_env(nbytes=heap)
        gm = SequenceParallelMLP(symm, hidden=hidden, ffn=args.gated_ffn, seq=seq, activation="swiglu")
        gm.x_local.copy_(torch.randn(gm.x_local.shape, generator=g, device=d.device).to(torch.bfloat16))
        flops_g = 2.0 * seq * hidden * (2 * f_g)
        best = None
        for copiers in args.copiers:
            us = time_eager(d, lambda: all_gather_gemm(symm, gm.x_local, gm.x_full, gm.w1, gm.h, activation="swiglu", num_copiers=copiers),
                            args.iters, args.warmup, check=symm.check) * 1e3
            if best is None or us < best[0]:
                best = (us, copiers)
        wg_t, wu_t = gm.w_gate.t(), gm.w_up.t()

        def base_gated():
            if tp > 1:
                dist.all_gather_into_tensor(x_full, gm.x_local)
            else:
                x_full.copy_(gm.x_local)
            return torch.nn.functional.silu(torch.matmul(x_full, wg_t)) * torch.matmul(x_full, wu_t)

        base_us = time_eager(d, base_gated, args.iters, args.warmup) * 1e3
        ref = base_gated().float()
        all_gather_gemm(symm, gm.x_local, gm.x_full, gm.w1, gm.h, activation="swiglu", num_copiers=best[1])
        torch.cuda.synchronize()
        err_g = (gm.h.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-9)
        roof = roofline_us(flops_g, ag_bytes)
        out["all_gather_gemm_swiglu"] = {"ffn": args.gated_ffn, "n_per_rank": 2 * f_g, "us": round(best[0], 2), "copier_ctas": best[1],
                                         "tflops_per_gpu": round(flops_g / best[0] / 1e6, 1), "roofline_us": round(roof, 2),
                                         "frac_of_roofline": round(roof / best[0], 3), "nccl_cublas_us": round(base_us, 2),
                                         "speedup": round(base_us / best[0], 3), "rel_err": err_g}
    d.barrier()
    symm.destroy()
    if args.standalone:
        d.close()
    return out if d.rank == 0 else {}


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--seq", type=int, default=8192)
    p.add_argument("--hidden", type=int, default=8192)
    p.add_argument("--ffn", type=int, default=28672)
    p.add_argument("--gated", action="store_true", help="also time the gated (SwiGLU) all-gather -> GEMM, N = 2 x gated-ffn / tp per rank")
    p.add_argument("--gated-ffn", type=int, default=28672)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--copiers", type=int, nargs="*", default=[8, 12, 16, 24])
    p.add_argument("--reducers", type=int, nargs="*", default=[16, 24, 32])
    args = p.parse_args(argv)
    args.standalone = True
    res = run(args)
    if res:
        print(json.dumps({"sp_mlp": res}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
