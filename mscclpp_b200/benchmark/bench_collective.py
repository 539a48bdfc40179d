"""Collective benchmark: candidate algorithms x message size, eager and CUDA-graph timing, bus bandwidth,
correctness against an fp32 reference and NCCL on the same buffers for comparison
(reference: python/mscclpp_benchmark/bench_collective.py:192-241,373-432).

    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.bench_collective \
        --collective allreduce --dtype bfloat16 --min-bytes 1024 --max-bytes 1073741824 --json out.json
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from .common import Dist, time_eager, time_graph
from .correctness import error_stats, passes

DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def bus_bandwidth_gbs(collective: str, nbytes: int, world: int, us: float) -> float:
    """nccl-tests convention: allreduce moves 2(n-1)/n of the buffer per rank, allgather/reducescatter (n-1)/n of the
    large buffer."""
    factor = 2.0 * (world - 1) / world if collective == "allreduce" else (world - 1) / world
    return nbytes * factor / (us * 1e-6) / 1e9


def run(args) -> int:
    import mscclpp_b200 as mp
    from mscclpp_b200.ext import AlgorithmCollectionBuilder

    d = Dist()
    n = mp.native()
    dtype = DTYPES[args.dtype]
    native_dtype = mp.torch_dtype_to_native(dtype)
    esize = torch.empty((), dtype=dtype).element_size()
    symm = mp.SymmetricMemory.from_env(nbytes=3 * args.max_bytes + (256 << 20))
    executor = n.Executor(symm.heap)
    coll = AlgorithmCollectionBuilder().build_default_algorithms(symm)
    candidates = [a for a in coll.get_by_collective(args.collective) if not args.algorithms or a.name in args.algorithms]
    buf_in = symm.tensor((args.max_bytes // esize,), dtype)
    buf_out = symm.tensor((args.max_bytes // esize,), dtype)
    nccl_in = torch.empty(args.max_bytes // esize, dtype=dtype, device=d.device)
    nccl_out = torch.empty(args.max_bytes // esize, dtype=dtype, device=d.device)
    g = torch.Generator(device=d.device).manual_seed(17 + d.rank)
    buf_in.copy_(torch.randn(buf_in.numel(), generator=g, device=d.device).to(dtype))
    nccl_in.copy_(buf_in)
    rows = []
    size = args.min_bytes
    while size <= args.max_bytes:
        # `size` is the large buffer of the collective (allgather output, reducescatter input)
        big = size // esize // d.world * d.world
        small = big // d.world
        if args.collective == "allreduce":
            n_in, n_out = big, big
        elif args.collective == "allgather":
            n_in, n_out = small, big
        else:
            n_in, n_out = big, small
        row = {"bytes": big * esize, "algorithms": {}}
        iters = 50 if size <= (1 << 20) else (20 if size <= (64 << 20) else 8)
        # reference result through NCCL
        if d.world > 1:
            if args.collective == "allreduce":
                nccl_fn = lambda: dist.all_reduce(nccl_out[:n_out].copy_(nccl_in[:n_in]))  # noqa: E731
                time_fn = lambda: dist.all_reduce(nccl_out[:n_out])  # noqa: E731
            elif args.collective == "allgather":
                nccl_fn = time_fn = lambda: dist.all_gather_into_tensor(nccl_out[:n_out], nccl_in[:n_in])  # noqa: E731
            else:
                nccl_fn = time_fn = lambda: dist.reduce_scatter_tensor(nccl_out[:n_out], nccl_in[:n_in])  # noqa: E731
            nccl_fn()
            torch.cuda.synchronize()
            parts = [torch.empty(n_in, dtype=dtype, device=d.device) for _ in range(d.world)]
            dist.all_gather(parts, buf_in[:n_in])
            if args.collective == "allreduce":
                ref = torch.stack([p.float() for p in parts]).sum(0)
            elif args.collective == "allgather":
                ref = torch.cat(parts).float()
            else:
                ref = torch.stack([p.float() for p in parts]).sum(0)[d.rank * small:(d.rank + 1) * small]
            del parts
            row["nccl_us"] = round(time_eager(d, time_fn, iters, 5) * 1e3, 2)
            row["nccl_busbw_gbs"] = round(bus_bandwidth_gbs(args.collective, big * esize, d.world, row["nccl_us"]), 2)
        else:
            ref = buf_in[:n_out].float()
        for algo in candidates:
            lo, hi = algo.message_size_range
            msg = n_in * esize if args.collective != "allgather" else n_in * esize
            if not (lo <= msg <= hi):
                continue

            def call(stream=None, algo=algo):
                st = (stream or torch.cuda.current_stream()).cuda_stream
                rc = algo.execute(None, buf_in.data_ptr(), buf_out.data_ptr(), n_in * esize, n_out * esize, native_dtype, n.ReduceOp.SUM, st,
                                  executor, args.n_blocks, args.n_threads, True)
                if rc != 0:
                    raise RuntimeError(f"{algo.name}: error {rc}")

            try:
                buf_out[:n_out].zero_()
                d.barrier()
                call()
                torch.cuda.synchronize()
                symm.check()
                ok = d.all_true(passes(buf_out[:n_out], ref, d.world))
                stats = error_stats(buf_out[:n_out], ref)
                eager = time_eager(d, call, iters, 5, check=symm.check) * 1e3
                graph = time_graph(d, call, reps=10 if size <= (16 << 20) else 4, replays=3, check=symm.check) * 1e3
                best = min(eager, graph)
                row["algorithms"][algo.name] = {"eager_us": round(eager, 2), "graph_us": round(graph, 2), "ok": ok,
                                                "max_abs_err": stats["max_abs"],
                                                "busbw_gbs": round(bus_bandwidth_gbs(args.collective, big * esize, d.world, best), 2)}
            except Exception as e:  # noqa: BLE001
                row["algorithms"][algo.name] = {"error": str(e)[:120]}
                try:
                    symm.heap.reset_status()
                except Exception:  # noqa: BLE001
                    pass
        good = {k: v for k, v in row["algorithms"].items() if "graph_us" in v}
        if good:
            name = min(good, key=lambda k: min(good[k]["eager_us"], good[k]["graph_us"]))
            row["best"] = name
            row["best_us"] = min(good[name]["eager_us"], good[name]["graph_us"])
            row["busbw_gbs"] = good[name]["busbw_gbs"]
        rows.append(row)
        if d.rank == 0 and not args.quiet:
            nccl = f" nccl {row.get('nccl_us', float('nan')):9.2f} us {row.get('nccl_busbw_gbs', 0):7.1f} GB/s" if d.world > 1 else ""
            print(f"{row['bytes']:>12} B  best {row.get('best', '-'):<38} {row.get('best_us', float('nan')):9.2f} us "
                  f"{row.get('busbw_gbs', 0):7.1f} GB/s{nccl}", flush=True)
        size *= args.step
    result = {"collective": args.collective, "dtype": args.dtype, "world": d.world, "nvls": bool(symm.nvls), "rows": rows}
    if d.rank == 0:
        if args.json:
            with open(args.json, "w") as f:
                json.dump(result, f, indent=1)
        print(json.dumps({"bench_collective": args.collective, "world": d.world, "sizes": len(rows),
                          "all_ok": all(v.get("ok", False) for r in rows for v in r["algorithms"].values() if "ok" in v)}), flush=True)
    d.barrier()
    executor.reset()
    symm.destroy()
    d.close()
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--collective", default="allreduce", choices=["allreduce", "allgather", "reducescatter"])
    p.add_argument("--dtype", default="bfloat16", choices=sorted(DTYPES))
    p.add_argument("--min-bytes", type=int, default=1024)
    p.add_argument("--max-bytes", type=int, default=256 << 20)
    p.add_argument("--step", type=int, default=4)
    p.add_argument("--algorithms", nargs="*", default=[])
    p.add_argument("--n-blocks", type=int, default=0)
    p.add_argument("--n-threads", type=int, default=0)
    p.add_argument("--json", default="")
    p.add_argument("--quiet", action="store_true")
    return run(p.parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
