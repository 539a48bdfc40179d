"""Run one execution plan (a JSON file written by the DSL) through the Executor, check the result and time it.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m mscclpp_b200.benchmark.executor_test \
        -path plan.json --size 32M [--in_place] [--dtype float16] [--packet_type LL16] [--n_iters 10] [--n_graph_iters 10]
    python -m mscclpp_b200.benchmark.executor_test -path plan.json --size 1M --emulate     # all ranks of the plan on one GPU

The input of every rank is filled from a seed that depends on the rank; the expected output comes from the numpy plan
interpreter run on the same inputs (exact for integers, tolerance for floats), so any plan can be checked, not only the
standard collectives. Timing replays a CUDA graph of `n_iters` executions `n_graph_iters` times (device time, max over
ranks; with --emulate the same number of plain launches). Same role and flags as the reference's python/test/executor_test.py:63-125.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from typing import List, Tuple

import numpy as np

NP_DTYPES = {"float32": np.float32, "float16": np.float16, "int32": np.int32}


def parse_size(text: str) -> int:
    """'4096', '32K', '1M', '2G' (powers of 1024, case-insensitive, optional trailing B)."""
    m = re.fullmatch(r"\s*(\d+)\s*([kmg]?)b?\s*", text.lower())
    if not m:
        raise ValueError(f"bad size: {text!r}")
    return int(m.group(1)) << {"": 0, "k": 10, "m": 20, "g": 30}[m.group(2)]


def buffer_elems(collective: str, size_bytes: int, world: int, itemsize: int, in_place: bool) -> Tuple[int, int]:
    """(input elements, output elements) per rank for a message of `size_bytes` (the full-size buffer of the collective).
    In-place allgather / reducescatter use one buffer of the full size: each rank's own chunk is the input / the result."""
    total = size_bytes // itemsize
    total -= total % max(1, world)
    if total <= 0:
        raise ValueError("size too small for this world size and dtype")
    if collective == "allgather":
        return (total, total) if in_place else (total // world, total)
    if collective == "reducescatter":
        return (total, total) if in_place else (total, total // world)
    return total, total  # allreduce, alltoall, broadcast, and anything else: same size in and out


def make_inputs(world: int, elems: int, np_dtype, seed: int = 0) -> List[np.ndarray]:
    out = []
    for r in range(world):
        rng = np.random.default_rng(seed * 1000 + r)
        if np_dtype == np.int32:
            out.append(rng.integers(-1000, 1000, size=elems).astype(np_dtype))
        else:
            out.append(rng.uniform(-1, 1, size=elems).astype(np_dtype))
    return out


def expected_outputs(plan_json: str, inputs: List[np.ndarray], out_elems: int, in_place: bool) -> List[np.ndarray]:
    from ..language.interpreter import PlanInterpreter

    outs = None if in_place else [np.zeros(out_elems, dtype=inputs[0].dtype) for _ in inputs]
    return PlanInterpreter(plan_json).run([a.copy() for a in inputs], outs)


def matches(got: np.ndarray, expect: np.ndarray) -> bool:
    if got.dtype == np.int32:
        return bool(np.array_equal(got, expect))
    tol = 2e-3 if got.dtype == np.float32 else 2e-2
    return bool(np.allclose(got.astype(np.float32), expect.astype(np.float32), rtol=tol, atol=tol))


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("-path", "--execution_plan_path", required=True)
    p.add_argument("--size", required=True, help="message size, e.g. 4096, 32K, 1M")
    p.add_argument("--in_place", action="store_true")
    p.add_argument("--dtype", default="float16", choices=sorted(NP_DTYPES))
    p.add_argument("--packet_type", default="LL16", choices=["LL8", "LL16"])
    p.add_argument("--n_iters", type=int, default=10)
    p.add_argument("--n_graph_iters", type=int, default=10)
    p.add_argument("--emulate", action="store_true", help="run every rank of the plan on this one GPU")
    args = p.parse_args(argv)

    import torch

    from .. import SymmetricMemory, native
    from .common import Dist, time_graph

    n = native()
    plan_json = open(args.execution_plan_path).read()
    meta = json.loads(plan_json)
    collective = meta.get("collective", "allreduce")
    np_dtype = NP_DTYPES[args.dtype]
    tdtype = {"float32": torch.float32, "float16": torch.float16, "int32": torch.int32}[args.dtype]
    ndtype = {"float32": n.DataType.float32, "float16": n.DataType.float16, "int32": n.DataType.int32}[args.dtype]
    size = parse_size(args.size)
    itemsize = np.dtype(np_dtype).itemsize

    d = Dist() if not args.emulate else None
    plan0 = n.ExecutionPlan.from_string(plan_json, 0)
    world = plan0.n_ranks
    if d is not None and d.world != world:
        raise SystemExit(f"the plan is for {world} ranks, launched with {d.world}")
    rank = d.rank if d is not None else 0
    in_elems, out_elems = buffer_elems(collective, size, world, itemsize, args.in_place)
    heap_bytes = max(256 << 20, 4 * (in_elems + out_elems) * itemsize + (64 << 20))
    symm = SymmetricMemory.emulated(world, nbytes=heap_bytes, timeout_ms=5000) if args.emulate else SymmetricMemory.from_env(nbytes=heap_bytes)
    t_in = symm.tensor((in_elems,), tdtype)
    t_out = t_in if args.in_place else symm.tensor((out_elems,), tdtype)
    inputs = make_inputs(world, in_elems, np_dtype)
    expect = expected_outputs(plan_json, inputs, out_elems, args.in_place)
    if args.emulate:
        for r in range(world):
            symm.rank_view(t_in, r).copy_(torch.from_numpy(inputs[r]))
            if not args.in_place:
                symm.rank_view(t_out, r).zero_()
    else:
        t_in.copy_(torch.from_numpy(inputs[rank]))
        if not args.in_place:
            t_out.zero_()
        d.barrier()
    executor = n.Executor(symm.heap)
    plan = plan0 if rank == 0 else n.ExecutionPlan.from_string(plan_json, rank)
    packet = getattr(n.PacketType, args.packet_type)

    def call(stream=None):
        st = (stream or torch.cuda.current_stream()).cuda_stream
        executor.execute(rank, t_in.data_ptr(), t_out.data_ptr(), in_elems * itemsize, out_elems * itemsize, ndtype, plan, st, packet)

    call()
    torch.cuda.synchronize()
    symm.check()
    if args.emulate:
        ok = all(matches(symm.rank_view(t_out, r).cpu().numpy(), expect[r]) for r in range(world))
    else:
        ok = d.all_true(matches(t_out.cpu().numpy(), expect[rank]))

    us = float("nan")
    if ok and args.n_iters > 0 and not args.in_place:
        # (an in-place plan changes its own input, so repeated runs are timed only for out-of-place plans)
        if args.emulate:
            # all ranks in one cooperative launch: timed as plain launches (events around n_iters x n_graph_iters calls)
            for _ in range(2):
                call()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(args.n_iters * args.n_graph_iters):
                call()
            e.record()
            torch.cuda.synchronize()
            us = s.elapsed_time(e) / (args.n_graph_iters * args.n_iters) * 1e3
        else:
            us = time_graph(d, call, reps=args.n_iters, replays=args.n_graph_iters, check=symm.check) * 1e3
        symm.check()
    if rank == 0:
        print(json.dumps({"plan": meta.get("name", ""), "collective": collective, "world": world, "bytes": size, "dtype": args.dtype,
                          "in_place": args.in_place, "correct": ok, "us_per_execution": None if us != us else round(us, 2),
                          "emulated": bool(args.emulate)}), flush=True)
    executor.reset()
    symm.destroy()
    if d is not None:
        d.close()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
