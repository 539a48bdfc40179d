"""Shared plumbing of the benchmarks: process-group set-up, device timing, CUDA-graph timing."""
from __future__ import annotations

import os
from typing import Callable, Optional

import torch
import torch.distributed as dist


class Dist:
    """One process per GPU; world size 1 works without a launcher."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            dist.init_process_group("nccl", rank=self.rank, world_size=self.world, device_id=self.device)

    def barrier(self):
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, x: float) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], device=self.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok: bool) -> bool:
        if self.world == 1:
            return ok
        t = torch.tensor([1 if ok else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def close(self):
        if self.world > 1 and dist.is_initialized():
            dist.destroy_process_group()


_flush_buf = None


def flush_l2(device):
    """Overwrite a buffer larger than the 126 MB L2 so that the next timed launch starts cold."""
    global _flush_buf
    if _flush_buf is None or _flush_buf.device != device:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    _flush_buf.zero_()


def time_eager(d: Dist, fn: Callable[[], None], iters: int = 20, warmup: int = 5, check: Optional[Callable[[], None]] = None,
               flush: bool = False) -> float:
    """Milliseconds per call: CUDA events on the launching stream, barrier + synchronize on both sides, max over
    ranks. With flush=True every call is timed on its own after an L2 flush (slower, for inputs smaller than L2)."""
    for _ in range(warmup):
        fn()
    d.barrier()
    if flush:
        total = 0.0
        for _ in range(iters):
            flush_l2(d.device)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            d.barrier()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        ms = total / iters
    else:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        d.barrier()
        ms = s.elapsed_time(e) / iters
    if check is not None:
        check()
    return d.max(ms)


def time_graph(d: Dist, fn_on_stream: Callable[[torch.cuda.Stream], None], reps: int = 20, replays: int = 5,
               check: Optional[Callable[[], None]] = None) -> float:
    """Milliseconds per call with `reps` calls captured in one CUDA graph (no host launch cost between them)."""
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    d.barrier()
    with torch.cuda.stream(side):
        fn_on_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                fn_on_stream(side)
    d.barrier()
    graph.replay()  # warm-up replay
    d.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        graph.replay()
    e.record()
    d.barrier()
    if check is not None:
        check()
    return d.max(s.elapsed_time(e) / (replays * reps))


def hardware_profile(d: Dist, nvls: bool) -> str:
    name = torch.cuda.get_device_name(d.device).replace(" ", "_")
    return f"{name}-x{d.world}-{'nvls' if nvls else 'p2p'}"
