"""Reference arm of bench.py: the UNMODIFIED reference library (microsoft/mscclpp, built with CMake into
baseline/_ref) on its stock PyTorch path.

The reference is a communication library; its documented way into a PyTorch program is to stand in for NCCL
(LD_PRELOAD of libmscclpp_nccl.so, with MSCCLPP_NCCL_LIB_PATH naming the real NCCL for the calls it does not
implement; docs/quickstart.md "NCCL over MSCCL++", test/torch/correctness_test.py). A tensor-parallel layer built
on it is therefore

    p = torch.matmul(x, w.t())            # cuBLAS
    dist.all_reduce(p)                    # reference: ncclAllReduce -> its algorithm selector -> its kernels
    h = p + residual ; out = rms_norm(h)  # PyTorch

which is what this file times, at the same shapes, steps, warm-up and host<->device copies as the other arm of
bench.py. Nothing of the mscclpp_b200 package is imported here.

bench.py re-executes the interpreter on this file with the preload in place; it is not meant to be run by hand
(without the preload it would time plain NCCL and says so in its output).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

HIDDEN = 8192
K_SHARD = 1024
HEADLINE_T = 8192
TOKEN_SIZES = (1, 8, 128, 2048, 8192)
REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU every 200 ms (same fields as the other arm)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms",
                                          "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True, env={k: v for k, v in os.environ.items() if k not in ("LD_PRELOAD", "LD_AUDIT")})
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 8:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(names, r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}


def loaded_reference_libraries() -> list:
    libs = set()
    try:
        with open("/proc/self/maps") as f:
            for line in f:
                path = line.split()[-1] if "/" in line else ""
                if path.endswith(".so") or ".so." in path:
                    if os.path.realpath(path).startswith(os.path.realpath(REF_DIR)):
                        libs.add(os.path.basename(path))
    except OSError:
        pass
    return sorted(libs)


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--no-sweep", action="store_true")
    p.add_argument("--sweep-max-bytes", type=int, default=256 << 20)
    args = p.parse_args()

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29877")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    warmup = max(args.warmup, 3)

    # data plane: the "nccl" backend, whose NCCL symbols the preloaded reference library provides.
    # control plane (barriers, max over ranks): gloo, so that no bookkeeping call depends on which reduce ops and
    # dtypes the reference implements.
    dist.init_process_group("nccl", rank=rank, world_size=world)
    ctl = dist.new_group(backend="gloo")

    def barrier():
        torch.cuda.synchronize()
        dist.barrier(group=ctl)
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctl)
        return float(t.item())

    def time_steps(fn, steps, warm):
        for _ in range(warm):
            fn()
        barrier()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        return max_over_ranks(start.elapsed_time(end) / steps)  # ms per step

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    xs = {t: torch.randn((t, K_SHARD), generator=g, device=dev).to(torch.bfloat16) for t in TOKEN_SIZES}
    gw = torch.Generator(device=dev).manual_seed(rank)
    weight = (torch.randn((HIDDEN, K_SHARD), generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    gres = torch.Generator(device=dev).manual_seed(99)
    residual = torch.randn((HEADLINE_T, HIDDEN), generator=gres, device=dev).to(torch.bfloat16)
    gamma = torch.ones((HIDDEN,), dtype=torch.bfloat16, device=dev)
    w_t = weight.t()

    def layer(x, res):
        part = torch.matmul(x, w_t)
        dist.all_reduce(part)  # world 1: the reference returns at once (in place, nothing to copy)
        h = part + res
        return torch.nn.functional.rms_norm(h, (HIDDEN,), gamma, 1e-5), h

    # ---- the allreduce really is a sum over ranks (checked once, small and large message)
    check = {}
    for n in (4096, 4 << 20):
        t = torch.full((n,), float(rank + 1), dtype=torch.bfloat16, device=dev)
        dist.all_reduce(t)
        torch.cuda.synchronize()
        check[str(n * 2)] = bool((t.float() == world * (world + 1) / 2).all().item())
    barrier()

    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    if rank == 0:
        sampler.start()
    head = lambda: layer(xs[HEADLINE_T], residual)
    ms_per_step = time_steps(head, args.steps, warmup)

    tp_us, tp_graph_us = {}, {}
    side = torch.cuda.Stream()
    graphs_ok = True
    for t in TOKEN_SIZES:
        fn = lambda t=t: layer(xs[t], residual[:t])
        tp_us[str(t)] = round(time_steps(fn, max(10, args.steps), 5) * 1e3, 2)
        if not graphs_ok:
            continue
        try:
            reps = 10
            graph = torch.cuda.CUDAGraph()
            barrier()
            with torch.cuda.stream(side):
                fn()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(reps):
                        fn()
            barrier()
            tp_graph_us[str(t)] = round(time_steps(graph.replay, 5, 2) * 1e3 / reps, 2)
            del graph
        except Exception as e:  # noqa: BLE001
            # the reference refuses some algorithms under stream capture; the eager numbers above stay valid
            tp_graph_us[str(t)] = f"error: {str(e)[:80]}"
            graphs_ok = False

    # ---- end to end: pinned host -> device copy of the step's input, the layer, 4-byte result back, every step
    x_host = torch.randn((HEADLINE_T, K_SHARD)).to(torch.bfloat16).pin_memory()
    x_dev = torch.empty_like(x_host, device=dev)
    result_host = torch.empty((1,), dtype=torch.float32).pin_memory()

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        out, _ = layer(x_dev, residual)
        result_host.copy_(out[-1].sum(dtype=torch.float32).reshape(1), non_blocking=True)  # one small kernel on the last row
        torch.cuda.current_stream().synchronize()

    t_end = time.time() + 1.5
    while time.time() < t_end:
        for _ in range(20):
            head()
        torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop() if rank == 0 else {}
    # timed with the clock sampler stopped (a driver query by nvidia-smi inside a host-synchronised step stalls it)
    e2e_ms = time_steps(e2e_step, args.steps, warmup)

    # ---- allreduce sweep through the same path (ordinary torch tensors, in place), eager and CUDA-graph replay
    sweep = []
    if world > 1 and not args.no_sweep:
        buf = torch.empty((args.sweep_max_bytes // 2,), dtype=torch.bfloat16, device=dev).normal_()
        size = 1024
        graphs_ok = True  # small messages capture fine even where a large layer did not
        while size <= args.sweep_max_bytes:
            n = size // 2
            iters = 50 if size <= (1 << 20) else (20 if size <= (64 << 20) else 8)
            row = {"bytes": size}
            ms = time_steps(lambda: dist.all_reduce(buf[:n]), iters, 5)
            row["us"] = round(ms * 1e3, 2)
            row["busbw_gbs"] = round(size * 2 * (world - 1) / world / (ms * 1e-3) / 1e9, 2)
            if graphs_ok and size <= (16 << 20):
                try:
                    reps = 20
                    graph = torch.cuda.CUDAGraph()
                    barrier()
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side):
                            for _ in range(reps):
                                dist.all_reduce(buf[:n])
                    barrier()
                    row["graph_us"] = round(time_steps(graph.replay, 5, 2) * 1e3 / reps, 2)
                    del graph
                except Exception as e:  # noqa: BLE001
                    row["graph_err"] = str(e)[:80]
                    graphs_ok = False
            sweep.append(row)
            size *= 2

    if rank == 0:
        us = ms_per_step * 1e3
        preload = os.environ.get("LD_PRELOAD", "")
        line = {
            "impl": "reference",
            "metric": "fused_tp_layer_us (GEMM [T,1024]x[1024,8192] + allreduce + residual + RMSNorm, T=8192)",
            "value": round(us, 2),
            "unit": "us",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": False,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic (N(0,1) activations, N(0,0.02) random-init weights)",
            "config": {"model": "Llama-3-70B attention out-proj shard", "global_batch": HEADLINE_T, "seq_len": HEADLINE_T,
                       "parallelism": f"tp{world}", "hidden": HIDDEN, "k_per_rank": K_SHARD, "eps": 1e-5,
                       "l2": "working set 560 MB per step > 126 MB L2, no explicit flush",
                       "composition": "torch.matmul (cuBLAS) + dist.all_reduce through the reference's NCCL shim + torch add + rms_norm"},
            "tokens_per_s": round(HEADLINE_T / (ms_per_step * 1e-3), 1),
            "tp_layer_us": tp_us,
            "tp_layer_graph_replay_us": tp_graph_us,
            "e2e": {"value": round(e2e_ms * 1e3, 2), "unit": "us", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": None,
            "clocks": clocks,
            "allreduce_sweep": sweep,
            "allreduce_value_check": check,
            "reference_native_so": loaded_reference_libraries(),
            "preload": os.path.basename(preload) if preload else "none (plain NCCL was timed)",
        }
        print(json.dumps(line), flush=True)
    barrier()
    sys.stdout.flush()
    # every rank is idle here; should the teardown of the preloaded library stall, leave without it
    watchdog = threading.Timer(30.0, os._exit, (0,))
    watchdog.daemon = True
    watchdog.start()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
