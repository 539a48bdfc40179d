"""Convert a tracer dump directory into a Chrome/Perfetto trace (`chrome://tracing` JSON).

    python -m mscclpp_b200.utils.npkit_trace --npkit_dump_dir DIR --output_dir OUT

Reads `gpu_events_rank_R_buf_B`, `cpu_events_rank_R_channel_C`, the clock files and `gpu_time_sync_rank_R`
written by `npkit.dump`, pairs ENTRY/EXIT events per buffer and writes `npkit_event_trace.json`. The reference
ships an equivalent tool (tools/npkit/npkit_trace_generator.py:11-290) that learns event names by parsing the
C header; here the names come from the same header shipped inside the package.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import struct
from typing import Dict, List

_EVENT_HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "include", "mscclpp", "npkit",
                             "npkit_event.hpp")

_OP_NAMES = ["NOP", "BARRIER", "SIGNAL", "RELAXED_SIGNAL", "WAIT", "RELAXED_WAIT", "FLUSH", "PUT", "PUT_WITH_SIGNAL",
             "PUT_WITH_SIGNAL_AND_FLUSH", "GET", "COPY", "REDUCE", "REDUCE_SEND", "READ_REDUCE", "READ_REDUCE_SEND", "PUT_PACKETS",
             "READ_PUT_PACKETS", "COPY_PACKETS", "UNPACK_PACKETS", "REDUCE_PACKETS", "REDUCE_SEND_PACKETS", "REDUCE_COPY_PACKETS",
             "REDUCE_COPY_SEND_PACKETS", "GROUP_LOAD_REDUCE_STORE", "GROUP_STORE", "GROUP_STORE_PACKETS", "SEM_ACQUIRE", "SEM_RELEASE",
             "PIPELINE_BEGIN", "PIPELINE_END"]


def parse_event_header(path: str = _EVENT_HEADER) -> Dict[int, str]:
    """id -> name, with the executor operation range expanded to one name per operation type."""
    ids: Dict[int, str] = {}
    base_entry = base_exit = None
    with open(path) as f:
        for line in f:
            m = re.match(r"#define\s+NPKIT_EVENT_(\w+)\s+(0x[0-9A-Fa-f]+)", line)
            if not m:
                continue
            name, value = m.group(1), int(m.group(2), 16)
            if name == "EXECUTOR_OP_BASE_ENTRY":
                base_entry = value
            elif name == "EXECUTOR_OP_BASE_EXIT":
                base_exit = value
            else:
                ids[value] = name
    if base_entry is not None and base_exit is not None:
        for i, op in enumerate(_OP_NAMES):
            ids[base_entry + i] = f"EXECUTOR_OP_{op}_ENTRY"
            ids[base_exit + i] = f"EXECUTOR_OP_{op}_EXIT"
    return ids


def parse_event(raw: bytes) -> dict:
    lo, ts = struct.unpack("<QQ", raw)
    return {"id": lo & 0xFF, "size": (lo >> 8) & 0xFFFFFFFF, "rsvd": (lo >> 40) & 0xFFFFFF, "timestamp": ts}


def _read_events(path: str) -> List[dict]:
    with open(path, "rb") as f:
        data = f.read()
    return [parse_event(data[i:i + 16]) for i in range(0, len(data) - 15, 16)]


def _pair(events: List[dict], names: Dict[int, str], to_us, pid: int, tid: str) -> List[dict]:
    """ENTRY/EXIT pairs become complete ('X') slices; everything else becomes an instant event."""
    out, stack = [], {}
    for e in events:
        name = names.get(e["id"], f"EVENT_{e['id']:#x}")
        ts = to_us(e["timestamp"])
        if name.endswith("_ENTRY"):
            stack.setdefault(name[:-6], []).append((ts, e))
        elif name.endswith("_EXIT") and stack.get(name[:-5]):
            t0, e0 = stack[name[:-5]].pop()
            dur = max(ts - t0, 0.0)
            args = {"size": e0["size"], "rsvd": e0["rsvd"]}
            if dur > 0 and e0["size"]:
                args["bw (GB/s)"] = e0["size"] / dur / 1e3
            out.append({"ph": "X", "name": name[:-5], "cat": "GPU" if tid.startswith("buf") else "CPU", "ts": t0, "dur": dur, "pid": pid,
                        "tid": tid, "args": args})
        else:
            out.append({"ph": "i", "name": name, "ts": ts, "pid": pid, "tid": tid, "s": "t", "args": {"size": e["size"]}})
    return out


def convert_npkit_dump_to_trace(npkit_dump_dir: str, output_dir: str, names: Dict[int, str] | None = None) -> str:
    names = names or parse_event_header()
    files = os.listdir(npkit_dump_dir)
    ranks = sorted({int(f.split("_rank_")[1].split("_")[0]) for f in files if f.startswith(("gpu_events_rank_", "cpu_events_rank_"))})
    trace: List[dict] = []
    for rank in ranks:
        with open(os.path.join(npkit_dump_dir, f"gpu_clock_rate_rank_{rank}")) as f:
            gpu_khz = float(f.read())
        with open(os.path.join(npkit_dump_dir, f"cpu_clock_period_num_rank_{rank}")) as f:
            num = float(f.read())
        with open(os.path.join(npkit_dump_dir, f"cpu_clock_period_den_rank_{rank}")) as f:
            den = float(f.read())
        sync_path = os.path.join(npkit_dump_dir, f"gpu_time_sync_rank_{rank}")
        gpu0 = cpu0 = 0
        if os.path.exists(sync_path):
            with open(sync_path) as f:
                gpu0, cpu0 = (int(v) for v in f.read().split())
        cpu_us = lambda t: t * num / den * 1e6  # noqa: E731
        gpu_us = lambda t: cpu_us(cpu0) + (t - gpu0) / gpu_khz * 1e3  # noqa: E731  (device ticks -> host time line)
        for f in sorted(files):
            if f.startswith(f"gpu_events_rank_{rank}_buf_"):
                buf = int(f.rsplit("_", 1)[1])
                trace += _pair(_read_events(os.path.join(npkit_dump_dir, f)), names, gpu_us, rank, f"buf{buf}")
            elif f.startswith(f"cpu_events_rank_{rank}_channel_"):
                ch = int(f.rsplit("_", 1)[1])
                trace += _pair(_read_events(os.path.join(npkit_dump_dir, f)), names, cpu_us, rank, f"channel{ch}")
    trace.sort(key=lambda e: e["ts"])
    os.makedirs(output_dir, exist_ok=True)
    out_path = os.path.join(output_dir, "npkit_event_trace.json")
    with open(out_path, "w") as f:
        json.dump({"traceEvents": trace, "displayTimeUnit": "ns"}, f)
    return out_path


def main(argv=None):
    parser = argparse.ArgumentParser()
    parser.add_argument("--npkit_dump_dir", required=True)
    parser.add_argument("--output_dir", required=True)
    args = parser.parse_args(argv)
    print(convert_npkit_dump_to_trace(args.npkit_dump_dir, args.output_dir))


if __name__ == "__main__":
    main()
