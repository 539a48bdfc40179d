"""Performance-regression gate for the collective sweep.

    python -m torch.distributed.run --nproc-per-node 8 -m mscclpp_b200.benchmark.bench_collective --json sweep.json
    python -m mscclpp_b200.benchmark.check_perf sweep.json [--baseline FILE.jsonl] [--latency-tol 0.15] [--bandwidth-tol 0.05]

Every size of the result is compared with the baseline entry of the same collective, world size and byte count:
small messages (below `--split-bytes`, 1 MiB by default) by time, which may be at most `latency-tol` slower; large ones by
bus bandwidth, which may be at most `bandwidth-tol` lower. Exit code 0 = no regression, 1 = at least one, 2 = nothing
could be compared. Baselines are JSON-lines files (one size per line); the ones measured on B200s ship in
`mscclpp_b200/benchmark/baselines/`. Same idea and tolerances as the reference's perf gate
(test/deploy/run_tests.sh:21-63, test/mscclpp-test/check_perf_result.py:26-56).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, Iterable, List, Tuple

BASELINE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baselines")
Key = Tuple[str, int, int]


def load_baseline(path: str) -> Dict[Key, dict]:
    table: Dict[Key, dict] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            row = json.loads(line)
            table[(row["collective"], int(row["world"]), int(row["bytes"]))] = row
    return table


def result_rows(result: dict) -> Iterable[dict]:
    """Rows of a bench_collective --json file, or of a list of {collective, world, bytes, time_us, busbw_gbs}."""
    if isinstance(result, list):
        yield from result
        return
    for row in result.get("rows", []):
        if "best_us" not in row:
            continue
        yield {"collective": result["collective"], "world": result["world"], "bytes": row["bytes"], "time_us": row["best_us"],
               "busbw_gbs": row.get("busbw_gbs", 0.0)}


def default_baseline(collective: str, world: int, dtype: str = "bf16") -> str:
    return os.path.join(BASELINE_DIR, f"b200_{world}gpu_{collective}_{dtype}.jsonl")


def compare(rows: Iterable[dict], baseline: Dict[Key, dict], latency_tol: float = 0.15, bandwidth_tol: float = 0.05,
            split_bytes: int = 1 << 20) -> Tuple[List[dict], int]:
    """Returns (report lines, number of compared sizes). A report line has `status` ok | regression | missing."""
    report, compared = [], 0
    for row in rows:
        key = (row["collective"], int(row["world"]), int(row["bytes"]))
        base = baseline.get(key)
        if base is None:
            report.append({"bytes": key[2], "status": "missing"})
            continue
        compared += 1
        if key[2] < split_bytes:
            limit = base["time_us"] * (1.0 + latency_tol)
            bad = row["time_us"] > limit
            report.append({"bytes": key[2], "status": "regression" if bad else "ok", "metric": "time_us", "value": row["time_us"],
                           "baseline": base["time_us"], "limit": round(limit, 3)})
        else:
            limit = base["busbw_gbs"] * (1.0 - bandwidth_tol)
            bad = row["busbw_gbs"] < limit
            report.append({"bytes": key[2], "status": "regression" if bad else "ok", "metric": "busbw_gbs", "value": row["busbw_gbs"],
                           "baseline": base["busbw_gbs"], "limit": round(limit, 3)})
    return report, compared


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("result", help="bench_collective --json output")
    p.add_argument("--baseline", default="", help="JSON-lines baseline (default: the shipped file for this collective and world size)")
    p.add_argument("--latency-tol", type=float, default=0.15)
    p.add_argument("--bandwidth-tol", type=float, default=0.05)
    p.add_argument("--split-bytes", type=int, default=1 << 20)
    args = p.parse_args(argv)
    with open(args.result) as f:
        result = json.load(f)
    rows = list(result_rows(result))
    if not rows:
        print("no timed sizes in the result", file=sys.stderr)
        return 2
    # the shipped baseline of the result's element type when there is one (bf16 for every world size, fp16 for some)
    short = {"bfloat16": "bf16", "float16": "fp16", "float32": "fp32"}.get(result.get("dtype", "bfloat16") if isinstance(result, dict) else "bfloat16", "bf16")
    path = args.baseline or default_baseline(rows[0]["collective"], int(rows[0]["world"]), short)
    if not args.baseline and not os.path.exists(path):
        path = default_baseline(rows[0]["collective"], int(rows[0]["world"]))
    if not os.path.exists(path):
        print(f"no baseline file {path}", file=sys.stderr)
        return 2
    report, compared = compare(rows, load_baseline(path), args.latency_tol, args.bandwidth_tol, args.split_bytes)
    for line in report:
        print(json.dumps(line))
    if compared == 0:
        return 2
    return 1 if any(line["status"] == "regression" for line in report) else 0


if __name__ == "__main__":
    sys.exit(main())
