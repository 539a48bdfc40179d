"""Store of tuned launch configurations, keyed by hardware profile, collective, dtype and message size
(reference: python/mscclpp_benchmark/tuning_config.py:17-99 keeps the same kind of JSON store).

File layout: {"<profile>": {"<collective>/<dtype>": [{"max_bytes": N, "algorithm": str, "n_blocks": int,
"n_threads": int, "us": float}, ...sorted by max_bytes]}}. `lookup` returns the first entry whose max_bytes covers
the message.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional


class TuningConfig:
    def __init__(self, path: Optional[str] = None):
        self.path = path
        self.data: Dict[str, Dict[str, List[dict]]] = {}
        if path and os.path.exists(path):
            with open(path) as f:
                self.data = json.load(f)

    def record(self, profile: str, collective: str, dtype: str, max_bytes: int, algorithm: str, n_blocks: int, n_threads: int,
               us: float) -> None:
        rows = self.data.setdefault(profile, {}).setdefault(f"{collective}/{dtype}", [])
        rows[:] = [r for r in rows if r["max_bytes"] != max_bytes]
        rows.append({"max_bytes": int(max_bytes), "algorithm": algorithm, "n_blocks": int(n_blocks), "n_threads": int(n_threads),
                     "us": round(float(us), 3)})
        rows.sort(key=lambda r: r["max_bytes"])

    def lookup(self, profile: str, collective: str, dtype: str, nbytes: int) -> Optional[dict]:
        rows = self.data.get(profile, {}).get(f"{collective}/{dtype}", [])
        for r in rows:
            if nbytes <= r["max_bytes"]:
                return r
        return rows[-1] if rows else None

    def record_bench_result(self, profile: str, result: dict) -> int:
        """Takes the best algorithm of every size from a `bench_collective --json` result (default launch shapes). Returns
        the number of sizes recorded. The stores shipped in `benchmark/baselines/tuned_b200.json` were made this way from
        the measured ladders."""
        n = 0
        for row in result.get("rows", []):
            if "best" not in row:
                continue
            self.record(profile, result["collective"], result["dtype"], row["bytes"], row["best"], 0, 0, row["best_us"])
            n += 1
        return n

    @staticmethod
    def shipped() -> "TuningConfig":
        """The store measured on B200 machines of 2, 4 and 8 GPUs that comes with the package."""
        return TuningConfig(os.path.join(os.path.dirname(os.path.abspath(__file__)), "baselines", "tuned_b200.json"))

    def save(self, path: Optional[str] = None) -> str:
        path = path or self.path
        if not path:
            raise ValueError("no path to save the tuning configuration to")
        tmp = f"{path}.tmp.{os.getpid()}"
        with open(tmp, "w") as f:
            json.dump(self.data, f, indent=1, sort_keys=True)
        os.replace(tmp, path)
        return path

    def make_selector(self, profile: str):
        """An algorithm selector (for `AlgorithmCollectionBuilder.set_algorithm_selector`) that follows the store."""
        names = {"float16": "float16", "bfloat16": "bfloat16", "float32": "float32"}

        def selector(algo_map, request):
            dtype = names.get(getattr(request.dtype, "name", str(request.dtype)), "bfloat16")
            row = self.lookup(profile, request.collective, dtype, request.message_size)
            if row is None:
                return None
            return algo_map.get(request.collective, {}).get(row["algorithm"])

        return selector
