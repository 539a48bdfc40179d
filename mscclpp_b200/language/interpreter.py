"""CPU interpreter of JSON execution plans (numpy).

Runs every rank and every thread block of a plan on host arrays with the executor's semantics
(chunk -> byte mapping and op behaviour of src/core/executor/execution_plan.cc:478-668 and
src/core/include/execution_kernel.hpp:46-798), so that an algorithm written in the DSL can be checked
without a GPU, and so that the GPU executor has an oracle to be compared with.

Model:
  * thread blocks are coroutines scheduled round-robin; one blocks on wait / barrier / semaphore /
    packet flags and resumes when the condition holds; no progress by anybody = deadlock = error;
  * channel signals are counters (the k-th channel from rank a to rank b is paired with the k-th
    channel from b to a, as the executor pairs connections by per-peer tag order);
  * LL packets are payload bytes plus one validity flag per 8-byte word kept beside the scratch
    buffer; a packet read blocks until every word of its range carries the launch flag;
  * reductions accumulate in float32 inside one op and round to the element type once per op, which
    is what the sm_100a kernels of this library do (the reference sums in the element type).
"""
from __future__ import annotations

import json
import math
from typing import Dict, List, Optional, Sequence, Union

import numpy as np


class PlanError(RuntimeError):
    pass


class Deadlock(PlanError):
    pass


def calc_offset(size_units: int, index: int, parts: int, alignment: int) -> int:
    """Byte offset of chunk `index` when `size_units * alignment` bytes are split into `parts` chunks."""
    q, r = divmod(size_units, parts)
    return (index * q + min(index, r)) * alignment


_PKT_WORD = 8  # payload bytes that share one LL16 flag pair


class _RankMem:
    def __init__(self, inp: np.ndarray, out: np.ndarray, scratch_bytes: int):
        self.buf = {"i": inp.view(np.uint8).reshape(-1), "o": out.view(np.uint8).reshape(-1),
                    "s": np.zeros(scratch_bytes, dtype=np.uint8)}
        self.flags = np.zeros((scratch_bytes + _PKT_WORD - 1) // _PKT_WORD + 1, dtype=np.int64)


class PlanInterpreter:
    def __init__(self, plan: Union[str, dict]):
        self.plan = json.loads(plan) if isinstance(plan, str) else plan
        self.gpus = self.plan["gpus"]
        self.nranks = len(self.gpus)
        self.alignment = int(self.plan.get("buffer_alignment", 16))
        self.launches = 0
        self._pair_channels()

    # ------------------------------------------------------------------ static structure
    def _pair_channels(self):
        """mate[(type, rank, channel id)] = (peer rank, peer channel id)."""
        self.mate: Dict[tuple, tuple] = {}
        per_type: Dict[str, List[List[int]]] = {}
        for g in self.gpus:
            for ch in g["channels"]:
                if ch["channel_type"] in ("memory", "port"):
                    per_type.setdefault(ch["channel_type"], [[] for _ in range(self.nranks)])[g["id"]] = ch["connected_to"]
        for ctype, tables in per_type.items():
            for r, peers in enumerate(tables):
                seen: Dict[int, int] = {}
                for cid, p in enumerate(peers):
                    k = seen.get(p, 0)
                    seen[p] = k + 1
                    back = [i for i, q in enumerate(tables[p]) if q == r]
                    if k < len(back):
                        self.mate[(ctype, r, cid)] = (p, back[k])

    # ------------------------------------------------------------------ execution
    def run(self, inputs: Sequence[np.ndarray], outputs: Optional[Sequence[np.ndarray]] = None,
            max_steps: int = 50_000_000) -> List[np.ndarray]:
        """Execute one launch. inputs[r] / outputs[r] are rank r's buffers (same dtype). In-place plans
        may pass outputs=None, then outputs alias inputs. Returns the output arrays."""
        if len(inputs) != self.nranks:
            raise PlanError(f"plan has {self.nranks} ranks, got {len(inputs)} inputs")
        inplace = outputs is None
        if inplace:
            outputs = inputs
        self.dtype = inputs[0].dtype
        self.launches += 1
        self.flag = self.launches
        in_bytes, out_bytes = inputs[0].nbytes, outputs[0].nbytes
        g0 = self.gpus[0]
        if g0["input_chunks"] != 0:
            self.S, self.C = in_bytes, g0["input_chunks"]
        else:
            self.S, self.C = out_bytes, g0["output_chunks"]
        if g0["input_chunks"] and g0["output_chunks"] and not inplace:
            if in_bytes * g0["output_chunks"] != out_bytes * g0["input_chunks"]:
                raise PlanError("input and output sizes do not describe the same chunk size")
        if self.S % self.alignment:
            raise PlanError(f"message size {self.S} is not a multiple of the plan alignment {self.alignment}")
        chunk_upper = calc_offset(self.S // self.alignment, 1, self.C, self.alignment) if self.C else 0
        self.chunk_upper = max(chunk_upper, math.ceil(self.S / max(self.C, 1)))
        self.mem = [_RankMem(inputs[r], outputs[r], g["scratch_chunks"] * self.chunk_upper + 64)
                    for r, g in enumerate(self.gpus)]
        if not hasattr(self, "_persist"):
            self._persist = True
            self.inbound: Dict[tuple, int] = {}
            self.expected: Dict[tuple, int] = {}
        self.barrier_arrivals: Dict[tuple, int] = {}
        self.sems = {(g["id"], i): s["init_value"] for g in self.gpus for i, s in enumerate(g.get("semaphores", []))}

        tasks = []
        for g in self.gpus:
            for tb in g["threadblocks"]:
                tasks.append(self._run_tb(g, tb))
        steps = 0
        alive = list(tasks)
        while alive:
            progressed = False
            nxt = []
            for t in alive:
                try:
                    status = next(t)
                    if status == "progress":
                        progressed = True
                    nxt.append(t)
                except StopIteration:
                    progressed = True
            alive = nxt
            steps += 1
            if alive and not progressed:
                raise Deadlock(f"no thread block can make progress ({len(alive)} still blocked)")
            if steps > max_steps:
                raise PlanError("step limit exceeded")
        return list(outputs)

    # ------------------------------------------------------------------ operand resolution
    def _span(self, operand: dict, tbg: Optional[dict], it: Optional[tuple]):
        """(byte offset, byte length) of an operand in payload space."""
        a = self.alignment
        units = self.S // a
        start = calc_offset(units, operand["index"], self.C, a)
        end = calc_offset(units, operand["index"] + operand["size"], self.C, a)
        if tbg is not None:
            span_units = (end - start) // a
            s2 = calc_offset(span_units, tbg["tb_id"], tbg["tbg_size"], a)
            e2 = calc_offset(span_units, tbg["tb_id"] + 1, tbg["tbg_size"], a)
            start, end = start + s2, start + e2
        if it is not None:
            unit, i = it
            lo = min(start + i * unit, end)
            hi = min(lo + unit, end)
            start, end = lo, hi
        return start, end - start

    def _local(self, rank: int, operand: dict):
        return rank, operand["type"]

    def _remote(self, g: dict, tb: dict, op: dict, operand: dict):
        ctype = op.get("channel_type", "memory")
        refs = [r for r in tb["remote_buffer_refs"] if r["access_channel_type"] == ctype]
        if not refs:
            raise PlanError(f"thread block {tb['id']} of rank {g['id']} has no remote buffers for {ctype} channels")
        rb = g["remote_buffers"][refs[0]["remote_buffer_ids"][operand["buffer_id"]]]
        return rb["rank"], rb["type"]

    def _resolve(self, g, tb, op, operand):
        if "buffer_id" in operand:
            return self._remote(g, tb, op, operand)
        return self._local(g["id"], operand)

    def _bytes(self, rank: int, btype: str, off: int, n: int) -> np.ndarray:
        buf = self.mem[rank].buf[btype]
        if off < 0 or off + n > buf.size:
            raise PlanError(f"access [{off}, {off + n}) outside the {btype} buffer of rank {rank} ({buf.size} bytes)")
        return buf[off:off + n]

    def _typed(self, raw: np.ndarray) -> np.ndarray:
        return raw.view(self.dtype)

    def _tb_channel(self, tb: dict, ctype: str, local_idx: int) -> int:
        for ch in tb["channels"]:
            if ch["channel_type"] == ctype:
                return ch["channel_ids"][local_idx]
        raise PlanError(f"thread block {tb['id']} has no {ctype} channels")

    # ------------------------------------------------------------------ packets
    def _pkt_mark(self, rank: int, off: int, n: int):
        f = self.mem[rank].flags
        f[off // _PKT_WORD:(off + n + _PKT_WORD - 1) // _PKT_WORD] = self.flag

    def _pkt_ready(self, rank: int, off: int, n: int) -> bool:
        if n == 0:
            return True
        f = self.mem[rank].flags
        return bool(np.all(f[off // _PKT_WORD:(off + n + _PKT_WORD - 1) // _PKT_WORD] == self.flag))

    # ------------------------------------------------------------------ reductions
    def _reduce(self, parts: List[np.ndarray]) -> np.ndarray:
        if np.issubdtype(self.dtype, np.floating) and self.dtype != np.float64:
            acc = parts[0].astype(np.float32)
            for p in parts[1:]:
                acc = acc + p.astype(np.float32)
            return acc.astype(self.dtype)
        acc = parts[0].copy()
        for p in parts[1:]:
            acc = acc + p
        return acc

    # ------------------------------------------------------------------ thread block coroutine
    def _run_tb(self, g: dict, tb: dict):
        for op in tb["ops"]:
            yield from self._exec(g, tb, op, None)
            yield "progress"

    def _exec(self, g, tb, op, it):
        name = op["name"]
        rank = g["id"]
        tbg = op.get("tbg_info")
        src = op.get("src_buff", [])
        dst = op.get("dst_buff", [])

        def span(o):
            return self._span(o, tbg, it)

        if name == "nop":
            return
        if name == "pipeline":
            unit = op["iter_context"]["unit_size"]
            total = op["iter_context"]["num_chunks"] * self.chunk_upper
            iters = max(1, math.ceil(total / unit))
            for i in range(iters):
                for inner in op["ops"]:
                    yield from self._exec(g, tb, inner, (unit, i))
                    yield "progress"  # an inner op that completed may have unblocked another thread block
            return
        if name == "barrier":
            key = (rank, op["barrier_id"])
            n = op["num_threadblocks"]
            mine = self.barrier_arrivals.get(key, 0)
            self.barrier_arrivals[key] = mine + 1
            target = (mine // n + 1) * n
            while self.barrier_arrivals[key] < target:
                yield "blocked"
            return
        if name in ("signal", "rlxsignal"):
            ctype = op["channel_type"]
            for idx in op["channel_ids"]:
                cid = self._tb_channel(tb, ctype, idx)
                m = self.mate.get((ctype, rank, cid))
                if m is None:
                    raise PlanError(f"rank {rank} {ctype} channel {cid} has no counterpart on its peer")
                self.inbound[(ctype, m[0], m[1])] = self.inbound.get((ctype, m[0], m[1]), 0) + 1
            return
        if name in ("wait", "rlxwait"):
            ctype = op["channel_type"]
            for idx in op["channel_ids"]:
                key = (ctype, rank, self._tb_channel(tb, ctype, idx))
                self.expected[key] = self.expected.get(key, 0) + 1
                while self.inbound.get(key, 0) < self.expected[key]:
                    yield "blocked"
            return
        if name == "flush":
            return
        if name == "sem_acquire":
            for sid in op["semaphore_ids"]:
                while self.sems[(rank, sid)] <= 0:
                    yield "blocked"
                self.sems[(rank, sid)] -= 1
            return
        if name == "sem_release":
            for sid in op["semaphore_ids"]:
                self.sems[(rank, sid)] += 1
            return
        if name == "copy":
            (so, n), (do, _) = span(src[0]), span(dst[0])
            self._bytes(rank, dst[0]["type"], do, n)[:] = self._bytes(rank, src[0]["type"], so, n).copy()
            return
        if name in ("put", "pws", "pwsf"):
            for s, d in zip(src, dst):
                (so, n), (do, _) = span(s), span(d)
                dr, dt = self._resolve(g, tb, op, d)
                self._bytes(dr, dt, do, n)[:] = self._bytes(rank, s["type"], so, n).copy()
            if name != "put":
                ctype = op["channel_type"]
                for idx in op.get("channel_ids", []):
                    cid = self._tb_channel(tb, ctype, idx)
                    m = self.mate[(ctype, rank, cid)]
                    self.inbound[(ctype, m[0], m[1])] = self.inbound.get((ctype, m[0], m[1]), 0) + 1
            return
        if name == "get":
            for s, d in zip(src, dst):
                (so, n), (do, _) = span(s), span(d)
                sr, stype = self._resolve(g, tb, op, s)
                self._bytes(rank, d["type"], do, n)[:] = self._bytes(sr, stype, so, n).copy()
            return
        if name in ("re", "res", "rre", "rres"):
            parts = []
            n = None
            for s in src:
                so, n = span(s)
                sr, stype = self._resolve(g, tb, op, s)
                parts.append(self._typed(self._bytes(sr, stype, so, n)))
            result = self._reduce(parts)
            for d in dst:
                do, _ = span(d)
                dr, dt = self._resolve(g, tb, op, d)
                self._typed(self._bytes(dr, dt, do, n))[:] = result
            return
        if name == "ppkt":
            for i, d in enumerate(dst):
                s = src[i] if i < len(src) else src[0]
                (so, n), (do, _) = span(s), span(d)
                dr, dt = self._resolve(g, tb, op, d)
                self._bytes(dr, dt, do, n)[:] = self._bytes(rank, s["type"], so, n).copy()
                self._pkt_mark(dr, do, n)
            return
        if name == "rppkt":
            so, n = span(src[0])
            while not self._pkt_ready(rank, so, n):
                yield "blocked"
            data = self._bytes(rank, "s", so, n).copy()
            for d in dst:
                do, _ = span(d)
                dr, dt = self._resolve(g, tb, op, d)
                self._bytes(dr, dt, do, n)[:] = data
                self._pkt_mark(dr, do, n)
            return
        if name == "cpkt":
            (so, n), (do, _) = span(src[0]), span(dst[0])
            self._bytes(rank, "s", do, n)[:] = self._bytes(rank, src[0]["type"], so, n).copy()
            self._pkt_mark(rank, do, n)
            return
        if name == "upkt":
            (so, n), (do, _) = span(src[0]), span(dst[0])
            while not self._pkt_ready(rank, so, n):
                yield "blocked"
            self._bytes(rank, dst[0]["type"], do, n)[:] = self._bytes(rank, "s", so, n).copy()
            return
        if name in ("repkt", "respkt", "recpkt", "recspkt"):
            so0, n = span(src[0])
            parts = [self._typed(self._bytes(rank, src[0]["type"], so0, n))]
            for s in src[1:]:
                so, _ = span(s)
                while not self._pkt_ready(rank, so, n):
                    yield "blocked"
                parts.append(self._typed(self._bytes(rank, "s", so, n)))
            result = self._reduce(parts)
            do, _ = span(dst[0])
            self._typed(self._bytes(rank, dst[0]["type"], do, n))[:] = result
            rest = dst[1:]
            if name in ("recpkt", "recspkt") and rest:
                do, _ = span(rest[0])
                self._typed(self._bytes(rank, "s", do, n))[:] = result
                self._pkt_mark(rank, do, n)
                rest = rest[1:]
            for d in rest:
                do, _ = span(d)
                dr, dt = self._resolve(g, tb, op, d)
                self._typed(self._bytes(dr, dt, do, n))[:] = result
                self._pkt_mark(dr, do, n)
            return
        if name in ("glres", "gstore", "gstorepkt"):
            def switch(o):
                cid = self._tb_channel(tb, "switch", o["switch_channel_id"])
                chans = [c for c in g["channels"] if c["channel_type"] == "switch"]
                ch = chans[cid]
                return ch.get("buffer_type", ch.get("buff")), ch["rank_groups"][0]["ranks"]  # "buff": older plan files
            if name == "glres":
                btype, ranks = switch(src[0])
                so, n = span(src[0])
                result = self._reduce([self._typed(self._bytes(r, btype, so, n)) for r in ranks])
                dbt, dranks = switch(dst[0])
                do, _ = span(dst[0])
                for r in dranks:
                    self._typed(self._bytes(r, dbt, do, n))[:] = result
                return
            so, n = span(src[0])
            if name == "gstorepkt":
                while not self._pkt_ready(rank, so, n):
                    yield "blocked"
            data = self._bytes(rank, src[0]["type"], so, n).copy()
            dbt, dranks = switch(dst[0])
            do, _ = span(dst[0])
            for r in dranks:
                self._bytes(r, dbt, do, n)[:] = data
                if name == "gstorepkt":
                    self._pkt_mark(r, do, n)
            return
        raise PlanError(f"unknown op '{name}'")


# ---------------------------------------------------------------------- static checks
KNOWN_OPS = {"nop", "copy", "cpkt", "upkt", "re", "repkt", "recpkt", "sem_acquire", "sem_release", "signal", "wait",
             "rlxsignal", "rlxwait", "barrier", "flush", "get", "put", "ppkt", "rppkt", "pws", "pwsf", "res", "respkt",
             "recspkt", "rre", "rres", "gstore", "gstorepkt", "glres", "pipeline"}


def validate_plan(plan: Union[str, dict]) -> None:
    """Structural checks run before a plan is handed to any executor: known op names, chunk indices
    inside their buffers, channel / remote-buffer / semaphore references in range, signal and wait
    counts that pair up per channel. Raises PlanError with the first problem found."""
    p = json.loads(plan) if isinstance(plan, str) else plan
    for key in ("name", "collective", "protocol", "gpus"):
        if key not in p:
            raise PlanError(f"plan is missing '{key}'")
    if p["protocol"] not in ("Simple", "LL"):
        raise PlanError(f"unknown protocol {p['protocol']}")
    nranks = len(p["gpus"])
    sig: Dict[tuple, int] = {}
    wai: Dict[tuple, int] = {}
    interp = PlanInterpreter(p)
    for g in p["gpus"]:
        limits = {"i": g["input_chunks"], "o": g["output_chunks"], "s": g["scratch_chunks"]}
        if p.get("inplace"):
            limits["i"] = limits["o"] = max(limits["i"], limits["o"])
        nsem = len(g.get("semaphores", []))
        for ch in g["channels"]:
            if ch["channel_type"] in ("memory", "port"):
                for peer in ch["connected_to"]:
                    if not 0 <= peer < nranks or peer == g["id"]:
                        raise PlanError(f"rank {g['id']}: channel to invalid rank {peer}")
        for tb in g["threadblocks"]:
            chan_counts = {c["channel_type"]: len(c["channel_ids"]) for c in tb["channels"]}
            ref_counts = {r["access_channel_type"]: len(r["remote_buffer_ids"]) for r in tb.get("remote_buffer_refs", [])}

            def check_ops(ops):
                for op in ops:
                    name = op["name"]
                    if name not in KNOWN_OPS:
                        raise PlanError(f"rank {g['id']} tb {tb['id']}: unknown op '{name}'")
                    if name == "pipeline":
                        if op["iter_context"]["unit_size"] <= 0:
                            raise PlanError("pipeline with a non-positive unit size")
                        check_ops(op["ops"])
                        continue
                    ctype = op.get("channel_type")
                    for cid in op.get("channel_ids", []):
                        if name in ("glre",):
                            continue
                        if ctype and cid >= chan_counts.get(ctype, 0):
                            raise PlanError(f"rank {g['id']} tb {tb['id']} {name}: channel index {cid} out of range")
                    for sid in op.get("semaphore_ids", []):
                        if sid >= nsem:
                            raise PlanError(f"rank {g['id']} tb {tb['id']} {name}: semaphore {sid} out of range")
                    for operand in op.get("src_buff", []) + op.get("dst_buff", []):
                        if "buffer_id" in operand:
                            if operand["buffer_id"] >= ref_counts.get(ctype or "memory", 0):
                                raise PlanError(f"rank {g['id']} tb {tb['id']} {name}: remote buffer index out of range")
                            rb = g["remote_buffers"][[r for r in tb["remote_buffer_refs"] if r["access_channel_type"] == (ctype or "memory")][0]["remote_buffer_ids"][operand["buffer_id"]]]
                            peer = p["gpus"][rb["rank"]]
                            lim = {"i": peer["input_chunks"], "o": peer["output_chunks"], "s": peer["scratch_chunks"]}
                            if p.get("inplace"):
                                lim["i"] = lim["o"] = max(lim["i"], lim["o"])
                            if operand["index"] + operand["size"] > lim[rb["type"]]:
                                raise PlanError(f"rank {g['id']} tb {tb['id']} {name}: remote chunk range outside rank {rb['rank']}'s buffer")
                        elif "switch_channel_id" in operand:
                            if operand["switch_channel_id"] >= chan_counts.get("switch", 0):
                                raise PlanError(f"rank {g['id']} tb {tb['id']} {name}: switch channel index out of range")
                        else:
                            if operand["index"] < 0 or operand["index"] + operand["size"] > limits[operand["type"]]:
                                raise PlanError(f"rank {g['id']} tb {tb['id']} {name}: chunk range "
                                                f"[{operand['index']}, {operand['index'] + operand['size']}) outside buffer "
                                                f"'{operand['type']}' ({limits[operand['type']]} chunks)")
                    if name in ("signal", "rlxsignal", "pws", "pwsf", "wait", "rlxwait") and ctype in ("memory", "port"):
                        for idx in op.get("channel_ids", []):
                            cid = [c for c in tb["channels"] if c["channel_type"] == ctype][0]["channel_ids"][idx]
                            if name in ("wait", "rlxwait"):
                                wai[(ctype, g["id"], cid)] = wai.get((ctype, g["id"], cid), 0) + 1
                            else:
                                m = interp.mate.get((ctype, g["id"], cid))
                                if m is None:
                                    raise PlanError(f"rank {g['id']}: {ctype} channel {cid} has no counterpart")
                                sig[(ctype, m[0], m[1])] = sig.get((ctype, m[0], m[1]), 0) + 1
            check_ops(tb["ops"])
    for key in set(sig) | set(wai):
        if sig.get(key, 0) != wai.get(key, 0):
            raise PlanError(f"{key[0]} channel {key[2]} of rank {key[1]}: {sig.get(key, 0)} signal(s) arrive but "
                            f"{wai.get(key, 0)} wait(s) are issued")
