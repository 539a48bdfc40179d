"""The perf-regression gate: tolerances, small/large split, missing sizes, exit codes."""
import json

from mscclpp_b200.benchmark import check_perf


def _baseline(tmp_path):
    path = tmp_path / "base.jsonl"
    rows = [{"collective": "allreduce", "world": 8, "bytes": 1024, "time_us": 10.0, "busbw_gbs": 0.2},
            {"collective": "allreduce", "world": 8, "bytes": 1 << 26, "time_us": 170.0, "busbw_gbs": 700.0}]
    path.write_text("# comment\n" + "\n".join(json.dumps(r) for r in rows) + "\n")
    return str(path)


def _result(tmp_path, small_us, large_bw, extra=False):
    rows = [{"bytes": 1024, "best_us": small_us, "busbw_gbs": 0.1, "algorithms": {}},
            {"bytes": 1 << 26, "best_us": 180.0, "busbw_gbs": large_bw, "algorithms": {}}]
    if extra:
        rows.append({"bytes": 4096, "best_us": 11.0, "busbw_gbs": 0.5, "algorithms": {}})
        rows.append({"bytes": 8192, "algorithms": {}})  # a size that no algorithm could run: not compared
    path = tmp_path / "res.json"
    path.write_text(json.dumps({"collective": "allreduce", "world": 8, "rows": rows}))
    return str(path)


def test_within_tolerance_passes(tmp_path, capsys):
    rc = check_perf.main([_result(tmp_path, 11.4, 670.0, extra=True), "--baseline", _baseline(tmp_path)])
    out = [json.loads(line) for line in capsys.readouterr().out.splitlines()]
    assert rc == 0
    assert [o["status"] for o in out] == ["ok", "ok", "missing"]
    assert out[0]["metric"] == "time_us" and out[1]["metric"] == "busbw_gbs"


def test_latency_and_bandwidth_regressions(tmp_path, capsys):
    assert check_perf.main([_result(tmp_path, 11.6, 700.0), "--baseline", _baseline(tmp_path)]) == 1
    assert check_perf.main([_result(tmp_path, 10.0, 660.0), "--baseline", _baseline(tmp_path)]) == 1
    assert check_perf.main([_result(tmp_path, 11.6, 660.0), "--baseline", _baseline(tmp_path), "--latency-tol", "0.2",
                            "--bandwidth-tol", "0.1"]) == 0
    capsys.readouterr()


def test_nothing_to_compare(tmp_path, capsys):
    res = tmp_path / "r.json"
    res.write_text(json.dumps({"collective": "allgather", "world": 2, "rows": [{"bytes": 64, "best_us": 1.0, "busbw_gbs": 1.0}]}))
    assert check_perf.main([str(res), "--baseline", _baseline(tmp_path)]) == 2
    assert check_perf.main([str(res)]) == 2  # no shipped baseline for that configuration
    capsys.readouterr()


def test_shipped_baseline_is_well_formed():
    table = check_perf.load_baseline(check_perf.default_baseline("allreduce", 8))
    assert len(table) >= 8
    sizes = sorted(k[2] for k in table)
    assert sizes[0] == 1024 and sizes[-1] >= (256 << 20)
    assert all(v["time_us"] > 0 and v["busbw_gbs"] > 0 for v in table.values())
    rows = [{"collective": "allreduce", "world": 8, "bytes": b, "time_us": v["time_us"], "busbw_gbs": v["busbw_gbs"]}
            for (_, _, b), v in table.items()]
    report, compared = check_perf.compare(rows, table)
    assert compared == len(rows) and all(r["status"] == "ok" for r in report)


def test_shipped_baselines_cover_2_4_8_gpus_and_the_gate_picks_by_dtype(tmp_path, capsys):
    import os

    for world in (2, 4, 8):
        table = check_perf.load_baseline(check_perf.default_baseline("allreduce", world))
        sizes = sorted(k[2] for k in table)
        assert len(sizes) == 21 and sizes[0] == 1024 and sizes[-1] == 1 << 30  # powers of two, 1 KB - 1 GB
    assert os.path.exists(check_perf.default_baseline("allreduce", 2, "fp16"))
    # a float16 result of two ranks is compared with the fp16 file; an element type without a file falls back to bf16
    base = check_perf.load_baseline(check_perf.default_baseline("allreduce", 2, "fp16"))
    rows = [{"bytes": b, "best_us": v["time_us"], "busbw_gbs": v["busbw_gbs"], "algorithms": {}} for (_, _, b), v in base.items()]
    for dtype in ("float16", "float32"):
        res = tmp_path / f"{dtype}.json"
        res.write_text(json.dumps({"collective": "allreduce", "world": 2, "dtype": dtype, "rows": rows}))
        rc = check_perf.main([str(res), "--latency-tol", "0.5", "--bandwidth-tol", "0.5"])
        assert rc == 0
    capsys.readouterr()
