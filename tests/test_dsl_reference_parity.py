"""Plan-format parity: for every example program that ships with the reference DSL
(python/mscclpp/language/tests/**), the plan compiled by this package's DSL must equal the plan
compiled by the reference DSL. Needs the reference checkout; skipped when it is not there.
A digest of each plan is also kept in tests/golden/dsl_plan_digests.json so that the check still
bites (against the last verified output) on machines without the reference."""
import glob
import hashlib
import json
import os
import re
import subprocess
import sys

import pytest

REF_PY = os.environ.get("MSCCLPP_REFERENCE_PYTHON", os.path.join(os.path.expanduser("~"), "reference", "python"))
EXAMPLES = os.path.join(REF_PY, "mscclpp", "language", "tests")
RUNNER = os.path.join(os.path.dirname(__file__), "_dsl_runner.py")
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "dsl_plan_digests.json")

# scripts that do not run under the reference itself (they use names it no longer defines)
BROKEN_UPSTREAM = {"single_node/allgather_ring.py", "single_node/alltoall/alltoall_pkt.py",
                   "unit_tests/put/put_with_signal_fuse_test.py"}


def _args_for(path):
    src = open(path).read()
    out = []
    for name, typ, rest in re.findall(r'add_argument\("--(\w+)", type=(\w+)(.*)\)', src):
        if "default=" in rest:
            continue
        if name == "name":
            v = "prog"
        elif name == "num_gpus":
            v = "2" if "send_recv" in path else "8"
        elif name in ("gpus_per_node", "nranks_per_node"):
            v = "4"
        elif typ == "int":
            v = "2"
        else:
            v = "x"
        out += ["--" + name, v]
    return out


def _normalise(o):
    if isinstance(o, dict):
        return {k: (sorted(v) if k == "access_channel_types" else _normalise(v)) for k, v in o.items()}
    if isinstance(o, list):
        return [_normalise(x) for x in o]
    return o


def _run(mode, script):
    r = subprocess.run([sys.executable, RUNNER, mode, REF_PY, script] + _args_for(script), capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    return _normalise(json.loads(r.stdout))


def _scripts():
    if not os.path.isdir(EXAMPLES):
        return []
    rel = [os.path.relpath(p, EXAMPLES) for p in sorted(glob.glob(EXAMPLES + "/**/*.py", recursive=True))]
    return [r for r in rel if r not in BROKEN_UPSTREAM]


@pytest.fixture(scope="session")
def compiled_plans():
    """{rel: (ours, theirs)} for every example, compiled concurrently (each compile is its own process)."""
    from concurrent.futures import ThreadPoolExecutor

    rels = _scripts()
    jobs = [(mode, rel) for rel in rels for mode in ("ours", "reference")]
    with ThreadPoolExecutor(max(2, os.cpu_count() or 2)) as pool:
        results = list(pool.map(lambda j: _try_run(j[0], os.path.join(EXAMPLES, j[1])), jobs))
    out = {}
    for (mode, rel), res in zip(jobs, results):
        out.setdefault(rel, {})[mode] = res
    return out


def _try_run(mode, script):
    try:
        return _run(mode, script)
    except Exception as e:  # reported by the test that looks at this entry
        return e


@pytest.mark.skipif(not os.path.isdir(EXAMPLES), reason="reference checkout not present")
@pytest.mark.parametrize("rel", _scripts())
def test_plan_equals_reference_plan(rel, compiled_plans):
    ours, theirs = compiled_plans[rel]["ours"], compiled_plans[rel]["reference"]
    for side in (ours, theirs):
        if isinstance(side, Exception):
            raise side
    assert ours == theirs
    digest = hashlib.sha256(json.dumps(ours, sort_keys=True).encode()).hexdigest()
    golden = json.load(open(GOLDEN)) if os.path.exists(GOLDEN) else {}
    if os.environ.get("MSCCLPP_UPDATE_GOLDEN"):
        golden[rel] = digest
        json.dump(golden, open(GOLDEN, "w"), indent=1, sort_keys=True)
    assert golden.get(rel) == digest, "plan changed since the digests were recorded (set MSCCLPP_UPDATE_GOLDEN=1 to re-record)"


def test_default_algorithm_digests_are_stable():
    """Plans of this package's own DSL algorithms are deterministic."""
    from mscclpp_b200.default_algos import single_node

    for name in single_node.ALGORITHMS:
        a = single_node.build(name, 4, instances=2).to_json()
        b = single_node.build(name, 4, instances=2).to_json()
        assert a == b
