"""The execution-plan files that the reference ships as inputs of its own executor tests (test/execution-files/*.json:
all-pairs allreduce with memory channels, LL-packet allreduce, pipelined switch-channel allreduce) must load and run here
unchanged: on the numpy interpreter (CPU) and on the GPU plan interpreter with all ranks emulated in one cooperative launch.
The files are looked for in the reference checkout and in the offline build of the reference; skipped when absent."""
import glob
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CANDIDATES = [os.environ.get("MSCCLPP_REFERENCE_PLANS", ""),
              os.path.join(os.path.expanduser("~"), "reference", "test", "execution-files"),
              os.path.join(HERE, "..", "baseline", "_ref", "share", "execution-files")]
PLAN_DIR = next((d for d in CANDIDATES if d and glob.glob(os.path.join(d, "*.json"))), None)
FILES = ["allreduce.json", "allreduce_packet.json", "allreduce_pipeline.json"]

needs_files = pytest.mark.skipif(PLAN_DIR is None, reason="the reference's execution-plan files are not on this machine")


def _load(name):
    text = open(os.path.join(PLAN_DIR, name)).read()
    plan = json.loads(text)
    return text, plan, len(plan["gpus"])


def _elems(plan, world):
    # a whole number of chunks per rank; the pipelined plan moves 512 KiB units, so give it several iterations
    chunks = plan["gpus"][0]["input_chunks"]
    return chunks * (1 << 20) if "pipeline" in json.dumps(plan["gpus"][0]["threadblocks"][0]["ops"][0]["name"]) else chunks * world * 512


@needs_files
@pytest.mark.parametrize("name", FILES)
def test_reference_plan_file_on_numpy_interpreter(name):
    from mscclpp_b200.language.interpreter import PlanInterpreter, validate_plan

    text, plan, world = _load(name)
    validate_plan(text)
    n = _elems(plan, world)
    ins = [np.random.default_rng(r).uniform(-1, 1, n).astype(np.float16) for r in range(world)]
    outs = PlanInterpreter(text).run([a.copy() for a in ins], None)
    want = np.sum([a.astype(np.float32) for a in ins], axis=0)
    for r in range(world):
        np.testing.assert_allclose(outs[r].astype(np.float32), want, rtol=2e-2, atol=2e-2)


@needs_files
@pytest.mark.parametrize("name", FILES)
def test_reference_plan_file_parses_natively(name):
    from mscclpp_b200 import native

    text, plan, world = _load(name)
    for r in range(world):
        p = native().ExecutionPlan.from_string(text, r)
        assert p.name == plan["name"] and p.collective == "allreduce"


@pytest.mark.gpu
@needs_files
@pytest.mark.parametrize("name", FILES)
def test_reference_plan_file_on_gpu_interpreter(name):
    from test_gpu_executor import _run_both

    text, plan, world = _load(name)
    n = _elems(plan, world)
    _run_both(text, world, n, n, np.float16, inplace=True, launches=2)
