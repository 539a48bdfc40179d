"""The tutorials and examples build against the package (CPU: compile only) and run on two GPUs (gpu marker)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TUTORIALS = {
    "01-basic-concepts": "gpu_ping_pong",
    "02-bootstrap": "gpu_ping_pong_mp",
    "03-memory-channel": "bidir_memory_channel",
    "04-port-channel": "bidir_port_channel",
    "05-switch-channel": "switch_allreduce",
}


def _build(name):
    d = os.path.join(ROOT, "examples", "tutorials", name)
    r = subprocess.run(["make", "-s", "-C", d], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    exe = os.path.join(d, TUTORIALS[name])
    assert os.path.exists(exe)
    return exe


@pytest.mark.parametrize("name", sorted(TUTORIALS))
def test_tutorial_compiles(name):
    _build(name)


def test_customized_algorithm_compiles_and_loads(tmp_path, monkeypatch):
    monkeypatch.setenv("MSCCLPP_CACHE_DIR", str(tmp_path))
    import mscclpp_b200 as mp

    compiler = mp.NativeCodeCompiler()
    module = compiler.compile("customized_allgather", os.path.join(ROOT, "examples", "customized-collective-algorithm", "customized_allgather.cu"))
    assert callable(module.create_allgather)
    assert compiler.get_arch() == "sm_100a"


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.gpu
@pytest.mark.skipif(_ngpus() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("name", sorted(TUTORIALS))
def test_tutorial_runs(name):
    exe = _build(name)
    args = [exe] + (["2", "127.0.0.1:50549"] if name == "05-switch-channel" else [])
    r = subprocess.run(args, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    assert "WRONG" not in r.stdout and "ran out of time" not in r.stdout


@pytest.mark.gpu
@pytest.mark.skipif(_ngpus() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("script", ["customized_comm_with_default_algo.py", "customized_comm_with_dsl.py", "customized_allgather.py"])
def test_torch_integration_example(script, tmp_path):
    n = min(_ngpus(), 8)
    env = dict(os.environ, MSCCLPP_CACHE_DIR=str(tmp_path), PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29761", os.path.join(ROOT, "examples", "torch-integration", script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert "WRONG" not in r.stdout
