"""Real multi-GPU checks (one process per GPU). Skipped unless at least two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("nvls", ["0", "1"])
def test_collectives_on_real_peers(nvls):
    n = min(_ngpus(), 8)
    env = dict(os.environ, MSCCLPP_TEST_NVLS=nvls)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29733", os.path.join(HERE, "mp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert '"ok": false' not in r.stdout


def _real_nccl():
    p = os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "nccl", "lib", "libnccl.so.2")
    return os.path.abspath(p) if os.path.exists(p) else ""


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("fallback", [True, False])
def test_nccl_shim_under_torch(fallback):
    """torch.distributed's NCCL backend runs on this library when the shim is preloaded."""
    from mscclpp_b200._core import native

    shim = os.path.join(os.path.dirname(native.__file__), "..", "lib", "libmscclpp_b200_nccl.so")
    shim = os.path.abspath(shim)
    assert os.path.exists(shim), "build the NCCL shim first"
    n = min(_ngpus(), 8)
    env = dict(os.environ, LD_PRELOAD=shim, MSCCLPP_HEAP_BYTES=str(1 << 30))
    env.pop("MSCCLPP_NCCL_LIB_PATH", None)
    if fallback:
        if not _real_nccl():
            pytest.skip("no NCCL library to fall back to")
        env["MSCCLPP_NCCL_LIB_PATH"] = _real_nccl()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(HERE, "nccl_shim_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert '"ok": true' in r.stdout and '"shim_loaded": true' in r.stdout


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least two GPUs")
def test_algorithm_collection_on_real_peers(tmp_path):
    n = min(_ngpus(), 8)
    env = dict(os.environ, MSCCLPP_CACHE_DIR=str(tmp_path))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29747", os.path.join(HERE, "algo_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-4000:], r.stderr[-3000:])
    assert '"ok": false' not in r.stdout


@pytest.mark.skipif(_ngpus() < 2, reason="needs at least two GPUs")
def test_fused_layer_flag_protocol_stress():
    """1000 back-to-back launches per mode / transport / fence flavour with per-row checksums against fp32."""
    n = min(_ngpus(), 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29751", os.path.join(HERE, "mp_stress_worker.py")]
    r = subprocess.run(cmd, env=dict(os.environ), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-4000:], r.stderr[-3000:])
    assert '"ok": false' not in r.stdout and "tp_fused_stress" in r.stdout
