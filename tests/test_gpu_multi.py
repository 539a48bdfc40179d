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
