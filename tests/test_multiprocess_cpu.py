"""Host-side multi-process paths with real processes: CPU ranks under torch.distributed.run with the gloo backend."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_ranks_bootstrap_ethernet_and_failure_detection(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29760 + world), os.path.join(HERE, "mp_cpu_worker.py")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert '"ok": false' not in r.stdout
    for check in ("bootstrap/all_gather", "ethernet/all_pairs_write_and_signal", "failure/semaphore_wait_gives_up",
                  "failure/bootstrap_times_out", "failure/survivors_regroup"):
        assert f'"check": "{check}", "ok": true' in r.stdout, (check, r.stdout[-2000:])
