"""`pip wheel .` works offline and the wheel carries the libraries, the headers, the kernel sources (user kernels and
native algorithms are compiled against them at run time) and the perf-gate baselines."""
import glob
import os
import shutil
import subprocess
import sys
import zipfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_wheel_builds_and_is_complete(tmp_path):
    leftovers = [os.path.join(ROOT, d) for d in ("build", "mscclpp_b200.egg-info") if not os.path.exists(os.path.join(ROOT, d))]
    try:
        r = subprocess.run([sys.executable, "-m", "pip", "wheel", "--no-deps", "--no-build-isolation", "--no-index", "-w", str(tmp_path), ROOT],
                           capture_output=True, text=True, timeout=1800)
    finally:
        for d in leftovers:  # setuptools builds inside the source tree; leave it as it was
            shutil.rmtree(d, ignore_errors=True)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    wheels = glob.glob(str(tmp_path / "mscclpp_b200-*.whl"))
    assert len(wheels) == 1
    assert "none-any" not in os.path.basename(wheels[0])  # compiled code inside: a platform wheel
    names = set(zipfile.ZipFile(wheels[0]).namelist())
    for needed in ("mscclpp_b200/lib/libmscclpp_b200.so", "mscclpp_b200/lib/libmscclpp_b200_nccl.so",
                   "mscclpp_b200/csrc/include/mscclpp/core.hpp", "mscclpp_b200/csrc/include/mscclpp/ext/nccl/nccl.h",
                   "mscclpp_b200/csrc/kernels/gemm_sm100.cuh", "mscclpp_b200/benchmark/baselines/b200_8gpu_allreduce_bf16.jsonl",
                   "mscclpp_b200/language/program.py", "mscclpp_b200/default_algos/multi_node.py"):
        assert needed in names, needed
    assert any(n.startswith("mscclpp_b200/lib/_native") and n.endswith(".so") for n in names)
