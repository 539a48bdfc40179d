"""The CMake project configures on a machine without a GPU and declares the expected targets (the full CMake build is
the same sources as the in-tree build and is not repeated here)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("cmake") is None or not os.path.exists("/usr/local/cuda/bin/nvcc"), reason="needs cmake and nvcc")
def test_cmake_configures_and_declares_targets(tmp_path):
    build = tmp_path / "b"
    r = subprocess.run(["cmake", "-S", ROOT, "-B", str(build), "-DMSCCLPP_B200_BUILD_TESTS=ON", "-DMSCCLPP_B200_BUILD_PYTHON=ON",
                        "-DMSCCLPP_B200_BUILD_EXAMPLES=ON"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "arch 100a" in r.stdout
    r = subprocess.run(["cmake", "--build", str(build), "--target", "help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    for target in ("mscclpp_b200", "mscclpp_b200_nccl", "mscclpp_b200_audit_nccl", "_native", "core_tests", "host_tests", "ib_tests", "fake_ibverbs",
                   "tutorial_01_basic_concepts", "customized_allgather", "peer_access_test"):
        assert target in r.stdout, target
    # the optional-dependency modules answer without the libraries being present
    for module in ("FindIBVerbs.cmake", "FindGDRCopy.cmake", "FindNUMA.cmake", "CheckBlackwellGpu.cmake"):
        assert os.path.exists(os.path.join(ROOT, "cmake", module))
