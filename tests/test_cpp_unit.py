"""Builds and runs the C++ unit tests of the host core (tests/cpp) with the in-tree test framework."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_core_unit_tests(tmp_path):
    pkg = os.path.join(ROOT, "mscclpp_b200")
    exe = str(tmp_path / "core_tests")
    cmd = ["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(pkg, "csrc", "include"), "-I", "/usr/local/cuda/include",
           os.path.join(ROOT, "tests", "cpp", "core_tests.cc"), "-o", exe, "-L", os.path.join(pkg, "lib"), "-lmscclpp_b200",
           f"-Wl,-rpath,{os.path.join(pkg, 'lib')}"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert "0 failures" in r.stdout and "PERF bootstrap_4_ranks" in r.stdout
