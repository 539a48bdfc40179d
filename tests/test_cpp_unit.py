"""Builds and runs the C++ unit tests of the host core (tests/cpp) with the in-tree test framework."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "mscclpp_b200")


def _build(tmp_path, name):
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(PKG, "csrc", "include"), "-I", os.path.join(PKG, "csrc"),
           "-I", "/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", name + ".cc"), "-o", exe,
           "-L", os.path.join(PKG, "lib"), "-lmscclpp_b200", f"-Wl,-rpath,{os.path.join(PKG, 'lib')}"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def test_cpp_core_unit_tests(tmp_path):
    exe = _build(tmp_path, "core_tests")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert "0 failures" in r.stdout and "PERF bootstrap_4_ranks" in r.stdout


def test_cpp_host_unit_tests(tmp_path):
    """Sockets, descriptor passing, JSON reader, algorithm registry, environment, and the plan loader on a DSL plan."""
    from mscclpp_b200.default_algos import single_node

    plan = tmp_path / "allreduce_8.json"
    plan.write_text(single_node.build("allreduce_allpairs", 8).to_json())
    exe = _build(tmp_path, "host_tests")
    env = dict(os.environ, MSCCLPP_TEST_PLAN=str(plan))
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert "0 failures" in r.stdout and "SKIPPED" not in r.stdout and "PERF socket_loopback_1MB" in r.stdout


def test_device_side_public_headers_compile(tmp_path):
    """assert_device / atomic_device / device / gpu / version headers in one sm_100a translation unit (compile only)."""
    nvcc = "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        import pytest

        pytest.skip("needs nvcc")
    for flags in ([], ["-DDEBUG_BUILD"]):
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", os.path.join(PKG, "csrc", "include"), "-c",
               os.path.join(ROOT, "tests", "kernels", "public_headers.cu"), "-o", str(tmp_path / "public_headers.o")] + flags
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-3000:]
