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


def _shared(tmp_path, src, out, flags=()):
    lib = str(tmp_path / out)
    cmd = ["g++", "-shared", "-fPIC", "-O1", "-I", os.path.join(PKG, "csrc"), os.path.join(ROOT, "tests", "cpp", src), "-o", lib, *flags]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    return lib


def test_cpp_infiniband_transport_against_software_provider(tmp_path):
    """IbvApi / IbCtx / IbQp / IbMr, IBConnection in both token modes, Host2HostSemaphore over it, error and time-limit
    paths, and the GDRCopy wrapper - against stand-ins for libibverbs and libgdrapi, loaded the way the real ones are.
    Run twice: with a provider that exports the fast-path calls and with one that, like libibverbs, offers them only
    through the device context's table."""
    exe = _build(tmp_path, "ib_tests")
    gdr = _shared(tmp_path, "fake_gdrapi.cc", "libfake_gdrapi.so")
    for out, flags in (("libfake_ibverbs.so", ()), ("libfake_ibverbs_ops.so", ("-DFAKE_IBV_NO_FASTPATH_SYMBOLS",))):
        ibv = _shared(tmp_path, "fake_ibverbs.cc", out, ("-DMSCCLPP_IB_OWN_ABI",) + flags)
        env = dict(os.environ, MSCCLPP_IBV_SO=ibv, MSCCLPP_GDRCOPY_SO=gdr)
        r = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
        assert "13 tests, 0 failures" in r.stdout


def test_infiniband_is_reported_absent_without_a_verbs_library(tmp_path):
    """Without a loadable verbs library the IB transports fail with an error that says so (and nothing else breaks)."""
    import sys

    code = (
        "import mscclpp_b200 as mp\n"
        "n = mp.native()\n"
        "ctx = n.Context.create() if hasattr(n.Context, 'create') else n.Context()\n"
        "try:\n"
        "    ctx.create_endpoint(n.EndpointConfig(n.Transport.IB0))\n"
        "    print('NO ERROR')\n"
        "except Exception as e:\n"
        "    print('ERR', e)\n"
    )
    env = dict(os.environ, MSCCLPP_IBV_SO=str(tmp_path / "no_such_library.so"), PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "ERR" in r.stdout and "InfiniBand" in r.stdout, r.stdout  # no device listed, or the library's load error


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
