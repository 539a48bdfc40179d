"""CPU-only checks of the Python surface: algorithm registry and selectors, the DSL compiler cache, the
kernel builder, `pack`, the package exports and the host-only calls of the NCCL shim."""
import ctypes
import os
import struct

import numpy as np
import pytest

import mscclpp_b200 as mp
from mscclpp_b200._core import native
from mscclpp_b200.default_algos import allreduce_allpairs, make_spec
from mscclpp_b200.language.collectives import AllReduce

N = native.load()


def test_reference_names_are_exported():
    for name in ("Communicator", "TcpBootstrap", "Transport", "MemoryChannel", "PortChannel", "ProxyService", "Executor",
                 "ExecutionPlan", "DataType", "ReduceOp", "PacketType", "RawGpuBuffer", "env", "is_nvls_supported", "Algorithm",
                 "AlgorithmCollection", "CommGroup", "GpuBuffer", "compile", "compile_native", "get_include", "get_lib", "npkit"):
        assert hasattr(mp, name), name
    assert os.path.isdir(mp.get_include()) and os.path.exists(os.path.join(mp.get_include(), "mscclpp", "core.hpp"))
    assert os.path.isdir(mp.get_lib())


def test_python_native_algorithm_roundtrip():
    calls = []

    def kernel(inp, out, in_bytes, out_bytes, dtype, op, stream, n_blocks, n_threads, symmetric, extras):
        calls.append((inp, out, in_bytes, out_bytes, dtype, op, n_blocks, n_threads, symmetric, dict(extras)))
        return 0

    inits = []
    algo = mp.Algorithm.from_callable("my_allreduce", "allreduce", kernel, init=lambda comm: inits.append(comm),
                                      min_message_size=16, max_message_size=1 << 20, tags={"fast": 1})
    assert algo.name == "my_allreduce" and algo.collective == "allreduce"
    assert algo.message_size_range == (16, 1 << 20)
    assert algo.tags == {"fast": 1}
    assert algo.is_native_algorithm() and not algo.is_dsl_algorithm()
    rc = algo.execute(None, 0x1000, 0x2000, 64, 64, N.DataType.float16, N.ReduceOp.SUM, nblocks=3, nthreads_per_block=128,
                      symmetric_memory=True, extras={"k": 7})
    rc2 = algo.execute(None, 0x1000, 0x2000, 64, 64, N.DataType.float16, N.ReduceOp.SUM)
    assert rc == 0 and rc2 == 0
    assert len(inits) == 1, "init runs once"
    assert calls[0][:4] == (0x1000, 0x2000, 64, 64) and calls[0][6:] == (3, 128, True, {"k": 7})
    algo.set_message_size_range(0, 99)
    assert algo.message_size_range == (0, 99)
    # capsule round trip (the exchange format with separately compiled modules)
    again = mp.Algorithm.create_from_native_capsule(algo._algorithm.to_native_capsule())
    assert again.name == "my_allreduce"


def test_collection_and_selectors():
    from mscclpp_b200.ext import AlgorithmCollectionBuilder

    AlgorithmCollectionBuilder.reset()
    builder = AlgorithmCollectionBuilder()
    small = mp.Algorithm.from_callable("small", "allreduce", lambda *a: 0, max_message_size=1024)
    large = mp.Algorithm.from_callable("large", "allreduce", lambda *a: 0, min_message_size=1025)
    builder.add_algorithm_builder(small)
    builder.add_algorithm_builder(large)
    seen = []

    def selector(algo_map, request):
        seen.append((request.collective, request.message_size))
        for algo in algo_map.get(request.collective, {}).values():
            lo, hi = algo.message_range
            if lo <= request.message_size <= hi:
                return algo
        return None

    builder.set_algorithm_selector(selector)
    coll = builder.build()
    assert len(coll) == 2 and {a.name for a in coll.get_by_collective("allreduce")} == {"small", "large"}
    req = N.CollectiveRequest()
    req.collective = "allreduce"
    req.message_size = 512
    assert coll.select(req).name == "small"
    req.message_size = 4096
    assert coll.select(req).name == "large"
    req.collective = "allgather"
    assert coll.select(req) is None  # the default fallback selector finds nothing either
    assert seen[0] == ("allreduce", 512)
    coll.register_algorithm("allgather", "ag", mp.Algorithm.from_callable("ag", "allgather", lambda *a: 0))
    assert len(coll) == 3
    AlgorithmCollectionBuilder.reset()


def test_dsl_compile_caches_plan(tmp_path, monkeypatch):
    monkeypatch.setenv("MSCCLPP_CACHE_DIR", str(tmp_path))
    spec = make_spec("cached_allreduce", AllReduce(4, 1, True), 4, tags={"t": 1})
    compiler = mp.DslCompiler()
    # the native Env singleton may have latched another cache dir: go through plan_path, which reports where it wrote
    path = compiler.plan_path(allreduce_allpairs, spec)
    assert path.exists()
    mtime = path.stat().st_mtime_ns
    assert compiler.plan_path(allreduce_allpairs, spec) == path and path.stat().st_mtime_ns == mtime, "second call hits the cache"
    other = compiler.plan_path(allreduce_allpairs, make_spec("cached_allreduce", AllReduce(4, 1, True), 4, instances=2))
    assert other != path
    algo = mp.compile(allreduce_allpairs, spec, rank=1)
    assert algo.is_dsl_algorithm() and algo.collective == "allreduce" and algo.name == "cached_allreduce"
    assert algo.tags == {"t": 1}


def test_pack_layout():
    from mscclpp_b200.utils import pack

    a = np.zeros(4, dtype=np.float32)
    blob = pack(a, 7, ctypes.c_size_t(1 << 40), True, 2.5, b"\x01\x02")
    assert blob == struct.pack("P", a.ctypes.data) + struct.pack("i", 7) + struct.pack("N", 1 << 40) + struct.pack("i", 1) + \
        struct.pack("f", 2.5) + b"\x01\x02"
    with pytest.raises(RuntimeError):
        pack(object())


def test_kernel_builder_compiles_against_the_headers(tmp_path):
    from mscclpp_b200.utils import KernelBuilder

    src = tmp_path / "k.cu"
    src.write_text(
        '#include <mscclpp/packet_device.hpp>\n#include <mscclpp/concurrency_device.hpp>\n'
        'extern "C" __global__ void scale(float* x, int n) {\n'
        '  int i = blockIdx.x * blockDim.x + threadIdx.x;\n  if (i < n) x[i] *= SCALE;\n}\n')
    kb = KernelBuilder("k.cu", "scale", file_dir=str(tmp_path), macro_dict={"SCALE": "2.0f"}, load=False)
    assert kb.cubin[:4] == b"\x7fELF"
    with pytest.raises(RuntimeError):
        KernelBuilder("k.cu", "scale", file_dir=str(tmp_path), macro_dict={"SCALE": "not_defined_anywhere"}, load=False)


def test_nccl_shim_host_calls():
    path = os.path.join(mp.get_lib(), "libmscclpp_b200_nccl.so")
    lib = ctypes.CDLL(path)
    v = ctypes.c_int(0)
    assert lib.ncclGetVersion(ctypes.byref(v)) == 0 and v.value >= 22000
    lib.ncclGetErrorString.restype = ctypes.c_char_p
    assert lib.ncclGetErrorString(0) == b"no error"
    assert b"invalid argument" in lib.ncclGetErrorString(4)
    uid = (ctypes.c_char * 128)()
    assert lib.ncclGetUniqueId(uid) == 0 and any(uid.raw), "a unique id carries the rendezvous address"
    assert lib.ncclGetVersion(None) == 4  # ncclInvalidArgument
    count = ctypes.c_int()
    assert lib.ncclCommCount(None, ctypes.byref(count)) == 4
    for sym in ("ncclAllReduce", "ncclAllGather", "ncclReduceScatter", "ncclBroadcast", "ncclReduce", "ncclSend", "ncclRecv",
                "ncclGroupStart", "ncclGroupEnd", "ncclCommInitRank", "ncclCommInitRankConfig", "ncclCommSplit", "ncclCommDestroy",
                "ncclCommAbort", "ncclMemAlloc", "ncclMemFree", "ncclCommRegister", "ncclCommDeregister", "ncclAlltoAll",
                "ncclCommGetAsyncError", "ncclGetLastError", "ncclCommUserRank", "ncclCommCuDevice", "ncclRedOpCreatePreMulSum"):
        assert hasattr(lib, sym), sym


def test_npkit_trace_generator(tmp_path):
    """The converter pairs ENTRY/EXIT events of a synthetic dump and places GPU events on the host time line."""
    from mscclpp_b200.utils.npkit_trace import convert_npkit_dump_to_trace, parse_event_header

    names = parse_event_header()
    by_name = {v: k for k, v in names.items()}
    assert names[by_name["EXECUTOR_OP_PUT_ENTRY"] + 1] == "EXECUTOR_OP_PUT_WITH_SIGNAL_ENTRY"
    assert not set(range(by_name["EXECUTOR_OP_NOP_ENTRY"], by_name["EXECUTOR_OP_PIPELINE_END_ENTRY"] + 1)) & \
        set(range(by_name["EXECUTOR_OP_NOP_EXIT"], by_name["EXECUTOR_OP_PIPELINE_END_EXIT"] + 1)), "entry and exit ranges are disjoint"

    def ev(type_, size, ts):
        return struct.pack("<QQ", type_ | (size << 8), ts)

    d = tmp_path / "dump"
    d.mkdir()
    (d / "gpu_events_rank_0_buf_0").write_bytes(
        ev(by_name["EXECUTOR_OP_PUT_ENTRY"], 4096, 5_000) + ev(by_name["EXECUTOR_OP_PUT_EXIT"], 4096, 7_000))
    (d / "cpu_events_rank_0_channel_0").write_bytes(
        ev(by_name["CONN_ETH_WRITE_ENTRY"], 64, 1_000_000_500) + ev(by_name["CONN_ETH_WRITE_EXIT"], 64, 1_000_001_500))
    (d / "gpu_clock_rate_rank_0").write_text("1000000")
    (d / "cpu_clock_period_num_rank_0").write_text("1")
    (d / "cpu_clock_period_den_rank_0").write_text("1000000000")
    (d / "gpu_time_sync_rank_0").write_text("4000 1000000000")
    import json

    out = json.loads(open(convert_npkit_dump_to_trace(str(d), str(tmp_path / "out"))).read())["traceEvents"]
    put = next(e for e in out if e["name"] == "EXECUTOR_OP_PUT")
    assert put["ph"] == "X" and abs(put["dur"] - 2.0) < 1e-6 and abs(put["ts"] - (1e6 + 1.0)) < 1e-3
    assert abs(put["args"]["bw (GB/s)"] - 4096 / 2.0 / 1e3) < 1e-9
    wr = next(e for e in out if e["name"] == "CONN_ETH_WRITE")
    assert abs(wr["dur"] - 1.0) < 1e-6 and wr["tid"] == "channel0"


def test_shipped_tuning_store_and_its_selector():
    """The store measured on 2, 4 and 8 B200s: every size has an entry, and the selector made from it hands out the
    recorded algorithm."""
    from types import SimpleNamespace

    from mscclpp_b200.benchmark.tuning_config import TuningConfig

    store = TuningConfig.shipped()
    for world in (2, 4, 8):
        profile = f"NVIDIA_B200-x{world}-nvls"
        rows = store.data[profile]["allreduce/bfloat16"]
        assert len(rows) == 21 and rows[0]["max_bytes"] == 1024 and rows[-1]["max_bytes"] == 1 << 30
        assert store.lookup(profile, "allreduce", "bfloat16", 1 << 30)["algorithm"].endswith("zero_copy")
        assert "packet" in store.lookup(profile, "allreduce", "bfloat16", 2048)["algorithm"]
    selector = store.make_selector("NVIDIA_B200-x8-nvls")
    request = SimpleNamespace(collective="allreduce", dtype=SimpleNamespace(name="bfloat16"), message_size=128 << 10)
    algo_map = {"allreduce": {"default_allreduce_packet_ll128": "LL128", "default_allreduce_nvls_zero_copy": "NVLS"}}
    assert selector(algo_map, request) == "LL128"
    request.message_size = 64 << 20
    assert selector(algo_map, request) == "NVLS"
    assert store.make_selector("some-other-gpu")(algo_map, request) is None


def test_tuning_config_store(tmp_path):
    from mscclpp_b200.benchmark.tuning_config import TuningConfig

    path = str(tmp_path / "tuned.json")
    store = TuningConfig()
    store.record("B200-x8-nvls", "allreduce", "bfloat16", 1 << 20, "default_allreduce_packet", 32, 512, 11.5)
    store.record("B200-x8-nvls", "allreduce", "bfloat16", 1 << 10, "default_allreduce_nvls_packet", 8, 256, 6.0)
    store.record("B200-x8-nvls", "allreduce", "bfloat16", 1 << 20, "default_allreduce_nvls_zero_copy", 16, 512, 10.0)  # replaces
    store.save(path)
    again = TuningConfig(path)
    assert again.lookup("B200-x8-nvls", "allreduce", "bfloat16", 512)["algorithm"] == "default_allreduce_nvls_packet"
    assert again.lookup("B200-x8-nvls", "allreduce", "bfloat16", 4096)["algorithm"] == "default_allreduce_nvls_zero_copy"
    assert again.lookup("B200-x8-nvls", "allreduce", "bfloat16", 1 << 30)["n_blocks"] == 16  # beyond the table: last row
    assert again.lookup("other", "allreduce", "bfloat16", 4096) is None
    # the store doubles as an algorithm selector
    sel = again.make_selector("B200-x8-nvls")
    req = N.CollectiveRequest()
    req.collective, req.message_size, req.dtype = "allreduce", 100, N.DataType.bfloat16
    algo = mp.Algorithm.from_callable("default_allreduce_nvls_packet", "allreduce", lambda *a: 0)
    assert sel({"allreduce": {"default_allreduce_nvls_packet": algo._algorithm}}, req).name == "default_allreduce_nvls_packet"


def test_audit_library_redirects_nccl_loads(tmp_path):
    """LD_AUDIT with the audit library answers a dlopen of libnccl.so.2 with the shim (host-only: the shim's
    version query needs no GPU)."""
    import subprocess
    import sys

    lib = mp.get_lib()
    audit = os.path.join(lib, "libmscclpp_b200_audit_nccl.so")
    shim = os.path.join(lib, "libmscclpp_b200_nccl.so")
    assert os.path.exists(audit)
    code = ("import ctypes\n"
            "l = ctypes.CDLL('libnccl.so.2')\n"
            "l.ncclGetErrorString.restype = ctypes.c_char_p\n"
            "print(any('libmscclpp_b200_nccl' in x for x in open('/proc/self/maps')), l.ncclGetErrorString(5))\n")
    env = dict(os.environ, LD_AUDIT=audit, MSCCLPP_B200_NCCL_SHIM=shim)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip().startswith("True") and "invalid usage" in r.stdout


def test_comm_group_over_ethernet_on_cpu():
    """CommGroup (bootstrap + communicator + helpers) with two CPU ranks as threads: connections over the Ethernet
    transport, memory registration and exchange, semaphores, a write that lands in the peer's numpy buffer."""
    import socket
    import threading

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = {}

    def rank_main(rank):
        try:
            group = mp.CommGroup(interfaceIpPortTrio=f"127.0.0.1:{port}", rank=rank, size=2)
            assert (group.my_rank, group.nranks) == (rank, 2)
            peer = 1 - rank
            cfg = N.EndpointConfig(N.Transport.Ethernet, N.Device(N.DeviceType.CPU))
            conns = group.make_connection([peer], cfg)
            buf = np.full(256, rank + 1, dtype=np.int64)
            mems = group.register_tensor_with_connections(buf, conns)
            assert set(mems) == {0, 1}
            sems = group.make_semaphores(conns)
            h2h = N.Host2HostSemaphore(sems[peer])
            if rank == 0:
                conns[peer].write(mems[peer], 0, mems[rank], 0, buf.nbytes)
                conns[peer].flush()
                h2h.signal()
            else:
                h2h.wait()
                results["received"] = buf.copy()
            group.barrier()
            # bootstrap point-to-point helpers
            msg = np.arange(4, dtype=np.int32) + rank
            if rank == 0:
                group.send(msg, 1, 5)
            else:
                got = np.zeros(4, dtype=np.int32)
                group.recv(got, 0, 5)
                results["msg"] = got
            group.barrier()
        except Exception as e:  # noqa: BLE001
            results[f"error{rank}"] = repr(e)

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not any(k.startswith("error") for k in results), results
    assert (results["received"] == 1).all()
    assert results["msg"].tolist() == [0, 1, 2, 3]


def test_numa_helpers_and_reference_export_names():
    """NUMA helpers work from sysfs without libnuma; every name the reference's package exports exists here."""
    import os

    import mscclpp_b200 as mp

    assert mp.numa.parse_cpu_list("0-3, 8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    for bad in ("3-1", "a", "1-"):
        with pytest.raises(Exception):
            mp.numa.parse_cpu_list(bad)
    with pytest.raises(Exception):
        mp.numa.get_numa_node_cpus(4096)
    mp.numa.numa_bind(-1)  # "unknown node": nothing happens
    if os.path.exists("/sys/devices/system/node/node0/cpulist"):
        cpus = set(mp.numa.get_numa_node_cpus(0))
        before = os.sched_getaffinity(0)
        try:
            if cpus & before:
                mp.numa.numa_bind(0)
                assert os.sched_getaffinity(0) == cpus & before
        finally:
            os.sched_setaffinity(0, before)
    assert {m.name for m in mp.GpuBufferGranularity.__members__.values()} == {"MultiCastMinimum", "MultiCastRecommended"}
    assert callable(mp.alloc_shared_physical_cuda)
    # the public names of the reference's Python package (its __all__)
    reference_names = [
        'Algorithm', 'AlgorithmCollection', 'CommGroup', 'Communicator', 'Connection', 'DataType', 'Device',
        'DeviceType', 'EndpointConfig', 'EndpointConfigIb', 'ErrorCode', 'ExecutionPlan', 'Executor', 'Fifo',
        'GpuBuffer', 'GpuBufferGranularity', 'Host2DeviceSemaphore', 'Host2HostSemaphore', 'IbMode',
        'MemoryChannel', 'MemoryDevice2DeviceSemaphore', 'PacketType', 'PortChannel', 'ProxyService',
        'RawGpuBuffer', 'ReduceOp', 'RegisteredMemory', 'Semaphore', 'TcpBootstrap', 'Transport', 'TransportFlags',
        '__version__', 'alloc_shared_physical_cuda', 'connect_nvls_collective', 'env', 'get_include', 'get_lib',
        'is_bulk_supported', 'is_nvls_supported', 'npkit', 'numa', 'version',
    ]
    assert not [n for n in reference_names if not hasattr(mp, n)]


def test_compat_names_of_the_reference_layout():
    import warnings

    import mscclpp_b200 as mp
    from mscclpp_b200._core import buffer
    from mscclpp_b200.default_algos import multi_node
    from mscclpp_b200.default_algos.allgather_multi_nodes import allgather_multi_nodes
    from mscclpp_b200.default_algos.allreduce_multi_nodes import allreduce_multi_nodes
    from mscclpp_b200.default_algos.reducescatter_multi_nodes import reducescatter_multi_nodes

    assert allgather_multi_nodes is multi_node.allgather_multi_nodes
    assert allreduce_multi_nodes is multi_node.allreduce_multi_nodes
    assert reducescatter_multi_nodes is multi_node.reducescatter_multi_nodes
    assert buffer.GpuBufferGranularity is mp.GpuBufferGranularity

    class New:
        def __init__(self, x):
            self.x = x

    @mp.deprecated(New)
    class Old:
        pass

    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        obj = Old(3)
    assert isinstance(obj, New) and obj.x == 3
    assert any(issubclass(w.category, DeprecationWarning) and "Old is deprecated, use New" in str(w.message) for w in caught)


def test_nccl_shim_plan_handles_and_alltoall_names(tmp_path):
    """mscclLoadAlgo / mscclUnloadAlgo keep plans by handle; the entry points of the MSCCL++ header all exist."""
    import mscclpp_b200 as mp
    from mscclpp_b200.default_algos import single_node

    lib = ctypes.CDLL(os.path.join(mp.get_lib(), "libmscclpp_b200_nccl.so"))
    for name in ("ncclAllToAll", "ncclAlltoAll", "ncclAllToAllv", "mscclLoadAlgo", "mscclRunAlgo", "mscclUnloadAlgo"):
        assert hasattr(lib, name), name
    plan = tmp_path / "ar.json"
    plan.write_text(single_node.build("allreduce_allpairs", 4).to_json())
    h1, h2 = ctypes.c_int(0), ctypes.c_int(0)
    assert lib.mscclLoadAlgo(str(plan).encode(), ctypes.byref(h1), 0) == 0
    assert lib.mscclLoadAlgo(str(plan).encode(), ctypes.byref(h2), 3) == 0
    assert h1.value > 0 and h2.value != h1.value
    assert lib.mscclLoadAlgo(str(plan).encode(), ctypes.byref(h2), 4) != 0          # rank outside the plan
    assert lib.mscclLoadAlgo(b"/nonexistent/plan.json", ctypes.byref(h2), 0) != 0
    assert lib.mscclLoadAlgo(None, ctypes.byref(h2), 0) != 0
    assert lib.mscclUnloadAlgo(h1.value) == 0
    assert lib.mscclUnloadAlgo(h1.value) != 0                                         # already gone
    # running needs a communicator: a null one is refused, as is an unknown handle
    lib.mscclRunAlgo.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                        ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    assert lib.mscclRunAlgo(None, None, None, None, None, None, 16, 7, 0, 0, 0, 12345, None, None) != 0
    lib.ncclAllToAllv.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    assert lib.ncclAllToAllv(None, None, None, None, None, None, 7, None, None) != 0


def test_binding_synonyms_of_the_reference(native):
    import mscclpp_b200 as mp

    assert native.get_host_name(64, ".") and "." not in native.get_host_name(64, ".")
    assert mp.DataType.float8_e4m3fn == mp.DataType.float8_e4m3
    flags = mp.TransportFlags(mp.Transport.CudaIpc)
    flags |= mp.TransportFlags(mp.Transport.Ethernet)
    assert flags.count() == 2 and not flags.all()
    flags &= mp.TransportFlags(mp.Transport.Ethernet)
    assert flags.count() == 1 and flags.has(mp.Transport.Ethernet)
    for name in ("connect_on_setup", "send_memory_on_setup", "recv_memory_on_setup", "setup"):
        assert hasattr(mp.Communicator, name)
    for cls, name in ((mp.Connection, "context"), (mp.Semaphore, "connection"), (mp.Host2HostSemaphore, "connection"),
                      (mp.Host2DeviceSemaphore, "connection"), (mp.MemoryDevice2DeviceSemaphore, "connection"),
                      (native.RawGpuBuffer, "nelems"), (native.Endpoint, "config")):
        assert hasattr(cls, name), (cls, name)


def test_raw_buffer_dlpack_helper_parses_types(native):
    import torch

    from mscclpp_b200._core.native import parse_torch_dtype

    assert parse_torch_dtype("torch.float16") is torch.float16
    assert parse_torch_dtype("bfloat16") is torch.bfloat16
    assert parse_torch_dtype(torch.int32) is torch.int32
    with pytest.raises(ValueError):
        parse_torch_dtype("torch.nope")
    assert callable(native.RawGpuBuffer.to_dlpack)
