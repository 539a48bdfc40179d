"""CPU-only tests of the native runtime: bootstrap (threads play the ranks), Communicator over the
Ethernet transport with host memory, host semaphores, FIFO protocol, plan parsing, error mapping.
No GPU is needed: failures are made on the host (a rank that never joins, an unknown id)."""
import json
import socket
import threading
import time

import pytest


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run_ranks(n, fn):
    """Run fn(rank) on n threads; re-raise the first exception."""
    errors, results = [], [None] * n

    def work(r):
        try:
            results[r] = fn(r)
        except Exception as e:  # noqa: BLE001
            errors.append((r, e))

    threads = [threading.Thread(target=work, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    if errors:
        raise errors[0][1]
    return results


def _bootstraps(native, n):
    port = _free_port()
    boots = [native.TcpBootstrap(r, n) for r in range(n)]
    _run_ranks(n, lambda r: boots[r].initialize(f"127.0.0.1:{port}", 20))
    return boots


@pytest.mark.parametrize("n", [1, 2, 5])
def test_bootstrap_ip_port_allgather_barrier(native, n):
    boots = _bootstraps(native, n)

    def body(r):
        b = boots[r]
        assert b.get_rank() == r and b.get_n_ranks() == n and b.get_n_ranks_per_node() == n
        got = b.all_gather(bytes([r]) * 8)
        assert got == [bytes([i]) * 8 for i in range(n)]
        b.barrier()
        return True

    assert all(_run_ranks(n, body))


def test_bootstrap_unique_id_and_ordered_send_recv(native):
    n = 3
    boots = [native.TcpBootstrap(r, n) for r in range(n)]
    uid = boots[0].get_unique_id()
    assert len(uid) == 128
    _run_ranks(n, lambda r: boots[r].initialize(uid, 20))

    def body(r):
        b = boots[r]
        nxt, prv = (r + 1) % n, (r - 1) % n
        for i in range(5):
            b.send(f"msg{i} from {r}".encode(), nxt, 7)
        b.send(b"other tag", nxt, 8)
        got = [b.recv(prv, 7) for _ in range(5)]
        assert got == [f"msg{i} from {prv}".encode() for i in range(5)]  # per (peer, tag) order
        assert b.recv(prv, 8) == b"other tag"
        assert b.broadcast(b"root-data" if r == 1 else b"xxxxxxxxx", 1) == b"root-data"
        b.group_barrier([0, 2]) if r in (0, 2) else None
        return True

    assert all(_run_ranks(n, body))


def test_bootstrap_times_out_when_a_rank_never_joins(native):
    port = _free_port()
    b0 = native.TcpBootstrap(0, 2)
    t0 = time.time()
    with pytest.raises(native.Error) as ei:
        b0.initialize(f"127.0.0.1:{port}", 1)  # rank 1 never shows up
    assert ei.value.error_code == native.ErrorCode.Timeout
    assert time.time() - t0 < 10


def test_bootstrap_connect_timeout_without_root(native):
    port = _free_port()
    b1 = native.TcpBootstrap(1, 2)
    with pytest.raises(native.Error) as ei:
        b1.initialize(f"127.0.0.1:{port}", 1)  # nobody listens there
    assert ei.value.error_code == native.ErrorCode.Timeout


def test_bootstrap_reinitialise_many_times(native):
    for _ in range(5):
        boots = _bootstraps(native, 2)
        _run_ranks(2, lambda r: boots[r].barrier())


def test_communicator_ethernet_host_memory_and_host_semaphores(native):
    import ctypes

    n = 2
    boots = _bootstraps(native, n)
    size = 4096
    bufs = [(ctypes.c_ubyte * size)() for _ in range(n)]
    results = {}

    def body(r):
        comm = native.Communicator(boots[r])
        peer = 1 - r
        cfg = native.EndpointConfig(native.Transport.Ethernet, native.Device(native.DeviceType.CPU), -1)
        conn = comm.connect(cfg, peer, 0).get()
        assert conn.transport() == native.Transport.Ethernet
        assert comm.remote_rank_of(conn) == peer and comm.tag_of(conn) == 0
        for i in range(size):
            bufs[r][i] = (r * 100 + i) % 251
        local = comm.register_memory(ctypes.addressof(bufs[r]), size, native.TransportFlags(native.Transport.Ethernet))
        comm.send_memory(local, peer, 1)
        remote = comm.recv_memory(peer, 1).get()
        sem = native.Host2HostSemaphore(comm, conn)
        if r == 0:
            conn.write(remote, 1024, local, 0, 512)  # my first 512 bytes -> peer[1024:1536]
            conn.flush()
            sem.signal()
            sem.wait()
        else:
            sem.wait()
            results["peer_view"] = bytes(bufs[1][1024:1536])
            sem.signal()
        with pytest.raises(native.Error):
            conn.write(remote, size - 10, local, 0, 512)  # out of range
        boots[r].barrier()
        return True

    assert all(_run_ranks(n, body))
    assert results["peer_view"] == bytes((0 * 100 + i) % 251 for i in range(512))


def test_host_semaphore_wait_runs_out(native):
    boots = _bootstraps(native, 2)

    def body(r):
        comm = native.Communicator(boots[r])
        cfg = native.EndpointConfig(native.Transport.Ethernet, native.Device(native.DeviceType.CPU), -1)
        conn = comm.connect(cfg, 1 - r, 0).get()
        sem = native.Host2HostSemaphore(comm, conn)
        if r == 0:
            with pytest.raises(native.Error) as ei:
                sem.wait(1000)  # nobody signals
            assert ei.value.error_code == native.ErrorCode.Timeout
        boots[r].barrier()
        return True

    assert all(_run_ranks(2, body))


def test_ib_transport_is_refused_cleanly_without_a_device(native):
    """No verbs library or no HCA: the endpoint is refused with an error that says so (the transport itself is covered
    against a software provider in test_cpp_unit.py)."""
    ctx = native.Context.create()
    try:
        ctx.create_endpoint(native.EndpointConfig(native.Transport.IB0))
    except native.Error as e:
        assert e.error_code in (native.ErrorCode.InvalidUsage, native.ErrorCode.SystemError)
        assert "InfiniBand" in str(e)
    else:
        pytest.skip("this machine has an InfiniBand device")


def test_fifo_protocol_with_lap_wrap(native):
    with pytest.raises(native.Error):
        native.Fifo(100)  # not a power of two
    fifo = native.Fifo(8)
    assert fifo.size() == 8
    empty = fifo.poll()
    assert empty.fst == 0 and empty.snd == 0
    seen = []
    for lap in range(5):  # 5 laps over 8 slots: parity flips every lap
        for i in range(8):
            t = native.ProxyTrigger()
            t.fst, t.snd = lap * 8 + i + 1, 7
            fifo.push_from_host(t)
        for i in range(8):
            got = fifo.poll()
            assert (got.fst, got.snd) == (lap * 8 + i + 1, 7)
            fifo.pop()
            seen.append(got.fst)
        again = fifo.poll()
        assert again.fst == 0 and again.snd == 0  # consumed entries do not reappear
    assert seen == list(range(1, 41)) and fifo.consumed() == 40


def test_execution_plan_parsing_and_errors(native, tmp_path):
    from mscclpp_b200.default_algos import single_node

    text = single_node.build("allreduce_allpairs_packet", 4, instances=2).to_json()
    path = tmp_path / "plan.json"
    path.write_text(text)
    plan = native.ExecutionPlan(str(path), 3)
    assert plan.name == "allreduce_allpairs_packet" and plan.collective == "allreduce" and plan.protocol == "LL"
    assert plan.n_ranks == 4 and plan.is_in_place
    with pytest.raises(native.Error) as ei:
        native.ExecutionPlan.from_string(text, 9)  # no such rank
    assert ei.value.error_code == native.ErrorCode.ExecutorError
    with pytest.raises(native.Error):
        native.ExecutionPlan.from_string(text[: len(text) // 2], 0)  # truncated JSON
    bad = json.loads(text)
    bad["protocol"] = "LL128"
    with pytest.raises(native.Error):
        native.ExecutionPlan.from_string(json.dumps(bad), 0)


def test_env_and_version(native):
    env = native.env()
    assert env.log_level in ("ERROR", "DEBUG", "INFO", "WARN", "NONE")
    assert env.device_timeout_ms > 0 and env.heap_bytes > 0
    assert native.version().startswith("0.9.0")
    assert native.is_nvls_supported() in (True, False)
