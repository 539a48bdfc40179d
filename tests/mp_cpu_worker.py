"""CPU ranks as separate processes (launched by torch.distributed.run with the gloo backend from test_multiprocess_cpu.py):
bootstrap from a torch process group, ring collectives of the bootstrap, all-pairs Ethernet connections with memory
exchange and host semaphores, the IPC-domain query, and failure detection on the host - a rank that leaves between two
steps is noticed by the others through bounded waits (a bootstrap that times out, a semaphore wait that gives up), never
through a hang. Prints one JSON line per check on rank 0; exit code 0 = all good."""
import json
import os
import sys
import time

import numpy as np
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import mscclpp_b200 as mp  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    N = mp.native()
    failures = []

    def report(name, ok, **extra):
        if not ok:
            failures.append(name)
        if rank == 0:
            print(json.dumps({"check": name, "ok": bool(ok), **extra}), flush=True)

    group = mp.CommGroup(torch_group=dist.group.WORLD)
    report("bootstrap/identity", (group.my_rank, group.nranks) == (rank, world))
    report("bootstrap/one_host", group.nranks_per_node == world and group.nranks_per_ipc_domain == world,
           per_node=group.nranks_per_node, per_domain=group.nranks_per_ipc_domain)
    got = group.bootstrap.all_gather(bytes([rank]) * 4)
    report("bootstrap/all_gather", got == [bytes([r]) * 4 for r in range(world)])
    group.barrier()

    # all pairs over the Ethernet transport: every rank writes its block into every peer's buffer, then signals
    peers = [r for r in range(world) if r != rank]
    cfg = N.EndpointConfig(N.Transport.Ethernet, N.Device(N.DeviceType.CPU))
    conns = group.make_connection(peers, cfg)
    block = 1024
    buf = np.zeros(world * block, dtype=np.int64)
    buf[rank * block:(rank + 1) * block] = 1000 * (rank + 1) + np.arange(block)
    mems = group.register_tensor_with_connections(buf, conns)
    sems = {p: N.Host2HostSemaphore(s) for p, s in group.make_semaphores(conns).items()}
    for p in peers:
        conns[p].write(mems[p], rank * block * 8, mems[rank], rank * block * 8, block * 8)
        sems[p].signal()
    for p in peers:
        conns[p].flush()
        sems[p].wait()
    expect = np.concatenate([1000 * (r + 1) + np.arange(block) for r in range(world)])
    report("ethernet/all_pairs_write_and_signal", bool((buf == expect).all()))
    group.barrier()

    # ---- failure detection, host side. The last rank leaves now, between two steps, with nothing of its own in flight.
    leaver = world - 1
    if rank == leaver:
        dist.destroy_process_group()
        sys.exit(0)
    # (a) a wait for a signal that will never come gives up after its spin limit instead of hanging
    t0 = time.time()
    try:
        sems[leaver].wait(2_000_000)
        report("failure/semaphore_wait_gives_up", False)
    except N.Error as e:
        report("failure/semaphore_wait_gives_up", e.error_code == N.ErrorCode.Timeout, seconds=round(time.time() - t0, 2))
    # (b) a new bootstrap that the leaver never joins times out on every remaining rank
    port_box = [None]
    if rank == 0:
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port_box[0] = s.getsockname()[1]
    sub = dist.new_group(ranks=list(range(world - 1)))
    dist.broadcast_object_list(port_box, src=0, group=sub)
    again = N.TcpBootstrap.create(rank, world)
    t0 = time.time()
    try:
        again.initialize(f"127.0.0.1:{port_box[0]}", 2)
        report("failure/bootstrap_times_out", False)
    except N.Error as e:
        # rank 0 runs into its time limit; another survivor may instead see rank 0 give up and close the connection first.
        # Either way the call ends with an error within its bound instead of hanging.
        bounded = time.time() - t0 < 30
        ok = bounded and (e.error_code == N.ErrorCode.Timeout or rank != 0)
        if not ok:
            print(json.dumps({"rank": rank, "bootstrap_error": str(e), "code": str(e.error_code)}), flush=True)
        report("failure/bootstrap_times_out", ok, seconds=round(time.time() - t0, 2))
    # (c) the survivors carry on among themselves
    smaller = N.TcpBootstrap.create(rank, world - 1)
    if rank == 0:
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port_box[0] = s.getsockname()[1]
    dist.broadcast_object_list(port_box, src=0, group=sub)
    smaller.initialize(f"127.0.0.1:{port_box[0]}", 20)
    got = smaller.all_gather(bytes([rank + 10]))
    report("failure/survivors_regroup", got == [bytes([r + 10]) for r in range(world - 1)])
    smaller.barrier()
    dist.barrier(group=sub)
    if failures:
        print(json.dumps({"rank": rank, "failures": failures}), flush=True)
        sys.exit(1)
    os._exit(0)  # the default process group lost a member; skip its teardown


if __name__ == "__main__":
    main()
