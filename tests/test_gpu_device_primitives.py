"""Header-only device primitives (packets, copies, grid syncer, device semaphore, bounded waits), exercised through
small kernels compiled at run time with KernelBuilder against the package's headers."""
import ctypes
import os
import struct

import pytest
import torch

pytestmark = pytest.mark.gpu
KDIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels")


def _kernel(name):
    from mscclpp_b200.utils import KernelBuilder

    return KernelBuilder("device_primitives.cu", name, file_dir=KDIR).get_compiled_kernel()


def _offsets(fmt):
    """Byte offset of every field of a struct format (native alignment), for cooperative launches."""
    offs, pos = [], 0
    for ch in fmt:
        size = struct.calcsize(ch)
        pos = (pos + size - 1) // size * size
        offs.append(pos)
        pos += size
    return offs


@pytest.mark.parametrize("kind,nbytes", [(8, 4096), (16, 4096), (16, 1 << 20)])
def test_packets_cross_block(kind, nbytes):
    k = _kernel("packetPingPong")
    src = torch.randint(0, 2**31 - 1, (nbytes // 4,), dtype=torch.int32, device="cuda")
    packets = torch.zeros(nbytes * 2 // 4, dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    failed = torch.zeros(1, dtype=torch.int32, device="cuda")
    for flag in (1, 2):  # the second round reuses the packet buffer: only the new flag is accepted
        src.add_(flag)
        fmt = "PPPQIiP"
        params = struct.pack(fmt, src.data_ptr(), packets.data_ptr(), dst.data_ptr(), nbytes, flag, kind, failed.data_ptr())
        k.launch_kernel(params, 2, 256, stream=torch.cuda.current_stream(), cooperative=True, offsets=_offsets(fmt))
        torch.cuda.synchronize()
        assert int(failed.item()) == 0
        assert torch.equal(dst, src)


def test_ll128_lines_cross_block():
    k = _kernel("ll128PingPong")
    lines = 300
    src = torch.randint(0, 2**31 - 1, (lines * 8 * 4,), dtype=torch.int32, device="cuda")
    view = src.view(lines, 8, 4)
    view[:, 7, 2:] = 0  # the last 8 bytes of a line carry the flag, not payload
    buf = torch.zeros(lines * 32, dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    failed = torch.zeros(1, dtype=torch.int32, device="cuda")
    fmt = "PPPiQP"
    params = struct.pack(fmt, src.data_ptr(), buf.data_ptr(), dst.data_ptr(), lines, 0xABCD00000001, failed.data_ptr())
    k.launch_kernel(params, 2, 256, stream=torch.cuda.current_stream(), cooperative=True, offsets=_offsets(fmt))
    torch.cuda.synchronize()
    assert int(failed.item()) == 0
    assert torch.equal(dst, src)


@pytest.mark.parametrize("nbytes,src_off,dst_off", [(1, 0, 0), (13, 1, 3), (4099, 3, 3), (65536 + 7, 8, 1), (1 << 20, 16, 16)])
def test_copy_bytes_any_alignment(nbytes, src_off, dst_off):
    k = _kernel("copyOdd")
    src = torch.randint(0, 255, (nbytes + 64,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(nbytes + 64, dtype=torch.uint8, device="cuda")
    params = struct.pack("PPQ", dst.data_ptr() + dst_off, src.data_ptr() + src_off, nbytes)
    k.launch_kernel(params, 4, 128, stream=torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert torch.equal(dst[dst_off:dst_off + nbytes], src[src_off:src_off + nbytes])
    assert int(dst[:dst_off].sum()) == 0 and int(dst[dst_off + nbytes:].sum()) == 0  # nothing written outside


def test_device_syncer_rounds():
    k = _kernel("syncerRounds")
    blocks, rounds = 32, 5
    syncer = torch.zeros(4, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(blocks, dtype=torch.int32, device="cuda")
    sums = torch.zeros(rounds * blocks, dtype=torch.int32, device="cuda")
    failed = torch.zeros(1, dtype=torch.int32, device="cuda")
    fmt = "PPPiP"
    params = struct.pack(fmt, syncer.data_ptr(), scratch.data_ptr(), sums.data_ptr(), rounds, failed.data_ptr())
    k.launch_kernel(params, blocks, 64, stream=torch.cuda.current_stream(), cooperative=True, offsets=_offsets(fmt))
    torch.cuda.synchronize()
    assert int(failed.item()) == 0
    total = blocks * (blocks + 1) // 2
    expect = torch.tensor([(r + 1) * total for r in range(rounds) for _ in range(blocks)], dtype=torch.int32, device="cuda")
    assert torch.equal(sums, expect)


def test_device_semaphore_hand_off():
    k = _kernel("semaphoreHandOff")
    sem = torch.zeros(4, dtype=torch.int32, device="cuda")
    acquired = torch.zeros(1, dtype=torch.int32, device="cuda")
    failed = torch.zeros(1, dtype=torch.int32, device="cuda")
    fmt = "PiPP"
    params = struct.pack(fmt, sem.data_ptr(), 100, acquired.data_ptr(), failed.data_ptr())
    k.launch_kernel(params, 2, 32, stream=torch.cuda.current_stream(), cooperative=True, offsets=_offsets(fmt))
    torch.cuda.synchronize()
    assert int(failed.item()) == 0 and int(acquired.item()) == 100


def test_packet_wait_runs_out_and_reports():
    """Failure detection on the device: a wait whose flag never comes returns after its budget and leaves a record."""
    k = _kernel("packetWaitRunsOut")
    packets = torch.zeros(16, dtype=torch.int32, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")  # DeviceStatus, 64 bytes
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    params = struct.pack("PPQP", packets.data_ptr(), status.data_ptr(), 50_000_000, gave_up.data_ptr())  # 50 ms
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    k.launch_kernel(params, 1, 32, stream=torch.cuda.current_stream())
    end.record()
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 1
    assert 40.0 <= start.elapsed_time(end) < 2000.0
    st = status.cpu().tolist()
    assert st[0] == 2 and st[1] == 1, st[:4]  # code = packet time-out, poisoned
    # the context is still usable
    assert int((torch.ones(4, device="cuda") * 2).sum().item()) == 8


def test_fifo_push_with_and_without_a_consumer():
    """GPU -> host FIFO: triggers pushed by a kernel arrive in order on the host; with a stalled consumer the ring
    fills up and further pushes give up after their budget instead of spinning forever."""
    from mscclpp_b200 import native

    n = native()
    k = _kernel("fifoPush")
    fifo = n.Fifo(8)
    accepted = torch.zeros(1, dtype=torch.int32, device="cuda")
    raw = bytes(fifo.device_handle().raw)
    # stalled proxy: nobody pops; 8 slots accept 8 triggers, the 9th waits 30 ms and gives up
    params = raw + struct.pack("iQP", 12, 30_000_000, accepted.data_ptr())
    pad = (-len(raw)) % 8
    params = raw + b"\x00" * pad + struct.pack("iQP", 12, 30_000_000, accepted.data_ptr())
    k.launch_kernel(params, 1, 32, stream=torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert int(accepted.item()) == 8
    got = []
    while True:
        t = fifo.poll()
        if t.fst == 0:
            break
        got.append(t.fst)
        fifo.pop()
    assert got == list(range(1, 9))
