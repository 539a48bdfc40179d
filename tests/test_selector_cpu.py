"""The Python allreduce selector on a stand-in for the heap (no GPU): which algorithm a size gets at 2, 4 and 8 ranks,
with and without a multicast mapping, for buffers inside and outside the heap. Pins the measured switch-over points."""
import struct
from types import SimpleNamespace

import pytest

from mscclpp_b200.ops import collectives as C


def _symm(world, nvls, ll_slot_bytes=16 << 20, emulated=False):
    raw = bytearray(8 * 32)
    struct.pack_into("<Q", raw, 8 * 19, ll_slot_bytes)
    heap = SimpleNamespace(device_comm_bytes=lambda: bytes(raw))
    return SimpleNamespace(world=world, nvls=nvls, emulated_mode=emulated, heap=heap)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("nvls", [False, True])
def test_symmetric_buffers(world, nvls):
    s = _symm(world, nvls)
    small = "nvls_packet" if nvls else "packet"
    for n in (1 << 10, 32 << 10, 64 << 10):
        assert C.select_allreduce(s, n, True) == small
    assert C.select_allreduce(s, (64 << 10) + 16, True) == "packet128"
    top = C.ll128_max_bytes(world)
    assert top == {2: 4 << 20, 4: 512 << 10, 8: 256 << 10}[world]
    assert C.select_allreduce(s, top, True) == "packet128"
    beyond = C.select_allreduce(s, top + 16, True)
    assert beyond in ("packet", "nvls_zero_copy", "rsag_zero_copy")
    big = C.select_allreduce(s, 256 << 20, True)
    if not nvls or world == 2:
        assert big == "rsag_zero_copy"  # two ranks: the switch has nothing to combine from 4 MB on
    else:
        assert big == "nvls_zero_copy"
    if nvls and world == 2:
        assert C.select_allreduce(s, (4 << 20) + 16, True) == "rsag_zero_copy"


@pytest.mark.parametrize("world", [2, 8])
def test_buffers_outside_the_heap_take_the_pipelined_kernels(world):
    s = _symm(world, True)
    big = C.select_allreduce(s, 64 << 20, False)
    assert big == ("rsag_pipeline" if world == 2 else "nvls_block_pipeline")
    assert C.select_allreduce(_symm(world, False), 64 << 20, False) == "rsag_pipeline"
    assert C.select_allreduce(s, 8 << 10, False) == "nvls_packet"


def test_packet_range_is_bounded_by_the_scratch():
    tiny = _symm(8, True, ll_slot_bytes=32 << 10)  # room for 16 KB of payload per slot
    assert C.select_allreduce(tiny, 8 << 10, True) == "nvls_packet"
    assert C.select_allreduce(tiny, 32 << 10, True) != "nvls_packet"


def test_zero_copy_needs_whole_16_byte_words():
    with pytest.raises(ValueError):
        C.select_allreduce(_symm(8, True), (64 << 20) + 2, True)


def test_grids_are_sized_for_one_block_per_sm():
    for world in (2, 4, 8):
        for algo in ("packet", "nvls_packet", "rsag_zero_copy", "nvls_zero_copy"):
            for n in (1 << 10, 1 << 20, 64 << 20):
                blocks, threads = C._grid_for(n, algo, world)
                assert 1 <= blocks <= 148 and 32 <= threads <= 1024
