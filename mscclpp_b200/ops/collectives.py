"""Collective operations on symmetric memory, dispatched to the native sm_100a kernels.

Algorithm names follow the reference's default collection
(src/ext/collectives/algorithm_collection_builder.cc:64-104):
  "packet" / "nvls_packet"          one-shot LL16 over peer stores / one multimem.st per packet
  "allpair_packet"                  one-shot with 8-byte LL8 packets over peer stores
  "packet128"                       one-shot with 128-byte LL128 lines (120 bytes of payload + flag) over peer stores
  "rsag_zero_copy"                  two-shot over peer loads+stores, zero copy
  "nvls_zero_copy"                  two-shot through NVSwitch multimem.ld_reduce + multimem.st
  "nvls_block_pipeline" / "rsag_pipeline"   tensors OUTSIDE the heap: one kernel copies in, reduces through heap scratch
                                    (switch reduction / peer loads) and copies out, slice by slice
The selector mirrors the shape of the reference's Blackwell table
(src/ext/nccl/algorithm_selector.cc:52-89) with thresholds measured on B200.
"""
from __future__ import annotations

from typing import Optional

import torch

from .._core import native
from .._core.symm import SymmetricMemory, torch_dtype_to_native

MODE_ALLREDUCE, MODE_REDUCE_SCATTER, MODE_ALLGATHER, MODE_BROADCAST, MODE_ALLTOALL = 0, 1, 2, 3, 4

# bytes at or below which the one-shot LL path wins (tuned on 8xB200; see profiles/)
LL_MAX_BYTES = 512 << 10


def _stream(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _op(op: str):
    n = native.load()
    return {"sum": n.ReduceOp.SUM, "min": n.ReduceOp.MIN}[op]


def ll_max_bytes(world: int) -> int:
    """Largest message for which the one-shot packet algorithm wins (every rank sends its whole buffer to every peer, so
    the range shrinks as the world grows; measured on 2, 4 and 8 B200s)."""
    return (1 << 20) if world <= 2 else ((256 << 10) if world <= 4 else (128 << 10))


def select_allreduce(symm: SymmetricMemory, nbytes: int, symmetric: bool) -> str:
    ll_cap = _ll_capacity(symm)
    ll_max = ll_max_bytes(symm.world) * (1 if symmetric else 2)
    if nbytes <= (64 << 10) and nbytes <= ll_cap:
        return "nvls_packet" if symm.nvls else "packet"
    # 128-byte lines (15/16 payload) are ahead of the 16-byte packets from 64 KB on and of the two-shot kernels (two cross-rank
    # barriers, ~20 us before the first byte) up to a few MB: measured on two B200s in graph replay, 1 MB 7.1 vs 10.4 us
    # with LL16, 2 MB 11.0 vs 23.7 us two-shot, 4 MB 18.6 vs 27.2 us
    if nbytes <= ll128_max_bytes(symm.world) and (symmetric or not symm.emulated_mode):
        return "packet128"
    if nbytes <= min(ll_max, ll_cap):
        return "packet"
    # with two ranks the switch has nothing to combine: plain peer loads and stores on 128 SMs win from 4 MB on
    use_switch = symm.nvls and (symm.world > 2 or nbytes < (4 << 20))
    if not symmetric:  # (the pipelined kernels were tuned separately: through the switch up to 16 MB)
        return "nvls_block_pipeline" if symm.nvls and (symm.world > 2 or nbytes < (16 << 20)) else "rsag_pipeline"
    if nbytes % 16 != 0:
        raise ValueError("zero-copy allreduce needs a multiple of 16 bytes")
    return "nvls_zero_copy" if use_switch else "rsag_zero_copy"


PIPELINE_SLICE_BYTES = 64 << 10
PIPELINE_MAX_BLOCKS = 128


def _pipeline_scratch(symm: SymmetricMemory) -> torch.Tensor:
    """Heap scratch of the pipelined allreduce, made on first use (every rank gets here on the same call)."""
    cache = symm.__dict__.setdefault("_pipeline_scratch", None)
    if cache is None:
        n = native.load()
        nbytes = n.pipeline_scratch_bytes(PIPELINE_MAX_BLOCKS, _pipeline_slice(symm))
        cache = symm.tensor((nbytes,), torch.uint8)
        symm.__dict__["_pipeline_scratch"] = cache
    return cache


def _pipeline_slice(symm: SymmetricMemory) -> int:
    unit = 16 * symm.world
    return (PIPELINE_SLICE_BYTES + unit - 1) // unit * unit


def ll128_max_bytes(world: int) -> int:
    """Largest message the LL128 scratch is sized for: every rank receives the whole message from every peer, so the
    useful range (and the scratch, 2 x world x 1.07 x this) shrinks as the world grows (measured on eight B200s in graph
    replay: 256 KB 10.8 us against 22.6 us two-shot through the switch, 512 KB 17.8 against 23.2, 1 MB 33.0 against 24.1)."""
    return (4 << 20) if world <= 2 else ((512 << 10) if world <= 4 else (256 << 10))



def _ll128_scratch(symm: SymmetricMemory):
    """Heap scratch of the LL128 allreduce, made and zeroed on first use (every rank gets here on the same call)."""
    cache = symm.__dict__.get("_ll128_scratch")
    if cache is None:
        slot = (ll128_max_bytes(symm.world) + 119) // 120 * 128
        buf = symm.tensor((2 * symm.world * slot,), torch.uint8)
        ranks = range(symm.world) if symm.emulated_mode else [symm.rank]
        for r in ranks:
            (symm.rank_view(buf, r) if symm.emulated_mode else buf).zero_()
        torch.cuda.synchronize()
        symm.barrier()  # peers write lines into this scratch: nobody may start before everybody has zeroed it
        cache = (buf, slot)
        symm.__dict__["_ll128_scratch"] = cache
    return cache


def _ll_capacity(symm: SymmetricMemory) -> int:
    import struct

    raw = symm.heap.device_comm_bytes()
    # DeviceComm: 16 x u64 peerBase, mcBase, heapBytes, llScratchOff, llSlotBytes, ...
    ll_slot = struct.unpack_from("<Q", raw, 8 * 19)[0]
    return ll_slot // 2


def _grid_for(nbytes: int, algo: str, world: int) -> tuple[int, int]:
    if algo in ("packet", "nvls_packet", "allpair_packet"):
        units = max(1, (nbytes + 15) // 16)
        threads = 512
        blocks = max(1, min(56, (units + threads - 1) // threads))
        return blocks, threads
    if algo == "nvls_zero_copy":
        blocks = 16 if nbytes < (8 << 20) else (32 if nbytes < (64 << 20) else 64)
        return blocks, 512
    # peer loads are bound by what ONE SM can keep in flight over NVLink (measured on two B200s: 16 MB takes 100 / 61 /
    # 52 us with 32 / 64 / 128 thread blocks, and more than one block per SM is slower again): from 1 MB on, one block per
    # SM, 128 of them
    blocks = 32 if nbytes < (1 << 20) else 128
    return blocks, 512


def all_reduce(symm: SymmetricMemory, inp: torch.Tensor, out: Optional[torch.Tensor] = None, op: str = "sum",
               algo: Optional[str] = None, stream: Optional[torch.cuda.Stream] = None, n_blocks: int = 0,
               n_threads: int = 0) -> torch.Tensor:
    """out = reduce over ranks of inp (out defaults to inp, i.e. in place)."""
    n = native.load()
    out = inp if out is None else out
    assert inp.is_contiguous() and out.is_contiguous() and inp.dtype == out.dtype and inp.numel() == out.numel()
    nbytes = _nbytes(inp)
    if symm.emulated_mode or symm.world == 1:
        symmetric = symm.contains(inp) and symm.contains(out)
    else:  # agreed among the ranks: a rank-local test could send them into different kernels
        symmetric = symm.heap.symmetric_on_all_ranks(inp.data_ptr(), nbytes) and symm.heap.symmetric_on_all_ranks(out.data_ptr(), nbytes)
    algo = algo or select_allreduce(symm, nbytes, symmetric)
    if algo in ("nvls_block_pipeline", "rsag_pipeline"):
        scratch = _pipeline_scratch(symm)
        slice_bytes = _pipeline_slice(symm)
        blocks = n_blocks or max(1, min(PIPELINE_MAX_BLOCKS, (nbytes + slice_bytes - 1) // slice_bytes))
        emu_stride = 0
        if symm.emulated_mode:  # emulated ranks: row r of a [world, ...] tensor is rank r's buffer
            assert inp.shape[0] == symm.world and out.shape[0] == symm.world
            nbytes //= symm.world
            emu_stride = nbytes
            blocks = min(blocks, 16)
        n.pipeline_allreduce(symm.heap, inp.data_ptr(), out.data_ptr(), nbytes, torch_dtype_to_native(inp.dtype), _op(op), scratch.data_ptr(),
                             slice_bytes, blocks, n_threads or 512, _stream(stream), algo == "nvls_block_pipeline", emu_stride)
        return out
    blocks, threads = _grid_for(nbytes, algo, symm.world)
    blocks = n_blocks or blocks
    threads = n_threads or threads
    dt = torch_dtype_to_native(inp.dtype)
    if algo in ("packet", "nvls_packet", "allpair_packet"):
        if symm.emulated_mode and not symmetric:
            raise ValueError("emulated ranks need heap tensors")
        n.allreduce_ll(symm.heap, inp.data_ptr(), out.data_ptr(), nbytes, dt, _op(op), blocks, threads, _stream(stream),
                       algo == "nvls_packet", algo == "allpair_packet")
    elif algo == "packet128":
        if nbytes > ll128_max_bytes(symm.world):
            raise ValueError("packet128 takes messages up to ll128_max_bytes(world)")
        if symm.emulated_mode and not symmetric:
            raise ValueError("emulated ranks need heap tensors")
        scratch, slot = _ll128_scratch(symm)
        lines = (nbytes + 119) // 120
        blocks = n_blocks or max(1, min(64, (lines * 8 + 511) // 512))
        n.allreduce_ll128(symm.heap, inp.data_ptr(), out.data_ptr(), nbytes, dt, _op(op), scratch.data_ptr(), slot, blocks, n_threads or 512,
                          _stream(stream))
    elif algo in ("rsag_zero_copy", "nvls_zero_copy"):
        if not symmetric:
            raise ValueError(f"{algo} needs tensors from symm.tensor()")
        n.two_shot(symm.heap, inp.data_ptr(), out.data_ptr(), nbytes, dt, _op(op), MODE_ALLREDUCE, blocks, threads,
                   _stream(stream), algo == "nvls_zero_copy")
    else:
        raise ValueError(f"unknown allreduce algorithm {algo}")
    return out


def reduce_scatter(symm: SymmetricMemory, inp: torch.Tensor, out: torch.Tensor, op: str = "sum", nvls: Optional[bool] = None,
                   stream: Optional[torch.cuda.Stream] = None, n_blocks: int = 0) -> torch.Tensor:
    """out (1/world of inp) = this rank's slice of the reduction. Both tensors from symm.tensor()."""
    n = native.load()
    nvls = symm.nvls if nvls is None else nvls
    assert _nbytes(inp) == _nbytes(out) * symm.world
    blocks, threads = _grid_for(_nbytes(inp), "nvls_zero_copy" if nvls else "rsag_zero_copy", symm.world)
    n.two_shot(symm.heap, inp.data_ptr(), out.data_ptr(), _nbytes(inp), torch_dtype_to_native(inp.dtype), _op(op),
               MODE_REDUCE_SCATTER, n_blocks or blocks, threads, _stream(stream), nvls)
    return out


def all_gather(symm: SymmetricMemory, inp: torch.Tensor, out: torch.Tensor, nvls: Optional[bool] = None,
               stream: Optional[torch.cuda.Stream] = None, n_blocks: int = 0) -> torch.Tensor:
    """out (world x inp) = concatenation of every rank's inp. Both tensors from symm.tensor()."""
    n = native.load()
    nvls = symm.nvls if nvls is None else nvls
    assert _nbytes(out) == _nbytes(inp) * symm.world
    blocks, threads = _grid_for(_nbytes(out), "nvls_zero_copy" if nvls else "rsag_zero_copy", symm.world)
    n.two_shot(symm.heap, inp.data_ptr(), out.data_ptr(), _nbytes(out), torch_dtype_to_native(inp.dtype), _op("sum"),
               MODE_ALLGATHER, n_blocks or blocks, threads, _stream(stream), nvls)
    return out


def broadcast(symm: SymmetricMemory, inp: torch.Tensor, out: torch.Tensor, root: int, nvls: Optional[bool] = None,
              stream: Optional[torch.cuda.Stream] = None, n_blocks: int = 0) -> torch.Tensor:
    """Every rank's `out` = the root's `inp` (the root streams its buffer: one multimem.st, or one store per peer, per
    16 bytes). `out` from symm.tensor(); sizes multiples of 16 bytes."""
    n = native.load()
    nvls = symm.nvls if nvls is None else nvls
    assert _nbytes(inp) == _nbytes(out) and 0 <= root < symm.world
    blocks, threads = _grid_for(_nbytes(out), "nvls_zero_copy" if nvls else "rsag_zero_copy", symm.world)
    n.two_shot(symm.heap, inp.data_ptr(), out.data_ptr(), _nbytes(out), n.DataType.uint32, _op("sum"), MODE_BROADCAST, n_blocks or blocks,
               threads, _stream(stream), nvls, root)
    return out


def all_to_all(symm: SymmetricMemory, inp: torch.Tensor, out: torch.Tensor, stream: Optional[torch.cuda.Stream] = None,
               n_blocks: int = 0) -> torch.Tensor:
    """Chunk p of `inp` becomes chunk `rank` of rank p's `out` (equal chunks, peer stores). `out` from symm.tensor()."""
    n = native.load()
    assert _nbytes(inp) == _nbytes(out) and _nbytes(inp) % (16 * symm.world) == 0 and inp.data_ptr() != out.data_ptr()
    blocks, threads = _grid_for(_nbytes(out), "rsag_zero_copy", symm.world)
    n.two_shot(symm.heap, inp.data_ptr(), out.data_ptr(), _nbytes(out), n.DataType.uint32, _op("sum"), MODE_ALLTOALL, n_blocks or blocks,
               threads, _stream(stream), False, 0)
    return out


def _rinv_buffer(symm: SymmetricMemory, rows: int) -> torch.Tensor:
    """Symmetric fp32 [rows] scratch for the per-row 1/rms, allocated once per heap (every rank asks in the same order)."""
    cache = symm.__dict__.setdefault("_rinv_cache", {})
    cap = 1
    while cap < rows:
        cap <<= 1
    if cap not in cache:
        cache[cap] = symm.tensor((cap,), torch.float32)
    return cache[cap]


def all_reduce_rmsnorm(symm: SymmetricMemory, inp: torch.Tensor, out: torch.Tensor, residual_in: Optional[torch.Tensor],
                       residual_out: Optional[torch.Tensor], gamma: Optional[torch.Tensor], eps: float = 1e-5,
                       algo: Optional[str] = None, stream: Optional[torch.cuda.Stream] = None, n_blocks: int = 0) -> torch.Tensor:
    """Fused: h = allreduce(inp) + residual_in; residual_out = h; out = rmsnorm(h) * gamma.

    inp/out/residual_* are [rows, hidden]; residual_in is replicated on every rank (tensor parallel
    residual stream). One kernel: the reduction, the residual add and the norm never round-trip
    through HBM separately.
    """
    n = native.load()
    rows, hidden = inp.shape
    nbytes = _nbytes(inp)
    symmetric = all(symm.contains(t) for t in (inp, out) if t is not None) and \
        all(symm.contains(t) for t in (residual_in, residual_out) if t is not None)
    if algo is None:
        small = nbytes <= min(LL_MAX_BYTES, _ll_capacity(symm)) or rows < symm.world or not symmetric
        rows_ok = inp.dtype == torch.bfloat16 and hidden % 8 == 0 and hidden <= 8192 and not symm.emulated_mode
        algo = "packet" if small else ("rows" if rows_ok else ("nvls_zero_copy" if symm.nvls else "rsag_zero_copy"))
    dt = torch_dtype_to_native(inp.dtype)
    ptr = lambda t: 0 if t is None else t.data_ptr()
    if algo in ("rows", "rows_p2p"):
        # row-owner kernel: 64-thread groups keep a whole row in registers; with a residual stream the owners broadcast
        # h and one 1/rms per row only and every rank finishes `out` locally (half the NVLink bytes)
        if not symmetric or inp.dtype != torch.bfloat16:
            raise ValueError("the row-owner kernel needs bf16 tensors from symm.tensor()")
        mode = 1 if residual_out is not None else 0
        rinv = _rinv_buffer(symm, rows) if mode == 1 else None
        nvls = symm.nvls and algo == "rows"
        n.tp_reduce_norm(symm.heap, inp.data_ptr(), ptr(residual_in), ptr(residual_out), out.data_ptr(), ptr(gamma), ptr(rinv), rows, hidden,
                         eps, n_blocks, 0, mode, nvls, _stream(stream))
        if mode == 1:
            n.tp_scale_rows(residual_out.data_ptr(), rinv.data_ptr(), ptr(gamma), out.data_ptr(), rows, hidden, _stream(stream))
        return out
    if algo in ("packet", "nvls_packet"):
        blocks = n_blocks or max(1, min(rows, 64))
        threads = 1024 if hidden * inp.element_size() // 16 >= 1024 else 512
        n.allreduce_ll_rmsnorm(symm.heap, inp.data_ptr(), out.data_ptr(), rows, hidden, dt, eps, ptr(residual_in),
                               ptr(residual_out), ptr(gamma), blocks, threads, _stream(stream), algo == "nvls_packet")
    else:
        if not symmetric:
            raise ValueError(f"{algo} needs tensors from symm.tensor()")
        own_rows = (rows + symm.world - 1) // symm.world
        blocks = n_blocks or max(1, min(own_rows, 128))
        n.two_shot_rmsnorm(symm.heap, inp.data_ptr(), out.data_ptr(), rows, hidden, dt, eps, ptr(residual_in),
                           ptr(residual_out), ptr(gamma), True, blocks, 512, _stream(stream), algo == "nvls_zero_copy")
    return out
