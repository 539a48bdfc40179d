"""Expert-parallel MoE token exchange: dispatch (push over NVLink into an expert-grouped receive buffer) and
combine (pull the expert outputs back and apply the routing weights), one kernel each.

    disp = ExpertParallelDispatcher(symm, num_experts=64, hidden=4096, max_tokens=4096, topk=2)
    recv_x, counts, handle = disp.dispatch(x, topk_idx)          # recv_x rows are grouped by local expert
    expert_out = disp.expert_out                                  # write the experts' results into the same rows
    y = disp.combine(topk_idx, topk_weights, handle)

With ``fp8=True`` rows travel as e4m3 with one fp32 scale per 128 elements (``recv_x`` is uint8, scales in
``disp.recv_scales``), which halves the NVLink bytes of the dispatch. With ``fp8_combine=True`` the way back is halved
too: the expert outputs are combined from ``disp.expert_out_q`` (e4m3) and ``disp.expert_out_scales``, which the
experts' GEMM epilogue fills directly or ``disp.quantize_expert_out(rows)`` derives from ``disp.expert_out``. The
reference library has no MoE layer; it ships the bulk-copy primitives for writing one.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .._core import native
from .._core.symm import SymmetricMemory


class ExpertParallelDispatcher:
    def __init__(self, symm: SymmetricMemory, num_experts: int = 64, hidden: int = 4096, max_tokens: int = 4096, topk: int = 2,
                 capacity: Optional[int] = None, fp8: bool = False, fp8_combine: bool = False):
        assert num_experts % symm.world == 0 and hidden % 256 == 0
        self.symm, self.num_experts, self.hidden, self.max_tokens, self.topk, self.fp8 = symm, num_experts, hidden, max_tokens, topk, fp8
        self.experts_per_rank = num_experts // symm.world
        # uniform routing sends max_tokens * topk rows to every rank on average; leave room for imbalance
        self.capacity = capacity if capacity is not None else 2 * max_tokens * topk
        n = native.load()
        self.recv_x = symm.tensor((self.capacity, hidden), torch.uint8 if fp8 else torch.bfloat16)
        self.recv_scales = symm.tensor((self.capacity, hidden // 128), torch.float32) if fp8 else None
        self.recv_src = symm.tensor((self.capacity,), torch.int32)
        self.expert_out = symm.tensor((self.capacity, hidden), torch.bfloat16)
        self.fp8_combine = fp8_combine
        self.expert_out_q = symm.tensor((self.capacity, hidden), torch.uint8) if fp8_combine else None
        self.expert_out_scales = symm.tensor((self.capacity, hidden // 128), torch.float32) if fp8_combine else None
        self.workspace = symm.tensor((n.moe_workspace_bytes() // 4,), torch.int32)
        self.slot_map = symm.tensor((max_tokens, topk), torch.int32)
        self.recv_counts = symm.tensor((self.experts_per_rank + 1,), torch.int32)
        self.y = symm.tensor((max_tokens, hidden), torch.bfloat16)
        self._idx = symm.tensor((max_tokens, topk), torch.int32)
        self._weights = symm.tensor((max_tokens, topk), torch.float32)
        self._x = symm.tensor((max_tokens, hidden), torch.bfloat16)
        ranks = range(symm.world) if symm.emulated_mode else [symm.rank]
        for r in ranks:
            (symm.rank_view(self.workspace, r) if symm.emulated_mode else self.workspace).zero_()
        symm.barrier()  # peers write their counts into this workspace: nobody may start before everybody has zeroed it

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, n_blocks: int = 0,
                 stream: Optional[torch.cuda.Stream] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """x [T, hidden] bf16, topk_idx [T, topk] int32 (global expert ids, -1 = unused). Returns (recv_x, recv_counts,
        slot_map): rows [0, recv_counts[-1]) of recv_x are valid, the first recv_counts[0] belong to local expert 0, ...
        On emulated heaps pass x / topk_idx that are symmetric tensors filled per rank (see `stage`)."""
        n = native.load()
        t = x.shape[0]
        assert t <= self.max_tokens and x.shape[1] == self.hidden and topk_idx.shape == (t, self.topk)
        assert x.dtype == torch.bfloat16 and topk_idx.dtype == torch.int32 and x.is_contiguous() and topk_idx.is_contiguous()
        st = (stream or torch.cuda.current_stream()).cuda_stream
        n.moe_dispatch(self.symm.heap, x.data_ptr(), topk_idx.data_ptr(), self.slot_map.data_ptr(), self.recv_x.data_ptr(),
                       self.recv_scales.data_ptr() if self.fp8 else 0, self.recv_src.data_ptr(), self.recv_counts.data_ptr(),
                       self.workspace.data_ptr(), t, self.hidden, self.topk, self.num_experts, self.capacity, self.fp8, n_blocks, st)
        return self.recv_x, self.recv_counts, self.slot_map[:t]

    def quantize_expert_out(self, rows: int, rank: Optional[int] = None, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Quantise rows [0, rows) of expert_out into expert_out_q / expert_out_scales (e4m3, one scale per 128 elements).
        rank: which emulated rank's buffers (emulated heaps only)."""
        assert self.fp8_combine, "construct the dispatcher with fp8_combine=True"
        view = (lambda ten: self.symm.rank_view(ten, rank)) if (self.symm.emulated_mode and rank is not None) else (lambda ten: ten)
        st = (stream or torch.cuda.current_stream()).cuda_stream
        native.load().moe_quantize_rows(view(self.expert_out).data_ptr(), view(self.expert_out_q).data_ptr(), view(self.expert_out_scales).data_ptr(),
                                        rows, self.hidden, st)

    def combine(self, topk_idx: torch.Tensor, topk_weights: torch.Tensor, slot_map: torch.Tensor, expert_out: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, n_blocks: int = 0, stream: Optional[torch.cuda.Stream] = None,
                fp8: Optional[bool] = None) -> torch.Tensor:
        """y[t] = sum_k topk_weights[t, k] * expert_out(rank of expert k)[slot_map[t, k]]; returns y [T, hidden] bf16.
        fp8 (default: the dispatcher's fp8_combine): pull the rows from expert_out_q / expert_out_scales instead."""
        n = native.load()
        t = topk_idx.shape[0]
        fp8 = self.fp8_combine if fp8 is None else fp8
        if fp8:
            assert self.fp8_combine and expert_out is None
            expert_out = self.expert_out_q
        else:
            expert_out = self.expert_out if expert_out is None else expert_out
        out = self.y[:t] if out is None else out
        assert topk_weights.dtype == torch.float32 and topk_weights.shape == (t, self.topk) and slot_map.shape == (t, self.topk)
        st = (stream or torch.cuda.current_stream()).cuda_stream
        n.moe_combine(self.symm.heap, topk_idx.data_ptr(), topk_weights.data_ptr(), slot_map.data_ptr(), expert_out.data_ptr(), out.data_ptr(),
                      t, self.hidden, self.topk, self.num_experts, n_blocks, st, self.expert_out_scales.data_ptr() if fp8 else 0)
        return out

    # ------------------------------------------------------------------ helpers for tests and emulated heaps
    def stage(self, rank: int, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor] = None):
        """Copy one (emulated) rank's inputs into the symmetric staging tensors; returns the tensors to pass on."""
        t = x.shape[0]
        view = (lambda ten: self.symm.rank_view(ten, rank)) if self.symm.emulated_mode else (lambda ten: ten)
        view(self._x)[:t].copy_(x)
        view(self._idx)[:t].copy_(topk_idx)
        if topk_weights is not None:
            view(self._weights)[:t].copy_(topk_weights)
        return self._x[:t], self._idx[:t], self._weights[:t]


def dequantize_rows(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """uint8 e4m3 rows [R, H] with scales [R, H/128] -> fp32 [R, H] (the inverse of the dispatch quantiser)."""
    f = q.view(torch.float8_e4m3fn).float()
    return (f.view(q.shape[0], -1, 128) * scales.unsqueeze(-1)).view(q.shape[0], -1)
