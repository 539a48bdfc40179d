"""Tensor-parallel row-parallel projection with the collective fused into it.

    y = RMSNorm( allreduce_over_ranks( x_shard @ W_shard^T ) + residual ) * gamma

This is the attention out-projection (or MLP down-projection) of a TP decoder layer: each rank holds
a K-shard of the weight, the partial products are summed over ranks, added to the residual stream
and normalised for the next block. The reference library offers only the allreduce for this (its
motivating TP example allreduces a [2048, 8192] bf16 activation, test/torch/allreduce_temp_buff.py:22-60);
here the GEMM runs on tcgen05 tensor cores and the reduction, residual add and norm are one kernel
reading the partial products straight out of every rank's symmetric heap.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .._core.symm import SymmetricMemory
from ..ops.collectives import all_reduce_rmsnorm
from ..ops.gemm import gemm_bf16, pick_block_n


class RowParallelLinearNorm:
    """Weights are stored [out_features, k_shard] (nn.Linear layout of the rank's K slice)."""

    def __init__(self, symm: SymmetricMemory, out_features: int = 8192, k_shard: int = 1024, max_tokens: int = 8192,
                 eps: float = 1e-5, seed: int = 0, init_std: float = 0.02):
        self.symm = symm
        self.out_features = out_features
        self.k_shard = k_shard
        self.max_tokens = max_tokens
        self.eps = eps
        dev = symm.device
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + symm.rank)
        self.weight = (torch.randn((out_features, k_shard), generator=g, device=dev) * init_std).to(torch.bfloat16)
        # everything the collective kernel touches lives in the symmetric heap, at equal offsets on all ranks
        self.partial = symm.tensor((max_tokens, out_features), torch.bfloat16)
        self.out = symm.tensor((max_tokens, out_features), torch.bfloat16)
        self.residual_in = symm.tensor((max_tokens, out_features), torch.bfloat16)
        self.residual_out = symm.tensor((max_tokens, out_features), torch.bfloat16)
        self.gamma = symm.tensor((out_features,), torch.bfloat16)
        self.gamma.fill_(1.0)
        self.rinv = symm.tensor((max_tokens,), torch.float32)
        self._local_ws = None  # workspace of the one-kernel single-GPU path, made on first use
        self._sumsq_parts = None  # parts of the rows' sums of squares between the two launches of the two-kernel path
        self.launches_per_forward = 1  # forward_fused, mode 0

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, algo: Optional[str] = None,
                stream: Optional[torch.cuda.Stream] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: [T, k_shard] bf16 (this rank's activation shard). residual: [T, out_features] or None to
        use what is already in self.residual_in. Returns (normalised output, new residual), both [T, out]."""
        t = x.shape[0]
        assert t <= self.max_tokens and x.shape[1] == self.k_shard
        partial = self.partial[:t]
        if residual is not None:
            self.residual_in[:t].copy_(residual)
        gemm_bf16(x, self.weight, partial, stream=stream)  # two-SM tiles when the problem fills the GPU, else one-SM
        out, res_out = self.out[:t], self.residual_out[:t]
        all_reduce_rmsnorm(self.symm, partial, out, self.residual_in[:t], res_out, self.gamma, eps=self.eps, algo=algo,
                           stream=stream)
        return out, res_out

    def forward_fused(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, mode: Optional[int] = None,
                      nvls: Optional[bool] = None, block_n: int = 0, num_reducers: int = 0, num_gemm_ctas: int = 0,
                      rows_per_unit: int = 0, stream: Optional[torch.cuda.Stream] = None,
                      emulated_inputs=None, timeline: Optional[torch.Tensor] = None, row_offset: int = 0,
                      sys_fence: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Same result as forward(), in ONE kernel: GEMM tiles, cross-rank reduction, residual add and norm
        overlap tile by tile. mode 1 halves NVLink traffic by broadcasting h and 1/rms only and finishing
        `out` with a local pass (second, local-only launch); mode 0 is one launch; mode 3 is mode 1 with the local pass
        inside the same launch (owners announce the row units that have landed everywhere, and warps without a row to
        reduce turn landed rows into `out`). Default: mode 1 from 1024 tokens on
        (measured on 2 and 8 GPUs: the saved bytes outweigh the second launch there), else mode 0. block_n: N tile of the one-SM GEMM core (64/128/256), -1
        forces the two-SM core (256 x 256 tiles on SM pairs), 0 picks (two-SM from 1024 tokens on).

        emulated_inputs: for emulated heaps, [(x_r, weight_r)] for every emulated rank.
        timeline: optional int64 CUDA tensor [grid CTAs, 16] that receives per-CTA time stamps (ns): start, GEMM part
        done, reducer part done, rows reduced / ns waited / ns worked by the CTA's first reducer group, first row done,
        and (words 8-10) the ns of the work spent in the gather, the residual math and the broadcast stores.
        row_offset: the rows of x are rows [row_offset, row_offset + T) of the layer's buffers (the same on every rank);
        used to run a long sequence as a few launches, e.g. while later rows are still arriving from the host.
        sys_fence: how a finished row block is announced to the peers. False: GPU-scope fence, then relaxed system-scope
        flag stores (the default: the partial product lives in this GPU's memory and every peer load passes through
        this GPU's L2). True: system-scope fence and release stores. None: environment variable MSCCLPP_TP_SYS_FENCE."""
        from .._core import native

        n = native.load()
        t = x.shape[0]
        assert row_offset + t <= self.max_tokens and x.shape[1] == self.k_shard and x.is_contiguous()
        if mode is None:
            mode = 1 if t >= 1024 else 0
        if residual is not None:
            self.residual_in[row_offset:row_offset + t].copy_(residual)
        nvls = self.symm.nvls if nvls is None else nvls
        if block_n < 0 or (block_n == 0 and t >= 1024 and self.out_features % 256 == 0):
            bn = 0  # 256 x 256 tiles on pairs of SMs (tcgen05 cta_group::2)
        else:
            bn = block_n or pick_block_n(t, self.out_features)
        s = (stream or torch.cuda.current_stream()).cuda_stream
        if emulated_inputs is not None:
            a_ptrs = [xi.data_ptr() for xi, _ in emulated_inputs]
            b_ptrs = [wi.data_ptr() for _, wi in emulated_inputs]
        else:
            a_ptrs, b_ptrs = [x.data_ptr()], [self.weight.data_ptr()]
        rows = slice(row_offset, row_offset + t)
        n.tp_fused(self.symm.heap, a_ptrs, b_ptrs, self.partial[rows].data_ptr(), self.residual_in[rows].data_ptr(),
                   self.residual_out[rows].data_ptr(), self.out[rows].data_ptr(), self.gamma.data_ptr(), self.rinv[rows].data_ptr(), t,
                   self.out_features, self.k_shard, self.eps, bn, num_gemm_ctas, num_reducers, rows_per_unit, mode, nvls, s,
                   0 if timeline is None else timeline.data_ptr(), -1 if sys_fence is None else int(bool(sys_fence)))
        if mode == 1:  # (mode 3 has produced `out` already)
            ranks = range(self.symm.world) if self.symm.emulated_mode else [self.symm.rank]
            for r in ranks:  # one local pass per (emulated) rank
                view = (lambda t_: self.symm.rank_view(t_, r)) if self.symm.emulated_mode else (lambda t_: t_)
                n.tp_scale_rows(view(self.residual_out)[rows].data_ptr(), view(self.rinv)[rows].data_ptr(), self.gamma.data_ptr(),
                                view(self.out)[rows].data_ptr(), t, self.out_features, s)
        return self.out[rows], self.residual_out[rows]

    DECODE_MAX_TOKENS = 8

    def forward_decode(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, nvls: Optional[bool] = None, num_ctas: int = 0,
                       stream: Optional[torch.cuda.Stream] = None, emulated_inputs=None,
                       timeline: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """The layer for up to 8 tokens in ONE launch without tensor-core tiles: every SM streams the weight rows of its slab
        of output columns, the slabs are all-reduced with LL packets by the same thread blocks (no barrier between the
        ranks), residual add and RMSNorm follow in registers. Any world size, 1 included. k_shard must be a multiple of 256.
        nvls: packets leave through one multimem.st instead of one store per peer (default: where the heap has it and
        there are more than two ranks). timeline: optional zeroed int64 CUDA tensor [thread blocks, 8] that receives each
        block's time stamps in ns (entry, activations staged, weight pieces consumed, all warps done, allreduce + residual
        done, row-sum shares read, last store)."""
        from .._core import native

        n = native.load()
        t = x.shape[0]
        assert t <= self.DECODE_MAX_TOKENS and x.shape[1] == self.k_shard and x.is_contiguous() and self.k_shard % 256 == 0
        if residual is not None:
            self.residual_in[:t].copy_(residual)
        if nvls is None:
            nvls = bool(self.symm.nvls) and self.symm.world > 2
        s = (stream or torch.cuda.current_stream()).cuda_stream
        if emulated_inputs is not None:
            xp = [xi.data_ptr() for xi, _ in emulated_inputs]
            wp = [wi.data_ptr() for _, wi in emulated_inputs]
        else:
            xp, wp = [x.data_ptr()], [self.weight.data_ptr()]
        n.tp_decode(self.symm.heap, xp, wp, self.residual_in.data_ptr(), self.residual_out.data_ptr(), self.out.data_ptr(),
                    self.gamma.data_ptr(), t, self.out_features, self.k_shard, self.eps, nvls, num_ctas, s,
                    0 if timeline is None else timeline.data_ptr())
        return self.out[:t], self.residual_out[:t]

    def forward_local(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, two_sm: Optional[bool] = None,
                      stream: Optional[torch.cuda.Stream] = None, one_kernel: Optional[bool] = None, row_offset: int = 0,
                      probe: int = 0, timeline: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """World size 1 (no collective). one_kernel: ONE launch - the GEMM's epilogue adds the residual, stores h and
        accumulates every row's sum of squares, and extra warps normalise each 128-row block as soon as it is complete,
        while the MMAs of the later blocks run. one_kernel=False: the same epilogue, then a second, memory-bound launch
        that applies 1/rms and gamma. None picks by size: one launch up to 512 tokens (launch cost dominates there), two
        from there on (measured on B200: with the tensor pipe's operand traffic loading L2, the in-kernel normalisation
        of long sequences is slower than a separate pass at full memory bandwidth).
        timeline (one-kernel path, one-SM tiles): zeroed int64 CUDA tensor [148, 16] that receives per-CTA time stamps in ns
        (start, last MMA issued, MMA waits, epilogue waits and work, drain, first extra warp's rows / waits / work)."""
        from .._core import native

        assert self.symm.world == 1, "forward_local is the single-GPU path"
        n = native.load()
        t = x.shape[0]
        assert row_offset + t <= self.max_tokens and x.shape[1] == self.k_shard and x.is_contiguous()
        rows = slice(row_offset, row_offset + t)
        if residual is not None:
            self.residual_in[rows].copy_(residual)
        if two_sm is None:
            two_sm = t >= 1024 and self.out_features % 256 == 0
        if one_kernel is None:
            one_kernel = t <= 512
        s = (stream or torch.cuda.current_stream()).cuda_stream
        if one_kernel:
            ws_bytes = (n.tp_local_fused_workspace_bytes(self.max_tokens, self.out_features) + 255) // 256 * 256
            if self._local_ws is None:  # one workspace per 256-row-aligned launch that may be in flight: indexed by row offset
                self._local_ws = torch.empty((8, ws_bytes // 4), dtype=torch.float32, device=self.symm.device)
            ws = self._local_ws[(row_offset // 256) % 8]
            n.tp_local_fused(x.data_ptr(), self.weight.data_ptr(), self.residual_in[rows].data_ptr(), self.residual_out[rows].data_ptr(),
                             self.out[rows].data_ptr(), self.gamma.data_ptr(), ws.data_ptr(), t, self.out_features, self.k_shard,
                             self.eps, pick_block_n(t, self.out_features), two_sm, 0, s, probe, 0 if timeline is None else timeline.data_ptr())
            return self.out[rows], self.residual_out[rows]
        # the rows' sums of squares travel between the two launches in parts ([parts][t] floats, nothing to clear); launches
        # on disjoint row ranges use disjoint pieces of the buffer
        per_row = self.out_features // 64
        if self._sumsq_parts is None:
            self._sumsq_parts = torch.empty((self.max_tokens * per_row,), dtype=torch.float32, device=self.symm.device)
        parts_buf = self._sumsq_parts[row_offset * per_row:]
        parts = n.gemm_residual_sumsq(x.data_ptr(), self.weight.data_ptr(), self.residual_in[rows].data_ptr(), self.residual_out[rows].data_ptr(),
                                      parts_buf.data_ptr(), t, self.out_features, self.k_shard, pick_block_n(t, self.out_features), two_sm, s)
        n.tp_scale_rows_from_sumsq(self.residual_out[rows].data_ptr(), parts_buf.data_ptr(), parts, self.gamma.data_ptr(),
                                   self.out[rows].data_ptr(), t, self.out_features, self.eps, s)
        return self.out[rows], self.residual_out[rows]

    def forward_from_host(self, x_host: torch.Tensor, chunks: int = 4, **fused_kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
        """The layer on activations that are still in (pinned) host memory. The rows are cut into `chunks` pieces of whole
        256-row blocks; piece i+1 crosses PCIe on a copy stream while piece i is computed (one launch per piece, on the
        current stream, with the kernels writing straight into rows [r0, r1) of the layer's buffers). The residual
        stream is what self.residual_in already holds. Every rank must call it with the same shape and `chunks`.
        fused_kwargs go to forward_fused (world > 1). Returns (normalised output, new residual) for all rows."""
        t = x_host.shape[0]
        assert t <= self.max_tokens and x_host.shape[1] == self.k_shard and x_host.is_contiguous()
        dev = self.symm.device
        if getattr(self, "_x_stage", None) is None:
            self._x_stage = torch.empty((self.max_tokens, self.k_shard), dtype=torch.bfloat16, device=dev)
            self._h2d_stream = torch.cuda.Stream(device=dev)
            self._h2d_events = [torch.cuda.Event() for _ in range(64)]
        per = max(256, ((t + chunks - 1) // chunks + 255) // 256 * 256)
        bounds = [(r0, min(t, r0 + per)) for r0 in range(0, t, per)]
        cur = torch.cuda.current_stream()
        self._h2d_stream.wait_stream(cur)  # the staging rows are free once everything queued so far has read them
        with torch.cuda.stream(self._h2d_stream):
            for i, (r0, r1) in enumerate(bounds):
                self._x_stage[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                self._h2d_events[i].record(self._h2d_stream)
        for i, (r0, r1) in enumerate(bounds):
            cur.wait_event(self._h2d_events[i])
            x = self._x_stage[r0:r1]
            if self.symm.world == 1:
                self.forward_local(x, row_offset=r0)
            else:
                self.forward_fused(x, row_offset=r0, **fused_kwargs)
        return self.out[:t], self.residual_out[:t]

    @torch.no_grad()
    def reference(self, x_shards, weights, residual: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Plain PyTorch fp32 composition of the same layer (all shards given)."""
        acc = None
        for x, w in zip(x_shards, weights):
            p = (x.float() @ w.float().t()).to(torch.bfloat16).float()
            acc = p if acc is None else acc + p
        h = (acc.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
        y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps)
        return y.to(torch.bfloat16), h.to(torch.bfloat16)
