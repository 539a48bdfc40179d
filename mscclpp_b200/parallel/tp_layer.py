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
        self.launches_per_forward = 2

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, algo: Optional[str] = None,
                stream: Optional[torch.cuda.Stream] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: [T, k_shard] bf16 (this rank's activation shard). residual: [T, out_features] or None to
        use what is already in self.residual_in. Returns (normalised output, new residual), both [T, out]."""
        t = x.shape[0]
        assert t <= self.max_tokens and x.shape[1] == self.k_shard
        partial = self.partial[:t]
        if residual is not None:
            self.residual_in[:t].copy_(residual)
        gemm_bf16(x, self.weight, partial, block_n=pick_block_n(t, self.out_features), stream=stream)
        out, res_out = self.out[:t], self.residual_out[:t]
        all_reduce_rmsnorm(self.symm, partial, out, self.residual_in[:t], res_out, self.gamma, eps=self.eps, algo=algo,
                           stream=stream)
        return out, res_out

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
