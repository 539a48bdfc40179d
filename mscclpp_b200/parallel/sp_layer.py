"""Sequence-parallel MLP halves with the collective fused into the GEMM.

    up:    H[S, F/tp]  = act( all_gather(X_r)[S, H] @ W1_r[F/tp, H]^T )       all-gather -> GEMM, one kernel
    down:  Y_r[S/tp,H] = reduce_scatter( H[S, F/tp] @ W2_r[H, F/tp]^T )       GEMM -> reduce-scatter, one kernel

S = sequence (tokens of all ranks), H = hidden, F = ffn. Rank r holds rows [r*S/tp, (r+1)*S/tp) of the
sequence-sharded activations. The reference library supplies the all-gather and the reduce-scatter of this
pattern as separate collectives; here the transfers run inside the tcgen05 GEMM kernels and overlap the MMAs
block by block.
"""
from __future__ import annotations

from typing import Optional

import torch

from .._core import native
from .._core.symm import SymmetricMemory

ACTIVATIONS = {"none": 0, "gelu": 1, "silu": 2, "swiglu": 3}


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[F, K] gate and up projection weights -> the [2 F, K] matrix the "swiglu" epilogue expects: rows in groups of 64,
    the first 32 of a group gate features 32 b .. 32 b + 31, the other 32 the matching up features (F % 32 == 0). With
    it one all-gather -> GEMM launch produces silu(x W_gate^T) * (x W_up^T) directly, [S, F]."""
    f, k = w_gate.shape
    assert w_up.shape == (f, k) and f % 32 == 0
    return torch.stack([w_gate.view(f // 32, 32, k), w_up.view(f // 32, 32, k)], dim=1).reshape(2 * f, k).contiguous()


def all_gather_gemm(symm: SymmetricMemory, a_local: torch.Tensor, a_full: torch.Tensor, weight, out: torch.Tensor,
                    activation: str = "none", block_n: int = -1, num_copiers: int = 0, num_gemm_ctas: int = 0,
                    stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """out[S, N] = act(concat_r(a_local_r) @ weight^T). `a_local` [S/tp, K], `a_full` [S, K] workspace and `out` are
    symmetric-heap tensors; `weight` [N, K] is local (a list with one weight per rank for emulated heaps).
    activation "swiglu": `weight` is interleave_gate_up(w_gate, w_up) and `out` is [S, N / 2] = silu(gate) * up."""
    n = native.load()
    s_rows, k = a_full.shape
    weights = weight if isinstance(weight, (list, tuple)) else [weight]
    n_cols = weights[0].shape[0]
    assert a_local.shape == (s_rows // symm.world, k) and out.shape == (s_rows, n_cols // 2 if activation == "swiglu" else n_cols)
    if block_n < 0:  # 0 = two-SM tiles (256 x 256 on SM pairs) when the shape allows, else one-SM 256- or 128-wide tiles
        block_n = 0 if (s_rows % (symm.world * 256) == 0 and n_cols % 256 == 0) else (256 if n_cols % 256 == 0 else 128)
    assert all(w.shape == (n_cols, k) and w.is_contiguous() and w.dtype == torch.bfloat16 for w in weights)
    st = (stream or torch.cuda.current_stream()).cuda_stream
    n.all_gather_gemm(symm.heap, a_local.data_ptr(), a_full.data_ptr(), [w.data_ptr() for w in weights], out.data_ptr(), s_rows, n_cols, k,
                      block_n, num_gemm_ctas, num_copiers, ACTIVATIONS[activation], st)
    return out


def gemm_reduce_scatter(symm: SymmetricMemory, a, weight, partial: torch.Tensor, out: torch.Tensor, nvls: Optional[bool] = None,
                        block_n: int = -1, num_reducers: int = 0, num_gemm_ctas: int = 0,
                        stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """out_r[S/tp, N] = rows of sum_r(a_r @ weight_r^T) that rank r owns. `partial` [S, N] and `out` [S/tp, N] are
    symmetric-heap tensors; `a` [S, K] and `weight` [N, K] are local (lists with one entry per rank for emulated heaps)."""
    n = native.load()
    a_list = a if isinstance(a, (list, tuple)) else [a]
    w_list = weight if isinstance(weight, (list, tuple)) else [weight]
    s_rows, k = a_list[0].shape
    n_cols = w_list[0].shape[0]
    assert partial.shape == (s_rows, n_cols) and out.shape == (s_rows // symm.world, n_cols)
    if block_n < 0:
        block_n = 0 if (s_rows % (symm.world * 256) == 0 and n_cols % 256 == 0) else (256 if n_cols % 256 == 0 else 128)
    nvls = symm.nvls if nvls is None else nvls
    st = (stream or torch.cuda.current_stream()).cuda_stream
    n.tp_fused(symm.heap, [x.data_ptr() for x in a_list], [w.data_ptr() for w in w_list], partial.data_ptr(), 0, 0, out.data_ptr(), 0, 0,
               s_rows, n_cols, k, 0.0, block_n, num_gemm_ctas, num_reducers, 0, 2, nvls, st)
    return out


class SequenceParallelMLP:
    """MLP of one tensor-parallel rank on sequence-sharded activations (random-initialised weights): two matrices, or
    three with activation="swiglu" (gate and up projections interleaved into one [2 F/tp, hidden] matrix, so that the
    all-gather -> GEMM launch produces silu(gate) * up directly)."""

    def __init__(self, symm: SymmetricMemory, hidden: int = 8192, ffn: int = 28672, seq: int = 8192, activation: str = "gelu",
                 seed: int = 0, init_std: float = 0.02):
        tp = symm.world
        assert ffn % tp == 0 and seq % (tp * 128) == 0
        self.symm, self.hidden, self.ffn_shard, self.seq, self.activation = symm, hidden, ffn // tp, seq, activation
        dev = symm.device
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + symm.rank)
        if activation == "swiglu":
            self.w_gate = (torch.randn((self.ffn_shard, hidden), generator=g, device=dev) * init_std).to(torch.bfloat16)
            self.w_up = (torch.randn((self.ffn_shard, hidden), generator=g, device=dev) * init_std).to(torch.bfloat16)
            self.w1 = interleave_gate_up(self.w_gate, self.w_up)
        else:
            self.w1 = (torch.randn((self.ffn_shard, hidden), generator=g, device=dev) * init_std).to(torch.bfloat16)
        self.w2 = (torch.randn((hidden, self.ffn_shard), generator=g, device=dev) * init_std).to(torch.bfloat16)
        self.x_local = symm.tensor((seq // tp, hidden), torch.bfloat16)
        self.x_full = symm.tensor((seq, hidden), torch.bfloat16)
        self.h = symm.tensor((seq, self.ffn_shard), torch.bfloat16)
        self.partial = symm.tensor((seq, hidden), torch.bfloat16)
        self.y_local = symm.tensor((seq // tp, hidden), torch.bfloat16)
        self.launches_per_forward = 2

    def forward(self, x_local: Optional[torch.Tensor] = None, num_copiers: int = 0, num_reducers: int = 0,
                stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        if x_local is not None:
            self.x_local.copy_(x_local)
        all_gather_gemm(self.symm, self.x_local, self.x_full, self.w1, self.h, activation=self.activation, num_copiers=num_copiers,
                        stream=stream)
        gemm_reduce_scatter(self.symm, self.h, self.w2, self.partial, self.y_local, num_reducers=num_reducers, stream=stream)
        return self.y_local
