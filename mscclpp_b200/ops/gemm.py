"""bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), hand-written for sm_100a."""
from __future__ import annotations

from typing import Optional

import torch

from .._core import native


def pick_block_n(m: int, n: int) -> int:
    """Wider N tiles amortise the A tile; narrow ones spread a skinny problem over more SMs."""
    tiles_m = (m + 127) // 128
    for bn in (256, 128, 64):
        if n % bn == 0 and tiles_m * (n // bn) >= 120:
            return bn
    for bn in (64, 128, 256):
        if n % bn == 0:
            return bn
    raise ValueError("N must be a multiple of 64")


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, block_n: int = 0, num_ctas: int = 0,
              stream: Optional[torch.cuda.Stream] = None, two_sm: Optional[bool] = None, probe: int = 0, band: int = 0) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T  (w in nn.Linear layout: out_features x in_features).

    two_sm: run 256 x 256 tiles on pairs of SMs (tcgen05 cta_group::2); None picks it when the problem has enough
    such tiles to fill the GPU and no N tile was asked for.
    band: row blocks per band of the tile order (0 = default for the tile shape, -1 = plain column-major walk).
    probe: diagnostics only (the result is then garbage): bit 0 drops the operand loads, bit 1 the MMAs, bit 2 the
    epilogue's stores; timing each shows which of the kernel's three pipelines bounds a shape."""
    n = native.load()
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    m, k = a.shape
    nn, k2 = w.shape
    assert k == k2 and k % 64 == 0
    if out is None:
        out = torch.empty((m, nn), dtype=torch.bfloat16, device=a.device)
    assert out.is_contiguous() and out.shape == (m, nn)
    s = (stream or torch.cuda.current_stream()).cuda_stream
    if two_sm is None:
        two_sm = block_n == 0 and nn % 256 == 0 and ((m + 255) // 256) * (nn // 256) >= 74
    if two_sm:
        n.gemm_bf16_two_sm(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, nn, k, nn, num_ctas, 0, s, probe, band)
        return out
    bn = block_n or pick_block_n(m, nn)
    n.gemm_bf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, nn, k, nn, bn, num_ctas, 0, s, probe, band)
    return out
