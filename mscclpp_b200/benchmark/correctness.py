"""Correctness statistics for a collective's output against an fp32 reference
(reference: python/mscclpp_benchmark/correctness.py:247-264 reports the same kind of summary)."""
from __future__ import annotations

import torch

TOLERANCE = {torch.bfloat16: 2 ** -6, torch.float16: 2 ** -9, torch.float32: 1e-5}


def error_stats(got: torch.Tensor, ref_fp32: torch.Tensor) -> dict:
    diff = (got.float() - ref_fp32).abs()
    scale = max(ref_fp32.abs().max().item(), 1e-30)
    return {"max_abs": diff.max().item(), "mean_abs": diff.mean().item(), "max_rel_to_peak": diff.max().item() / scale,
            "mismatch_frac": (diff > TOLERANCE.get(got.dtype, 1e-5) * scale * 4).float().mean().item()}


def passes(got: torch.Tensor, ref_fp32: torch.Tensor, n_ranks: int) -> bool:
    """Sums of n values rounded to the storage type: allow a few ulps of the peak, growing with sqrt(n)."""
    st = error_stats(got, ref_fp32)
    return st["max_rel_to_peak"] <= TOLERANCE.get(got.dtype, 1e-5) * 4 * max(1.0, n_ranks ** 0.5)
