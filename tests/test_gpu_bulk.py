"""Bulk-copy (TMA, non-tensor) primitives in MoE-shaped patterns, compiled at run time with KernelBuilder."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_bulk_dispatch_combine_patterns(mode):
    from mscclpp_b200.utils import KernelBuilder, pack

    kernel = KernelBuilder("bulk_patterns.cu", "bulkPattern", file_dir=os.path.join(HERE, "kernels")).get_compiled_kernel()
    tokens, row = 96, 1024  # 4 KB rows
    g = torch.Generator(device="cuda").manual_seed(mode)
    src = torch.randn((tokens, row), generator=g, device="cuda")
    perm = torch.randperm(tokens, generator=g, device="cuda").to(torch.int32)
    dst = torch.ones((tokens, row), device="cuda") if mode == 2 else torch.zeros((tokens, row), device="cuda")
    failed = torch.zeros(1, dtype=torch.int32, device="cuda")
    # parameter block in the kernel's argument order: three pointers, two ints (8 bytes together), one pointer
    params = pack(src, dst, perm, row, mode, failed)
    kernel.launch_kernel(params, tokens, 32, shared=row * 4 + 128, stream=torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert int(failed.item()) == 0
    p = perm.long()
    if mode == 0:
        expect = torch.zeros_like(src)
        expect[p] = src
    elif mode == 1:
        expect = src[p]
    else:
        expect = torch.ones_like(src)
        expect[p] += src
    assert torch.equal(dst, expect)
