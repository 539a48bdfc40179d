"""tcgen05/TMEM bf16 GEMM against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,block_n", [
    (128, 256, 64, 256),
    (128, 256, 1024, 256),
    (256, 512, 128, 128),
    (1, 8192, 1024, 64),
    (8, 8192, 1024, 64),
    (200, 1024, 512, 128),
    (2048, 8192, 1024, 256),
    (777, 768, 320, 64),
    (4096, 4096, 512, 256),   # several bands of the L2-friendly tile order
    (2100, 2048, 192, 128),   # row tail inside the last band
])
def test_gemm_matches_fp32_reference(m, n, k, block_n):
    from mscclpp_b200.ops import gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_bf16(a, w, out, block_n=block_n)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_gemm_auto_tile_and_repeat():
    from mscclpp_b200.ops import gemm_bf16

    a = torch.randn((512, 1024), device="cuda").to(torch.bfloat16)
    w = (torch.randn((2048, 1024), device="cuda") * 0.02).to(torch.bfloat16)
    ref = (a.float() @ w.float().t())
    for _ in range(3):
        out = gemm_bf16(a, w)
        torch.cuda.synchronize()
        assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("m,n,k", [(512, 512, 256), (4096, 8192, 1024), (1000, 1024, 512)])
def test_gemm_two_sm_tiles(m, n, k):
    from mscclpp_b200.ops import gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_bf16(a, w, out, two_sm=True)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("one_kernel", [True, False])
@pytest.mark.parametrize("tokens,hidden,k,two_sm", [(200, 1024, 256, False), (1024, 2048, 512, True), (777, 512, 128, False),
                                                    (1, 8192, 1024, False), (2048, 8192, 1024, True), (1333, 2048, 256, True)])
def test_single_gpu_layer_gemm_epilogue_residual_sumsq(tokens, hidden, k, two_sm, one_kernel):
    """One GPU: GEMM whose epilogue adds the residual and accumulates the rows' sums of squares; the normalisation either
    in the same launch (rows handed to the epilogue warps block by block) or as a second, local pass."""
    import os

    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    symm = SymmetricMemory.emulated(1, nbytes=512 << 20, timeout_ms=3000)
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k, max_tokens=tokens)
    g = torch.Generator(device="cuda").manual_seed(tokens)
    x = torch.randn((tokens, k), generator=g, device="cuda").to(torch.bfloat16)
    residual = torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)
    layer.gamma.copy_((1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16))
    for rep in range(2):
        layer.out.fill_(float("nan"))
        out, res = layer.forward_local(x, residual, two_sm=two_sm, one_kernel=one_kernel)
        torch.cuda.synchronize()
    h = ((x.float() @ layer.weight.float().t()).to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
    y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps) * layer.gamma.float()).to(torch.bfloat16).float()
    assert (res.float() - h).abs().max().item() <= 0.02 * h.abs().max().item() + 0.05
    assert (out.float() - y).abs().max().item() <= 0.1
    symm.destroy()
