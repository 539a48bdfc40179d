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
