"""Native collective kernels against a plain PyTorch fp32 reference.

All ranks are emulated on ONE GPU: the kernels run every rank inside one cooperative launch
(gridDim.y = world), which exercises exactly the device code that runs across GPUs, minus NVLS.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def _symm(world, nbytes=192 << 20):
    from mscclpp_b200 import SymmetricMemory

    return SymmetricMemory.emulated(world, nbytes=nbytes, timeout_ms=2000)


def _fill(symm, t, seed):
    """Per-rank N(0,1) data, returns the list of per-rank tensors (fp32 copies)."""
    ref = []
    for r in range(symm.world):
        g = torch.Generator(device="cuda").manual_seed(seed * 100 + r)
        x = torch.randn(t.shape, generator=g, device="cuda", dtype=torch.float32)
        view = symm.rank_view(t, r)
        if t.dtype in (torch.int32,):
            x = (x * 100).round()
        view.copy_(x.to(t.dtype))
        ref.append(view.to(torch.float32).clone())
    return ref


def _tol(dtype):
    return {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 1e-5}.get(dtype, 0)


@pytest.mark.parametrize("algo", ["packet", "allpair_packet", "packet128"])
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("numel", [8, 40, 1024, 33000, 262144])
def test_allreduce_ll(world, dtype, numel, algo):
    from mscclpp_b200.ops import all_reduce
    from mscclpp_b200.ops.collectives import ll128_max_bytes

    if algo == "packet128" and numel * torch.empty((), dtype=dtype).element_size() > ll128_max_bytes(world):
        pytest.skip("beyond the range the LL128 scratch is sized for at this world size")
    symm = _symm(world)
    inp = symm.tensor((numel,), dtype)
    out = symm.tensor((numel,), dtype)
    for launch in range(3):  # consecutive launches alternate the LL scratch buffer
        ref = _fill(symm, inp, seed=launch + 1)
        expect = torch.stack(ref).sum(0)
        all_reduce(symm, inp, out, algo=algo, n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        for r in range(world):
            got = symm.rank_view(out, r).to(torch.float32)
            torch.testing.assert_close(got, expect.to(dtype).to(torch.float32), atol=_tol(dtype) * 4, rtol=_tol(dtype))
    symm.destroy()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("numel", [4096, 262144 + 8, 3 << 20])
def test_allreduce_pipeline_buffers_outside_the_heap(world, dtype, numel):
    """Ordinary CUDA tensors (not heap memory): one kernel copies in, reduces through heap scratch and copies out.
    Row r of the [world, numel] tensors is emulated rank r's buffer; with 4 blocks the larger sizes take many rounds."""
    from mscclpp_b200.ops import all_reduce

    symm = _symm(world)
    for launch in range(2):
        g = torch.Generator(device="cuda").manual_seed(numel + launch)
        x = torch.randn((world, numel), generator=g, device="cuda").to(dtype)
        out = torch.full_like(x, float("nan"))
        assert not symm.contains(x)
        all_reduce(symm, x, out, algo="rsag_pipeline", n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        expect = x.float().sum(0).to(dtype).float()
        for r in range(world):
            torch.testing.assert_close(out[r].float(), expect, atol=_tol(dtype) * 4, rtol=_tol(dtype))
    symm.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_allreduce_ll_int_and_min(world):
    from mscclpp_b200.ops import all_reduce

    symm = _symm(world)
    inp = symm.tensor((5000,), torch.int32)
    out = symm.tensor((5000,), torch.int32)
    ref = _fill(symm, inp, seed=7)
    all_reduce(symm, inp, out, algo="packet", n_blocks=2)
    torch.cuda.synchronize()
    symm.check()
    assert torch.equal(symm.rank_view(out, world - 1).to(torch.float32), torch.stack(ref).sum(0))
    finp = symm.tensor((4096,), torch.bfloat16)
    fout = symm.tensor((4096,), torch.bfloat16)
    ref = _fill(symm, finp, seed=9)
    all_reduce(symm, finp, fout, op="min", algo="packet", n_blocks=2)
    torch.cuda.synchronize()
    symm.check()
    assert torch.equal(symm.rank_view(fout, 0).to(torch.float32), torch.stack(ref).min(0).values)
    symm.destroy()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("numel", [1024, 8 * 1000 * 8, 1 << 20])
def test_allreduce_two_shot(world, dtype, numel):
    from mscclpp_b200.ops import all_reduce

    symm = _symm(world)
    inp = symm.tensor((numel,), dtype)
    out = symm.tensor((numel,), dtype)
    for launch in range(2):
        ref = _fill(symm, inp, seed=launch + 11)
        expect = torch.stack(ref).sum(0)
        all_reduce(symm, inp, out, algo="rsag_zero_copy", n_blocks=8)
        torch.cuda.synchronize()
        symm.check()
        for r in range(world):
            got = symm.rank_view(out, r).to(torch.float32)
            torch.testing.assert_close(got, expect.to(dtype).to(torch.float32), atol=_tol(dtype) * 4, rtol=_tol(dtype))
    # in place
    ref = _fill(symm, inp, seed=99)
    all_reduce(symm, inp, None, algo="rsag_zero_copy", n_blocks=8)
    torch.cuda.synchronize()
    symm.check()
    expect = torch.stack(ref).sum(0).to(dtype).to(torch.float32)
    torch.testing.assert_close(symm.rank_view(inp, world - 1).to(torch.float32), expect, atol=_tol(dtype) * 4, rtol=_tol(dtype))
    symm.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_reduce_scatter_and_all_gather(world):
    from mscclpp_b200.ops import all_gather, reduce_scatter

    symm = _symm(world)
    per = 4096 * 3
    full = symm.tensor((world * per,), torch.bfloat16)
    part = symm.tensor((per,), torch.bfloat16)
    ref = _fill(symm, full, seed=21)
    reduce_scatter(symm, full, part, nvls=False, n_blocks=4)
    torch.cuda.synchronize()
    symm.check()
    total = torch.stack(ref).sum(0)
    for r in range(world):
        got = symm.rank_view(part, r).to(torch.float32)
        torch.testing.assert_close(got, total[r * per:(r + 1) * per].to(torch.bfloat16).to(torch.float32), atol=8e-2, rtol=2e-2)
    ref = _fill(symm, part, seed=23)
    all_gather(symm, part, full, nvls=False, n_blocks=4)
    torch.cuda.synchronize()
    symm.check()
    expect = torch.cat(ref)
    for r in range(world):
        assert torch.equal(symm.rank_view(full, r).to(torch.float32), expect)
    symm.destroy()


def _rmsnorm_ref(parts, residual, gamma, eps, dtype):
    h = torch.stack(parts).sum(0).to(dtype).to(torch.float32)
    if residual is not None:
        h = (h + residual).to(dtype).to(torch.float32)
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    if gamma is not None:
        y = y * gamma
    return y.to(dtype).to(torch.float32), h


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("algo", ["packet", "rsag_zero_copy"])
@pytest.mark.parametrize("rows,hidden", [(1, 8192), (8, 8192), (24, 1024), (64, 4096)])
def test_allreduce_residual_rmsnorm(world, algo, rows, hidden):
    from mscclpp_b200.ops import all_reduce_rmsnorm

    if algo == "rsag_zero_copy" and rows < world:
        pytest.skip("row-sliced two-shot needs at least one row per rank")
    dtype = torch.bfloat16
    symm = _symm(world)
    inp = symm.tensor((rows, hidden), dtype)
    out = symm.tensor((rows, hidden), dtype)
    res_in = symm.tensor((rows, hidden), dtype)
    res_out = symm.tensor((rows, hidden), dtype)
    gamma = symm.tensor((hidden,), dtype)
    parts = _fill(symm, inp, seed=31)
    g = torch.Generator(device="cuda").manual_seed(5)
    residual = torch.randn((rows, hidden), generator=g, device="cuda").to(dtype)
    gam = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(dtype)
    for r in range(world):
        symm.rank_view(res_in, r).copy_(residual)
        symm.rank_view(gamma, r).copy_(gam)
        symm.rank_view(out, r).zero_()
        symm.rank_view(res_out, r).zero_()
    all_reduce_rmsnorm(symm, inp, out, res_in, res_out, gamma, eps=1e-5, algo=algo, n_blocks=4)
    torch.cuda.synchronize()
    symm.check()
    y_ref, h_ref = _rmsnorm_ref(parts, residual.float(), gam.float(), 1e-5, dtype)
    for r in range(world):
        torch.testing.assert_close(symm.rank_view(res_out, r).float(), h_ref, atol=6e-2, rtol=2e-2)
        torch.testing.assert_close(symm.rank_view(out, r).float(), y_ref, atol=6e-2, rtol=2e-2)
    symm.destroy()


def test_bounded_wait_reports_timeout():
    """A rank that never shows up makes the others' waits expire with a status, not hang: here the
    'missing rank' is simulated by launching the LL kernel for world=2 data but with a heap whose
    second emulated rank sends to a different scratch epoch (we poison the epoch of rank 1)."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.ops import all_reduce

    symm = SymmetricMemory.emulated(2, nbytes=64 << 20, timeout_ms=50)
    inp = symm.tensor((1024,), torch.float32, zero=True)
    out = symm.tensor((1024,), torch.float32, zero=True)
    # desynchronise the launch epochs of the two emulated ranks: their packet flags will never match
    ctrl1 = symm.rank_view(symm_ctrl_epoch(symm), 1)
    ctrl1.fill_(1000)
    all_reduce(symm, inp, out, algo="packet", n_blocks=1)
    torch.cuda.synchronize()  # returns: the waits gave up after ~50 ms
    n = symm.heap.status()
    assert n.code != 0 and n.poisoned == 1
    with pytest.raises(Exception):
        symm.check()
    # the context is still usable afterwards
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    symm.destroy()


def symm_ctrl_epoch(symm):
    from mscclpp_b200 import tensor_from_pointer

    return tensor_from_pointer(symm.heap.local_base, (1,), torch.int32, symm.device, owner=symm)


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("tokens,hidden,k", [(1, 1024, 256), (5, 2048, 512), (8, 8192, 1024)])
def test_decode_layer_one_kernel(world, tokens, hidden, k):
    """Up to 8 tokens: weight-streaming slabs + one-shot packet allreduce + residual + RMSNorm in one launch, all ranks
    emulated on one GPU; three launches in a row alternate the packet scratch."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    symm = SymmetricMemory.emulated(world, nbytes=256 << 20, timeout_ms=3000)
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k, max_tokens=8)
    g = torch.Generator(device="cuda").manual_seed(tokens + hidden)
    ws = [(torch.randn((hidden, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    gam = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16)
    for r in range(world):
        symm.rank_view(layer.gamma, r).copy_(gam)
    ctas = max(1, 128 // world)
    for rep in range(3):
        xs = [torch.randn((tokens, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        residual = torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)
        for r in range(world):
            symm.rank_view(layer.residual_in, r)[:tokens].copy_(residual)
            symm.rank_view(layer.out, r).fill_(float("nan"))
            symm.rank_view(layer.residual_out, r).fill_(float("nan"))
        layer.forward_decode(xs[0], nvls=False, num_ctas=ctas, emulated_inputs=list(zip(xs, ws)))
        torch.cuda.synchronize()
        symm.check()
        acc = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws))
        h = (acc.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
        y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps) * gam.float()).to(torch.bfloat16).float()
        for r in range(world):
            got_h = symm.rank_view(layer.residual_out, r)[:tokens].float()
            got_y = symm.rank_view(layer.out, r)[:tokens].float()
            assert (got_h - h).abs().max().item() <= 0.02 * h.abs().max().item() + 0.05, f"rank {r} rep {rep}"
            assert (got_y - y).abs().max().item() <= 0.1, f"rank {r} rep {rep}"
    symm.destroy()


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("mode", [0, 1, 3])
@pytest.mark.parametrize("tokens,hidden,k", [(1, 1024, 128), (8, 2048, 256), (128, 8192, 256), (300, 1024, 512), (1024, 2048, 128)])
def test_fused_tp_layer_one_kernel(world, mode, tokens, hidden, k):
    """GEMM + allreduce + residual + RMSNorm in one launch, all ranks emulated on one GPU."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    symm = SymmetricMemory.emulated(world, nbytes=256 << 20, timeout_ms=3000)
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k, max_tokens=tokens)
    g = torch.Generator(device="cuda").manual_seed(tokens + hidden)
    xs = [torch.randn((tokens, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn((hidden, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    residual = torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)
    gam = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16)
    for r in range(world):
        symm.rank_view(layer.residual_in, r)[:tokens].copy_(residual)
        symm.rank_view(layer.gamma, r).copy_(gam)
        symm.rank_view(layer.out, r).zero_()
        symm.rank_view(layer.residual_out, r).zero_()
    for rep in range(2):
        layer.forward_fused(xs[0], mode=mode, nvls=False, num_reducers=4, num_gemm_ctas=max(1, 24 // world),
                            emulated_inputs=list(zip(xs, ws)))
        torch.cuda.synchronize()
        symm.check()
    acc = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws))
    h = (acc.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
    y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps) * gam.float()).to(torch.bfloat16).float()
    for r in range(world):
        got_h = symm.rank_view(layer.residual_out, r)[:tokens].float()
        got_y = symm.rank_view(layer.out, r)[:tokens].float()
        assert (got_h - h).abs().max().item() <= 0.02 * h.abs().max().item() + 0.05
        assert (got_y - y).abs().max().item() <= 0.1
    symm.destroy()


def test_fused_tp_layer_timeline_stamps():
    """The optional per-CTA time stamps of the fused kernel: ordered, and the reducer groups account for rows."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    world, tokens, hidden, k = 2, 512, 2048, 128
    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=3000)
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k, max_tokens=tokens)
    xs = [torch.randn((tokens, k), device="cuda").to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn((hidden, k), device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    gemm_ctas, reducers = 8, 4
    tl = torch.zeros((gemm_ctas + reducers, 16), dtype=torch.int64, device="cuda")
    layer.forward_fused(xs[0], mode=1, nvls=False, block_n=256, num_reducers=reducers, num_gemm_ctas=gemm_ctas,
                        emulated_inputs=list(zip(xs, ws)), timeline=tl)
    torch.cuda.synchronize()
    symm.check()
    t = tl.cpu()
    assert (t[:, 0] > 0).all()
    assert (t[:, 1] >= t[:, 0]).all() and (t[:, 2] >= t[:, 1]).all()
    assert int(t[:, 3].sum()) > 0  # first groups of the CTAs reduced rows
    assert (t[:, 8] + t[:, 9] + t[:, 10] <= t[:, 5]).all()  # the phases are parts of the time spent on rows
    assert (t[:gemm_ctas, 1] > t[:gemm_ctas, 0]).all()  # GEMM CTAs spent time in the matmul
    symm.destroy()


@pytest.mark.parametrize("world,rows_per_rank,k,n_cols,act", [(2, 256, 256, 256, "none"), (4, 128, 512, 512, "gelu"), (8, 128, 256, 256, "silu")])
def test_all_gather_gemm_one_kernel(world, rows_per_rank, k, n_cols, act):
    """All-gather -> GEMM in one launch (copier CTAs + gated tcgen05 GEMM), all ranks emulated on one GPU."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.sp_layer import all_gather_gemm

    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=3000)
    s_rows = world * rows_per_rank
    a_local = symm.tensor((rows_per_rank, k), torch.bfloat16)
    a_full = symm.tensor((s_rows, k), torch.bfloat16)
    out = symm.tensor((s_rows, n_cols), torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(world * 100 + k)
    ws = [(torch.randn((n_cols, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    for rep in range(2):
        shards = [torch.randn((rows_per_rank, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        for r in range(world):
            symm.rank_view(a_local, r).copy_(shards[r])
            symm.rank_view(a_full, r).fill_(float("nan"))  # own rows are never copied there: must not be read
            symm.rank_view(out, r).zero_()
        all_gather_gemm(symm, a_local, a_full, ws, out, activation=act, block_n=256 if n_cols % 256 == 0 else 128, num_copiers=2,
                        num_gemm_ctas=max(1, 16 // world))
        torch.cuda.synchronize()
        symm.check()
        full = torch.cat(shards).float()
        for r in range(world):
            ref = full @ ws[r].float().t()
            if act == "gelu":
                ref = torch.nn.functional.gelu(ref, approximate="tanh")
            elif act == "silu":
                ref = torch.nn.functional.silu(ref)
            got = symm.rank_view(out, r).float()
            assert (got - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.02, (r, rep)
    symm.destroy()


@pytest.mark.parametrize("world,rows_per_rank,k,ffn,block_n", [(2, 256, 256, 256, 256), (4, 128, 512, 128, 128), (2, 256, 128, 384, -1)])
def test_all_gather_gemm_swiglu(world, rows_per_rank, k, ffn, block_n):
    """All-gather -> GEMM over interleaved gate / up weights with the gated epilogue: out = silu(x Wg^T) * (x Wu^T), one
    launch, all ranks emulated on one GPU; against the fp32 composition."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.sp_layer import all_gather_gemm, interleave_gate_up

    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=3000)
    s_rows = world * rows_per_rank
    a_local = symm.tensor((rows_per_rank, k), torch.bfloat16)
    a_full = symm.tensor((s_rows, k), torch.bfloat16)
    out = symm.tensor((s_rows, ffn), torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(world * 31 + ffn)
    wg = [(torch.randn((ffn, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    wu = [(torch.randn((ffn, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    ws = [interleave_gate_up(a, b) for a, b in zip(wg, wu)]
    for rep in range(2):
        shards = [torch.randn((rows_per_rank, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        for r in range(world):
            symm.rank_view(a_local, r).copy_(shards[r])
            symm.rank_view(a_full, r).fill_(float("nan"))
            symm.rank_view(out, r).fill_(float("nan"))
        all_gather_gemm(symm, a_local, a_full, ws, out, activation="swiglu", block_n=block_n, num_copiers=2, num_gemm_ctas=max(2, 16 // world))
        torch.cuda.synchronize()
        symm.check()
        full = torch.cat(shards).float()
        for r in range(world):
            ref = torch.nn.functional.silu(full @ wg[r].float().t()) * (full @ wu[r].float().t())
            got = symm.rank_view(out, r).float()
            assert (got - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.02, (r, rep)
    symm.destroy()


@pytest.mark.parametrize("world,rows_per_rank,k,n_cols", [(2, 256, 128, 512), (4, 128, 256, 1024), (8, 128, 64, 256)])
def test_gemm_reduce_scatter_one_kernel(world, rows_per_rank, k, n_cols):
    """GEMM -> reduce-scatter in one launch: rank r ends with its row block of the summed product."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.sp_layer import gemm_reduce_scatter

    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=3000)
    s_rows = world * rows_per_rank
    partial = symm.tensor((s_rows, n_cols), torch.bfloat16)
    out = symm.tensor((rows_per_rank, n_cols), torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(world * 10 + k)
    for rep in range(2):
        xs = [torch.randn((s_rows, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        ws = [(torch.randn((n_cols, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
        for r in range(world):
            symm.rank_view(out, r).zero_()
        gemm_reduce_scatter(symm, xs, ws, partial, out, nvls=False, block_n=256 if n_cols % 256 == 0 else 128, num_reducers=3,
                            num_gemm_ctas=max(1, 16 // world))
        torch.cuda.synchronize()
        symm.check()
        total = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws))
        for r in range(world):
            ref = total[r * rows_per_rank:(r + 1) * rows_per_rank]
            got = symm.rank_view(out, r).float()
            assert (got - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.05, (r, rep)
    symm.destroy()


def _moe_reference(xs, idxs, wts, world, experts, f):
    """fp32 PyTorch model of dispatch -> expert function f(e, rows) -> combine, for all ranks."""
    ys = []
    for r in range(world):
        y = torch.zeros_like(xs[r], dtype=torch.float32)
        for k in range(idxs[r].shape[1]):
            e = idxs[r][:, k]
            valid = e >= 0
            contrib = torch.zeros_like(y)
            for ex in range(experts):
                m = valid & (e == ex)
                if m.any():
                    contrib[m] = f(ex, xs[r][m].float())
            y += wts[r][:, k:k + 1] * contrib
        ys.append(y)
    return ys


@pytest.mark.parametrize("world,experts,tokens,hidden,topk,fp8", [(2, 8, 200, 512, 2, False), (4, 16, 96, 1024, 2, True), (8, 64, 64, 4096, 2, False),
                                                                  (8, 64, 33, 1024, 4, True)])
def test_moe_dispatch_combine(world, experts, tokens, hidden, topk, fp8):
    """Dispatch pushes every (token, expert) pair into the hosting rank's expert-grouped buffer; combine pulls the expert
    outputs back. All ranks emulated on one GPU; checked against a plain PyTorch model of the same exchange."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.moe import ExpertParallelDispatcher, dequantize_rows

    symm = SymmetricMemory.emulated(world, nbytes=256 << 20, timeout_ms=3000)
    disp = ExpertParallelDispatcher(symm, num_experts=experts, hidden=hidden, max_tokens=tokens, topk=topk, fp8=fp8)
    el = experts // world
    g = torch.Generator(device="cuda").manual_seed(world * 1000 + tokens)
    for rep in range(2):
        xs = [torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        idxs = [torch.stack([torch.randperm(experts, generator=g, device="cuda")[:topk] for _ in range(tokens)]).to(torch.int32) for _ in range(world)]
        idxs[0][0, 0] = -1  # an unused slot
        wts = [torch.rand((tokens, topk), generator=g, device="cuda") for _ in range(world)]
        for r in range(world):
            x_s, idx_s, w_s = disp.stage(r, xs[r], idxs[r], wts[r])
        recv_x, counts, slot_map = disp.dispatch(x_s, idx_s, n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        # every destination holds exactly the rows routed to it, grouped by expert, tagged with their source
        for d in range(world):
            cnt = symm.rank_view(counts, d).cpu().tolist()
            expect_cnt = [sum(int((idxs[s] == d * el + j).sum()) for s in range(world)) for j in range(el)]
            assert cnt[:el] == expect_cnt and cnt[el] == sum(expect_cnt)
            rows = symm.rank_view(recv_x, d)[:cnt[el]]
            src = symm.rank_view(disp.recv_src, d)[:cnt[el]].cpu()
            got = dequantize_rows(rows, symm.rank_view(disp.recv_scales, d)[:cnt[el]]) if fp8 else rows.float()
            want = torch.stack([xs[int(v) >> 24][int(v) & 0xFFFFFF].float() for v in src.tolist()]) if cnt[el] else got
            tol = 0.07 * want.abs().max().item() if fp8 else 0.0
            assert (got - want).abs().max().item() <= tol
            # the expert of a row follows from its position
            bounds = [0]
            for c_ in expect_cnt:
                bounds.append(bounds[-1] + c_)
            for j in range(el):
                for v in src[bounds[j]:bounds[j + 1]].tolist():
                    s_, t_ = int(v) >> 24, int(v) & 0xFFFFFF
                    assert (idxs[s_][t_] == d * el + j).any()
        # experts: out = (e + 1) * 0.5 * row  (cheap, expert dependent)
        for d in range(world):
            cnt = symm.rank_view(counts, d).cpu().tolist()
            rows = symm.rank_view(recv_x, d)
            val = dequantize_rows(rows[:cnt[el]], symm.rank_view(disp.recv_scales, d)[:cnt[el]]) if fp8 else rows[:cnt[el]].float()
            out = symm.rank_view(disp.expert_out, d)
            start = 0
            for j in range(el):
                out[start:start + cnt[j]] = (val[start:start + cnt[j]] * (0.5 * (d * el + j + 1))).to(torch.bfloat16)
                start += cnt[j]
        y = disp.combine(idx_s, w_s, slot_map, n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        ref = _moe_reference(xs, idxs, wts, world, experts, lambda e, rows: (rows * (0.5 * (e + 1))).to(torch.bfloat16).float())
        for r in range(world):
            got = symm.rank_view(y, r).float()
            scale = ref[r].abs().max().item()
            assert (got - ref[r]).abs().max().item() <= (0.08 if fp8 else 0.02) * scale + 0.02, (r, rep)
    symm.destroy()


@pytest.mark.parametrize("world,experts,tokens,hidden,topk", [(2, 8, 120, 512, 2), (8, 64, 48, 4096, 2), (4, 16, 64, 1024, 4)])
def test_moe_combine_fp8_payload(world, experts, tokens, hidden, topk):
    """Combine with e4m3 expert outputs (1 x 128 scales): the stand-alone quantiser against a PyTorch model of it, then the
    combined rows against the fp32 weighted sum of the bf16 expert outputs (tolerance of the e4m3 rounding)."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.moe import ExpertParallelDispatcher, dequantize_rows

    symm = SymmetricMemory.emulated(world, nbytes=256 << 20, timeout_ms=3000)
    disp = ExpertParallelDispatcher(symm, num_experts=experts, hidden=hidden, max_tokens=tokens, topk=topk, fp8_combine=True)
    el = experts // world
    g = torch.Generator(device="cuda").manual_seed(world * 77 + tokens)
    for rep in range(2):
        xs = [torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
        idxs = [torch.stack([torch.randperm(experts, generator=g, device="cuda")[:topk] for _ in range(tokens)]).to(torch.int32) for _ in range(world)]
        wts = [torch.rand((tokens, topk), generator=g, device="cuda") for _ in range(world)]
        for r in range(world):
            x_s, idx_s, w_s = disp.stage(r, xs[r], idxs[r], wts[r])
        recv_x, counts, slot_map = disp.dispatch(x_s, idx_s, n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        for d in range(world):
            cnt = symm.rank_view(counts, d).cpu().tolist()
            rows = symm.rank_view(recv_x, d)
            out = symm.rank_view(disp.expert_out, d)
            start = 0
            for j in range(el):
                out[start:start + cnt[j]] = (rows[start:start + cnt[j]].float() * (0.5 * (d * el + j + 1))).to(torch.bfloat16)
                start += cnt[j]
            disp.quantize_expert_out(cnt[el], rank=d)
            torch.cuda.synchronize()
            # the quantiser: scale = amax / 448 per 128 elements, values within one e4m3 step of the input
            val = out[:cnt[el]].float()
            scales = symm.rank_view(disp.expert_out_scales, d)[:cnt[el]]
            want_scale = val.view(cnt[el], -1, 128).abs().amax(-1) / 448.0
            want_scale = torch.where(want_scale > 0, want_scale, torch.ones_like(want_scale))
            assert torch.allclose(scales, want_scale, rtol=1e-5, atol=0)
            back = dequantize_rows(symm.rank_view(disp.expert_out_q, d)[:cnt[el]], scales)
            assert (back - val).abs().max().item() <= 0.07 * val.abs().max().item()
        y = disp.combine(idx_s, w_s, slot_map, n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        ref = _moe_reference(xs, idxs, wts, world, experts, lambda e, rows: (rows * (0.5 * (e + 1))).to(torch.bfloat16).float())
        for r in range(world):
            got = symm.rank_view(y, r).float()
            assert (got - ref[r]).abs().max().item() <= 0.08 * ref[r].abs().max().item() + 0.02, (r, rep)
    symm.destroy()


def test_moe_dispatch_reports_small_receive_buffer():
    """A receive buffer that cannot hold the routed rows is reported as an error; nothing is written out of bounds."""
    from mscclpp_b200 import SymmetricMemory, native
    from mscclpp_b200.parallel.moe import ExpertParallelDispatcher

    symm = SymmetricMemory.emulated(2, nbytes=64 << 20, timeout_ms=1000)
    disp = ExpertParallelDispatcher(symm, num_experts=4, hidden=256, max_tokens=64, topk=2, capacity=16)
    x = torch.ones((64, 256), dtype=torch.bfloat16, device="cuda")
    idx = torch.tensor([[0, 1]] * 64, dtype=torch.int32, device="cuda")  # everything goes to rank 0
    for r in range(2):
        x_s, idx_s, _ = disp.stage(r, x, idx)
    disp.dispatch(x_s, idx_s, n_blocks=2)
    torch.cuda.synchronize()
    with pytest.raises(native().Error):
        symm.check()
    assert int(symm.rank_view(disp.slot_map, 0).max()) == -1
    symm.heap.reset_status()
    symm.destroy()


@pytest.mark.parametrize("world,rows_per_rank", [(2, 256), (4, 512)])
def test_two_sm_core_in_fused_kernels(world, rows_per_rank):
    """The fused kernels on the two-SM GEMM core (256 x 256 tiles on CTA pairs, clusters of two): all-gather -> GEMM,
    GEMM -> reduce-scatter and the fused TP layer, all ranks emulated on one GPU."""
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.sp_layer import all_gather_gemm, gemm_reduce_scatter
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    symm = SymmetricMemory.emulated(world, nbytes=256 << 20, timeout_ms=3000)
    s_rows, k, n_cols = world * rows_per_rank, 256, 512
    g = torch.Generator(device="cuda").manual_seed(world + rows_per_rank)
    ctas = max(2, (24 // world) & ~1)
    # all-gather -> GEMM
    a_local = symm.tensor((rows_per_rank, k), torch.bfloat16)
    a_full = symm.tensor((s_rows, k), torch.bfloat16)
    out = symm.tensor((s_rows, n_cols), torch.bfloat16)
    ws = [(torch.randn((n_cols, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    shards = [torch.randn((rows_per_rank, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    for rep in range(2):
        for r in range(world):
            symm.rank_view(a_local, r).copy_(shards[r])
            symm.rank_view(out, r).zero_()
        all_gather_gemm(symm, a_local, a_full, ws, out, block_n=0, num_copiers=2, num_gemm_ctas=ctas)
        torch.cuda.synchronize()
        symm.check()
    full = torch.cat(shards).float()
    for r in range(world):
        ref = full @ ws[r].float().t()
        assert (symm.rank_view(out, r).float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.02
    # GEMM -> reduce-scatter
    partial = symm.tensor((s_rows, n_cols), torch.bfloat16)
    out_rs = symm.tensor((rows_per_rank, n_cols), torch.bfloat16)
    xs = [torch.randn((s_rows, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    for rep in range(2):
        gemm_reduce_scatter(symm, xs, ws, partial, out_rs, nvls=False, block_n=0, num_reducers=2, num_gemm_ctas=ctas)
        torch.cuda.synchronize()
        symm.check()
    total = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws))
    for r in range(world):
        ref = total[r * rows_per_rank:(r + 1) * rows_per_rank]
        assert (symm.rank_view(out_rs, r).float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.05
    # fused TP layer (GEMM + allreduce + residual + RMSNorm)
    tokens = 512
    layer = RowParallelLinearNorm(symm, out_features=n_cols, k_shard=k, max_tokens=tokens)
    xt = [torch.randn((tokens, k), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    residual = torch.randn((tokens, n_cols), generator=g, device="cuda").to(torch.bfloat16)
    for r in range(world):
        symm.rank_view(layer.residual_in, r)[:tokens].copy_(residual)
        symm.rank_view(layer.gamma, r).fill_(1.0)
    for mode in (0, 1):
        for rep in range(2):
            layer.forward_fused(xt[0], mode=mode, nvls=False, block_n=-1, num_reducers=2, num_gemm_ctas=ctas, emulated_inputs=list(zip(xt, ws)))
            torch.cuda.synchronize()
            symm.check()
        acc = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xt, ws))
        h = (acc.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
        y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps)).to(torch.bfloat16).float()
        for r in range(world):
            assert (symm.rank_view(layer.residual_out, r)[:tokens].float() - h).abs().max().item() <= 0.02 * h.abs().max().item() + 0.05
            assert (symm.rank_view(layer.out, r)[:tokens].float() - y).abs().max().item() <= 0.1
    symm.destroy()


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (777, 512, 256), (2048, 1024, 512)])
def test_two_sm_gemm(m, n, k):
    from mscclpp_b200.ops.gemm import gemm_bf16

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    d = gemm_bf16(a, w, two_sm=True)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    assert (d.float() - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 0.01


@pytest.mark.parametrize("world,rows,hidden,with_residual", [(2, 100, 1024, True), (4, 64, 8192, True), (8, 333, 4096, False)])
def test_row_owner_allreduce_rmsnorm(world, rows, hidden, with_residual):
    """Standalone allreduce + residual + RMSNorm on the fused kernel's reducer (row owners, whole rows in registers)."""
    from mscclpp_b200 import SymmetricMemory, native

    n = native()
    symm = SymmetricMemory.emulated(world, nbytes=128 << 20, timeout_ms=3000)
    partial = symm.tensor((rows, hidden), torch.bfloat16)
    res_in = symm.tensor((rows, hidden), torch.bfloat16)
    res_out = symm.tensor((rows, hidden), torch.bfloat16)
    out = symm.tensor((rows, hidden), torch.bfloat16)
    gamma = symm.tensor((hidden,), torch.bfloat16)
    rinv = symm.tensor((rows,), torch.float32)
    g = torch.Generator(device="cuda").manual_seed(rows)
    parts = [torch.randn((rows, hidden), generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    residual = torch.randn((rows, hidden), generator=g, device="cuda").to(torch.bfloat16)
    gam = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16)
    for r in range(world):
        symm.rank_view(partial, r).copy_(parts[r])
        symm.rank_view(res_in, r).copy_(residual)
        symm.rank_view(gamma, r).copy_(gam)
    mode = 1 if with_residual else 0
    for rep in range(2):
        for r in range(world):
            symm.rank_view(out, r).zero_()
        n.tp_reduce_norm(symm.heap, partial.data_ptr(), res_in.data_ptr() if with_residual else 0, res_out.data_ptr() if with_residual else 0,
                         out.data_ptr(), gamma.data_ptr(), rinv.data_ptr(), rows, hidden, 1e-5, 4, 0, mode, False,
                         torch.cuda.current_stream().cuda_stream)
        if mode == 1:
            for r in range(world):
                n.tp_scale_rows(symm.rank_view(res_out, r).data_ptr(), symm.rank_view(rinv, r).data_ptr(), gamma.data_ptr(),
                                symm.rank_view(out, r).data_ptr(), rows, hidden, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        symm.check()
    acc = sum(p.float() for p in parts).to(torch.bfloat16).float()
    h = (acc + residual.float()).to(torch.bfloat16).float() if with_residual else acc
    y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float()).to(torch.bfloat16).float()
    for r in range(world):
        assert (symm.rank_view(out, r).float() - y).abs().max().item() <= 0.1
        if with_residual:
            assert (symm.rank_view(res_out, r).float() - h).abs().max().item() <= 0.02 * h.abs().max().item() + 0.05
    symm.destroy()


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("algo", ["packet", "rsag_zero_copy"])
def test_fp8_allreduce_accumulates_in_fp32(world, dtype, algo):
    """FP8 inputs are summed in fp32 and rounded once: the result equals round(fp32 sum) and its error is never
    larger than that of summing in fp8 step by step (the property the reference checks in test_fp8_accum.py)."""
    from mscclpp_b200.ops import all_reduce

    symm = _symm(world)
    numel = 16384
    inp = symm.tensor((numel,), dtype)
    out = symm.tensor((numel,), dtype)
    vals = []
    for r in range(world):
        g = torch.Generator(device="cuda").manual_seed(900 + r)
        x = (torch.randn(numel, generator=g, device="cuda") * 0.5).to(dtype)
        symm.rank_view(inp, r).copy_(x)
        vals.append(x.float())
    all_reduce(symm, inp, out, algo=algo, n_blocks=4)
    torch.cuda.synchronize()
    symm.check()
    exact = torch.stack(vals).sum(0)
    oracle = exact.to(dtype).float()          # one rounding of the fp32 sum
    stepwise = vals[0].clone()
    for v in vals[1:]:
        stepwise = (stepwise + v).to(dtype).float()   # what accumulating in fp8 would give
    for r in range(world):
        got = symm.rank_view(out, r).float()
        assert torch.equal(got, oracle), (r, (got - oracle).abs().max().item())
    assert (oracle - exact).abs().mean().item() <= (stepwise - exact).abs().mean().item() + 1e-9
    symm.destroy()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_broadcast_and_all_to_all(world):
    """Native broadcast (root streams into every rank) and all-to-all (peer stores), all ranks emulated on one GPU."""
    from mscclpp_b200.ops import all_to_all, broadcast

    symm = _symm(world)
    per = 4096
    src = symm.tensor((world * per,), torch.float32)
    dst = symm.tensor((world * per,), torch.float32)
    for r in range(world):
        symm.rank_view(src, r).copy_(torch.arange(world * per, device="cuda", dtype=torch.float32) + 100000 * r)
    for root in (0, world - 1):
        for r in range(world):
            symm.rank_view(dst, r).zero_()
        broadcast(symm, src, dst, root=root, nvls=False, n_blocks=4)
        torch.cuda.synchronize()
        symm.check()
        want = symm.rank_view(src, root)
        for r in range(world):
            assert torch.equal(symm.rank_view(dst, r), want)
    for r in range(world):
        symm.rank_view(dst, r).zero_()
    all_to_all(symm, src, dst, n_blocks=4)
    torch.cuda.synchronize()
    symm.check()
    for r in range(world):
        want = torch.cat([symm.rank_view(src, p)[r * per:(r + 1) * per] for p in range(world)])
        assert torch.equal(symm.rank_view(dst, r), want)
    symm.destroy()
