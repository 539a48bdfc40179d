"""Multi-process GPU checks, one rank per GPU (launched by torch.distributed.run from test_gpu_multi.py
or by hand). Exercises the real symmetric heap (VMM + fd passing + multicast) and every allreduce path
against an fp32 reference. Prints one JSON line per rank-0 check; exit code 0 = all good."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mscclpp_b200 import SymmetricMemory  # noqa: E402
from mscclpp_b200.ops import all_gather, all_reduce, all_reduce_rmsnorm, reduce_scatter  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    nvls = os.environ.get("MSCCLPP_TEST_NVLS", "1") == "1"
    symm = SymmetricMemory.from_env(nbytes=1 << 30, enable_nvls=nvls, timeout_ms=5000)
    failures = []

    def report(name, ok, **extra):
        if not ok:
            failures.append(name)
        if rank == 0:
            print(json.dumps({"check": name, "ok": bool(ok), **extra}), flush=True)

    def gathered_reference(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        return torch.stack([p.float() for p in parts]).sum(0)

    algos = ["packet", "allpair_packet", "packet128", "rsag_zero_copy"] + (["nvls_packet", "nvls_zero_copy"] if symm.nvls else [])
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for numel in (256, 4096, 65536, 1 << 20):
            inp = symm.tensor((numel,), dtype)
            out = symm.tensor((numel,), dtype)
            for algo in algos:
                if algo in ("packet", "nvls_packet", "allpair_packet") and numel * inp.element_size() > (1 << 20):
                    continue
                if algo == "packet128" and numel * inp.element_size() > (1 << 20):
                    continue
                for rep in range(2):
                    g = torch.Generator(device=dev).manual_seed(rank * 7 + numel + rep)
                    inp.copy_(torch.randn((numel,), generator=g, device=dev).to(dtype))
                    expect = gathered_reference(inp).to(dtype).float()
                    out.zero_()
                    torch.cuda.synchronize()
                    dist.barrier()
                    all_reduce(symm, inp, out, algo=algo)
                    torch.cuda.synchronize()
                    symm.check()
                    tol = {torch.bfloat16: 6e-2, torch.float16: 8e-3, torch.float32: 1e-4}[dtype]
                    err = (out.float() - expect).abs().max().item()
                    report(f"allreduce/{algo}/{dtype}/{numel}/{rep}", err <= tol * max(1.0, expect.abs().max().item()), err=err)
            symm.release(out)
            symm.release(inp)

    # ordinary tensors (outside the heap): the pipelined kernel, sizes with a tail and of many rounds
    for dtype in (torch.bfloat16, torch.float32):
        for numel in (70001, 1 << 20, (5 << 20) + 24):
            for algo in ["rsag_pipeline"] + (["nvls_block_pipeline"] if symm.nvls else []):
                for rep in range(2):
                    g = torch.Generator(device=dev).manual_seed(rank * 11 + numel + rep)
                    x = torch.randn((numel,), generator=g, device=dev).to(dtype)
                    y = torch.full_like(x, float("nan"))
                    expect = gathered_reference(x).to(dtype).float()
                    torch.cuda.synchronize()
                    dist.barrier()
                    all_reduce(symm, x, y, algo=algo)
                    torch.cuda.synchronize()
                    symm.check()
                    tol = {torch.bfloat16: 6e-2, torch.float32: 1e-4}[dtype]
                    err = (y.float() - expect).abs().max().item()
                    report(f"allreduce_outside_heap/{algo}/{dtype}/{numel}/{rep}", err <= tol * max(1.0, expect.abs().max().item()), err=err)
    # default choice for an ordinary tensor, in place
    x = torch.randn((3 << 20,), device=dev).to(torch.bfloat16)
    expect = gathered_reference(x).to(torch.bfloat16).float()
    dist.barrier()
    all_reduce(symm, x)
    torch.cuda.synchronize()
    symm.check()
    report("allreduce_outside_heap/default/in_place", (x.float() - expect).abs().max().item() <= 6e-2 * max(1.0, expect.abs().max().item()))

    # reduce-scatter / all-gather
    per = 8192
    full = symm.tensor((world * per,), torch.bfloat16)
    part = symm.tensor((per,), torch.bfloat16)
    for use_nvls in ([False, True] if symm.nvls else [False]):
        full.copy_(torch.randn((world * per,), device=dev).to(torch.bfloat16))
        expect = gathered_reference(full)[rank * per:(rank + 1) * per].to(torch.bfloat16).float()
        dist.barrier()
        reduce_scatter(symm, full, part, nvls=use_nvls)
        torch.cuda.synchronize()
        symm.check()
        report(f"reduce_scatter/nvls={use_nvls}", (part.float() - expect).abs().max().item() < 0.1)
        part.copy_(torch.full((per,), float(rank + 1), device=dev).to(torch.bfloat16))
        dist.barrier()
        all_gather(symm, part, full, nvls=use_nvls)
        torch.cuda.synchronize()
        symm.check()
        expect = torch.arange(1, world + 1, device=dev).repeat_interleave(per).float()
        report(f"all_gather/nvls={use_nvls}", torch.equal(full.float(), expect))

    # fused allreduce + residual + RMSNorm
    for rows, hidden in ((1, 8192), (8, 8192), (128, 8192), (512, 4096), (1000, 8192)):
        x = symm.tensor((rows, hidden), torch.bfloat16)
        y = symm.tensor((rows, hidden), torch.bfloat16)
        r_in = symm.tensor((rows, hidden), torch.bfloat16)
        r_out = symm.tensor((rows, hidden), torch.bfloat16)
        gamma = symm.tensor((hidden,), torch.bfloat16)
        gen = torch.Generator(device=dev).manual_seed(4242)
        r_in.copy_(torch.randn((rows, hidden), generator=gen, device=dev).to(torch.bfloat16))
        gamma.copy_((1 + 0.1 * torch.randn((hidden,), generator=gen, device=dev)).to(torch.bfloat16))
        x.copy_(torch.randn((rows, hidden), device=dev).to(torch.bfloat16))
        h = (gathered_reference(x).to(torch.bfloat16).float() + r_in.float()).to(torch.bfloat16).float()
        ref = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()).to(torch.bfloat16).float()
        cands = ["packet"] + (["nvls_packet"] if symm.nvls else [])
        if rows >= world:
            cands += ["rsag_zero_copy", "rows_p2p"] + (["nvls_zero_copy", "rows"] if symm.nvls else [])
        for algo in cands:
            if algo in ("packet", "nvls_packet") and rows * hidden * 2 > (1 << 20):
                continue
            y.zero_()
            r_out.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            all_reduce_rmsnorm(symm, x, y, r_in, r_out, gamma, eps=1e-5, algo=algo)
            torch.cuda.synchronize()
            symm.check()
            e1 = (y.float() - ref).abs().max().item()
            e2 = (r_out.float() - h).abs().max().item()
            report(f"allreduce_rmsnorm/{algo}/{rows}x{hidden}", e1 < 0.1 and e2 <= 0.02 * h.abs().max().item() + 0.05, err=e1, res_err=e2)
        for t in (gamma, r_out, r_in, y, x):
            symm.release(t)

    # one-kernel fused TP layer (GEMM + allreduce + residual + RMSNorm)
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    layer = RowParallelLinearNorm(symm, out_features=4096, k_shard=512, max_tokens=1024, seed=3)
    gen = torch.Generator(device=dev).manual_seed(777)
    layer.gamma.copy_((1 + 0.1 * torch.randn((4096,), generator=gen, device=dev)).to(torch.bfloat16))
    for tokens in (1, 8, 100, 1024):
        gen = torch.Generator(device=dev).manual_seed(1000 + tokens)
        residual = torch.randn((tokens, 4096), generator=gen, device=dev).to(torch.bfloat16)
        x = torch.randn((tokens, 512), device=dev).to(torch.bfloat16)
        part = (x.float() @ layer.weight.float().t()).to(torch.bfloat16)
        h = (gathered_reference(part).to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
        ref = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps) * layer.gamma.float()).to(torch.bfloat16).float()
        for use_nvls in ([False, True] if symm.nvls else [False]):
            for mode in (0, 1, 3):
                layer.out.zero_()
                layer.residual_out.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                for rep in range(2):
                    out, res = layer.forward_fused(x, residual, mode=mode, nvls=use_nvls)
                torch.cuda.synchronize()
                symm.check()
                e1 = (out.float() - ref).abs().max().item()
                e2 = (res.float() - h).abs().max().item()
                report(f"tp_fused/T={tokens}/nvls={use_nvls}/mode={mode}", e1 < 0.12 and e2 <= 0.02 * h.abs().max().item() + 0.05, err=e1, res_err=e2)

    # decode kernel: weight-streaming GEMV slabs + one-shot packet allreduce + residual + RMSNorm in one launch
    for tokens in (1, 3, 8):
        gen = torch.Generator(device=dev).manual_seed(2000 + tokens)
        residual = torch.randn((tokens, 4096), generator=gen, device=dev).to(torch.bfloat16)
        x = torch.randn((tokens, 512), device=dev).to(torch.bfloat16)
        part = (x.float() @ layer.weight.float().t()).to(torch.bfloat16)
        h = (gathered_reference(part).to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
        ref = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + layer.eps) * layer.gamma.float()).to(torch.bfloat16).float()
        for use_nvls in ([False, True] if symm.nvls else [False]):
            layer.out.zero_()
            layer.residual_out.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            for rep in range(3):
                out, res = layer.forward_decode(x, residual, nvls=use_nvls)
            torch.cuda.synchronize()
            symm.check()
            e1 = (out.float() - ref).abs().max().item()
            e2 = (res.float() - h).abs().max().item()
            report(f"tp_decode/T={tokens}/nvls={use_nvls}", e1 < 0.12 and e2 <= 0.02 * h.abs().max().item() + 0.05, err=e1, res_err=e2)

    # sequence-parallel halves: all-gather -> GEMM and GEMM -> reduce-scatter, one kernel each
    from mscclpp_b200.parallel.sp_layer import all_gather_gemm, gemm_reduce_scatter

    rows_per_rank, k, n_cols = 256, 1024, 1024
    s_rows = rows_per_rank * world
    a_local = symm.tensor((rows_per_rank, k), torch.bfloat16)
    a_full = symm.tensor((s_rows, k), torch.bfloat16)
    d = symm.tensor((s_rows, n_cols), torch.bfloat16)
    gen = torch.Generator(device=dev).manual_seed(4242 + rank)
    w = (torch.randn((n_cols, k), generator=gen, device=dev) * 0.05).to(torch.bfloat16)
    for rep in range(3):
        a_local.copy_(torch.randn((rows_per_rank, k), generator=gen, device=dev).to(torch.bfloat16))
        parts = [torch.empty_like(a_local) for _ in range(world)]
        dist.all_gather(parts, a_local)
        ref = torch.nn.functional.gelu(torch.cat(parts).float() @ w.float().t(), approximate="tanh")
        a_full.fill_(float("nan"))
        d.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        all_gather_gemm(symm, a_local, a_full, w, d, activation="gelu")
        torch.cuda.synchronize()
        symm.check()
        err = (d.float() - ref).abs().max().item()
        report(f"all_gather_gemm/{rep}", err <= 0.02 * ref.abs().max().item() + 0.02, err=err)
    partial = symm.tensor((s_rows, n_cols), torch.bfloat16)
    out_rs = symm.tensor((rows_per_rank, n_cols), torch.bfloat16)
    for use_nvls in ([False, True] if symm.nvls else [False]):
        for rep in range(2):
            x = torch.randn((s_rows, k), generator=gen, device=dev).to(torch.bfloat16)
            mine = (x.float() @ w.float().t()).to(torch.bfloat16)
            total = gathered_reference(mine)
            out_rs.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            gemm_reduce_scatter(symm, x, w, partial, out_rs, nvls=use_nvls)
            torch.cuda.synchronize()
            symm.check()
            ref = total[rank * rows_per_rank:(rank + 1) * rows_per_rank]
            err = (out_rs.float() - ref).abs().max().item()
            report(f"gemm_reduce_scatter/nvls={use_nvls}/{rep}", err <= 0.02 * ref.abs().max().item() + 0.05, err=err)

    # MoE expert-parallel dispatch / combine on real peers
    from mscclpp_b200.parallel.moe import ExpertParallelDispatcher, dequantize_rows

    experts, hid, toks, topk = 8 * world, 2048, 512, 2
    el = experts // world
    for fp8 in (False, True):
        disp = ExpertParallelDispatcher(symm, num_experts=experts, hidden=hid, max_tokens=toks, topk=topk, fp8=fp8)
        gen = torch.Generator(device=dev).manual_seed(31 + rank)
        for rep in range(2):
            xm = torch.randn((toks, hid), generator=gen, device=dev).to(torch.bfloat16)
            idx = torch.stack([torch.randperm(experts, generator=gen, device=dev)[:topk] for _ in range(toks)]).to(torch.int32)
            wt = torch.rand((toks, topk), generator=gen, device=dev)
            torch.cuda.synchronize()
            dist.barrier()
            recv_x, counts, slot_map = disp.dispatch(xm, idx)
            torch.cuda.synchronize()
            symm.check()
            cnt = counts.cpu().tolist()
            # what should have arrived: gather everybody's tokens and routing
            all_x = [torch.empty_like(xm) for _ in range(world)]
            all_idx = [torch.empty_like(idx) for _ in range(world)]
            dist.all_gather(all_x, xm)
            dist.all_gather(all_idx, idx)
            expect_cnt = [sum(int((all_idx[s] == rank * el + j).sum()) for s in range(world)) for j in range(el)]
            src = disp.recv_src[:cnt[el]].cpu().tolist()
            rows = recv_x[:cnt[el]]
            got = dequantize_rows(rows, disp.recv_scales[:cnt[el]]) if fp8 else rows.float()
            want = torch.stack([all_x[v >> 24][v & 0xFFFFFF].float() for v in src]) if src else got
            err = (got - want).abs().max().item() if src else 0.0
            report(f"moe_dispatch/fp8={fp8}/{rep}", cnt[:el] == expect_cnt and err <= (0.07 * want.abs().max().item() if fp8 else 0.0), err=err)
            start = 0
            for j in range(el):
                disp.expert_out[start:start + cnt[j]] = (got[start:start + cnt[j]] * (0.5 * (rank * el + j + 1))).to(torch.bfloat16)
                start += cnt[j]
            torch.cuda.synchronize()
            dist.barrier()
            y = disp.combine(idx, wt, slot_map)
            torch.cuda.synchronize()
            symm.check()
            ref = torch.zeros((toks, hid), device=dev)
            for k in range(topk):
                e = idx[:, k].long()
                ref += wt[:, k:k + 1] * (xm.float() * (0.5 * (e + 1)).unsqueeze(1)).to(torch.bfloat16).float()
            err = (y.float() - ref).abs().max().item()
            report(f"moe_combine/fp8={fp8}/{rep}", err <= (0.08 if fp8 else 0.02) * ref.abs().max().item() + 0.02, err=err)

    dist.barrier()
    symm.destroy()
    dist.destroy_process_group()
    if failures:
        print(f"rank {rank}: {len(failures)} failures: {failures[:5]}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
