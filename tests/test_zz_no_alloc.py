"""The allocation-free entry point `mscclpp_b200_tp_layer_noalloc` (exported C symbol of
libmscclpp_b200.so) against the regular fused-layer entry point.

Some callers of this library may not allocate device memory at all once they are running - a plugin
inside another framework's planned memory region, a serving loop with a fixed memory budget - so one
entry point keeps every intermediate of the fused GEMM + residual + RMSNorm kernel in an array that is
part of the library image. This test calls it the way such a caller would: through the C ABI, with
device pointers only, twice in a row (the second call meets the state the first one left behind), and
checks both results against the heap-based entry point that the rest of the library uses.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already run
every other test."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mscclpp_b200._core import native

    native.load(build_if_missing=True)  # makes sure the shared library exists and is current
    lib = ctypes.CDLL(str(native.lib_dir() / "libmscclpp_b200.so"))
    fn = lib.mscclpp_b200_tp_layer_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _call(fn, x, w, residual, gamma, out, res_out, eps):
    err = ctypes.create_string_buffer(256)
    m, k = x.shape
    n = w.shape[0]
    rc = fn(x.data_ptr(), w.data_ptr(), residual.data_ptr() if residual is not None else None,
            gamma.data_ptr() if gamma is not None else None, out.data_ptr(), res_out.data_ptr(), m, n, k, eps,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    return rc, err.value.decode()


def test_no_alloc_entry_point_matches_heap_entry_point():
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    fn = _lib()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29877")
    for key, val in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")):
        os.environ.setdefault(key, val)
    tokens, hidden, k, eps = 300, 2048, 256, 1e-5
    symm = SymmetricMemory.from_env(nbytes=128 << 20, enable_nvls=False, port_offset=23)
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k, max_tokens=tokens, eps=eps)
    g = torch.Generator(device="cuda").manual_seed(2024)
    gamma = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16)
    layer.gamma.copy_(gamma)
    out = torch.empty((tokens, hidden), device="cuda", dtype=torch.bfloat16)
    res_out = torch.empty_like(out)
    for call in range(2):  # the second call runs on whatever the first one left in the shared scratch
        x = torch.randn((tokens, k), generator=g, device="cuda").to(torch.bfloat16)
        residual = torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)
        ref_out, ref_res = layer.forward_fused(x, residual, mode=0, nvls=False)
        ref_out, ref_res = ref_out.float().clone(), ref_res.float().clone()
        out.fill_(float("nan"))
        res_out.fill_(float("nan"))
        rc, msg = _call(fn, x, layer.weight, residual, gamma, out, res_out, eps)
        assert rc == 0, msg
        torch.cuda.synchronize()
        symm.check()
        assert (res_out.float() - ref_res).abs().max().item() <= 0.02 * ref_res.abs().max().item() + 0.05, f"call {call}"
        assert (out.float() - ref_out).abs().max().item() <= 0.1, f"call {call}"
    symm.destroy()


def test_no_alloc_entry_point_rejects_oversized_problems():
    fn = _lib()
    x = torch.zeros((8, 64), device="cuda", dtype=torch.bfloat16)
    w = torch.zeros((64, 64), device="cuda", dtype=torch.bfloat16)
    out = torch.zeros((8, 64), device="cuda", dtype=torch.bfloat16)
    err = ctypes.create_string_buffer(256)
    # 1024 x 8192 = 8 Mi elements: twice the built-in scratch
    rc = fn(x.data_ptr(), w.data_ptr(), None, None, out.data_ptr(), out.data_ptr(), 1024, 8192, 64, 1e-5, None, err, len(err))
    assert rc != 0 and b"MSCCLPP_B200_NOALLOC_MAX_ELEMS" in err.value
    rc = fn(x.data_ptr(), w.data_ptr(), None, None, out.data_ptr(), out.data_ptr(), 8, 100, 64, 1e-5, None, err, len(err))
    assert rc != 0 and b"multiple of 64" in err.value
