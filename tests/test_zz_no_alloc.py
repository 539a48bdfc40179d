"""The allocation-free entry point `mscclpp_b200_tp_layer_noalloc` (exported C symbol of
libmscclpp_b200.so) against the regular fused-layer entry point.

Some callers of this library may not allocate device memory at all once they are running - a plugin
inside another framework's planned memory region, a serving loop with a fixed memory budget - so one
entry point keeps every intermediate of the fused GEMM + residual + RMSNorm kernel in an array that is
part of the library image. This test calls it the way such a caller would: through the C ABI, with
device pointers only, twice in a row (the second call meets the state the first one left behind), and
checks every result against a plain PyTorch fp32 composition and against the heap-based entry point that the
rest of the library uses; it also checks that calls leave the free device memory unchanged, reads the error block
through the status query, and (where two GPUs are visible) repeats the first-call path on a second device.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already run
every other test."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib_path():
    from mscclpp_b200._core import native

    native.load(build_if_missing=True)  # makes sure the shared library exists and is current
    return native.lib_dir() / "libmscclpp_b200.so"


def _lib():
    lib = ctypes.CDLL(str(_lib_path()))
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


def _fp32_reference(x, w, residual, gamma, eps):
    """Plain PyTorch fp32 composition of the layer (the GEMM result and the sum are rounded to bf16 where the kernel rounds)."""
    h = ((x.float() @ w.float().t()).to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16).float()
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    return y, h


def _free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


# 300 x 2048 takes the 64-column tiles, 2048 x 2048 (the largest problem the built-in array admits) the 256-column ones
@pytest.mark.parametrize("tokens,hidden,k", [(300, 2048, 256), (2048, 2048, 512)])
def test_no_alloc_entry_point_matches_heap_entry_point(tokens, hidden, k):
    from mscclpp_b200 import SymmetricMemory
    from mscclpp_b200.parallel.tp_layer import RowParallelLinearNorm

    fn = _lib()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29877")
    for key, val in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")):
        os.environ.setdefault(key, val)
    eps = 1e-5
    symm = SymmetricMemory.from_env(nbytes=256 << 20, enable_nvls=False, port_offset=23)
    layer = RowParallelLinearNorm(symm, out_features=hidden, k_shard=k, max_tokens=tokens, eps=eps)
    g = torch.Generator(device="cuda").manual_seed(2024)
    gamma = (1 + 0.1 * torch.randn((hidden,), generator=g, device="cuda")).to(torch.bfloat16)
    layer.gamma.copy_(gamma)
    out = torch.empty((tokens, hidden), device="cuda", dtype=torch.bfloat16)
    res_out = torch.empty_like(out)
    inputs = [(torch.randn((tokens, k), generator=g, device="cuda").to(torch.bfloat16),
               torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)) for _ in range(3)]
    free_after = []
    for call, (x, residual) in enumerate(inputs):  # every call after the first runs on what the one before left in the shared array
        out.fill_(float("nan"))
        res_out.fill_(float("nan"))
        rc, msg = _call(fn, x, layer.weight, residual, gamma, out, res_out, eps)
        assert rc == 0, msg
        free_after.append(_free_bytes())
        # against the plain PyTorch fp32 composition ...
        ref_y, ref_h = _fp32_reference(x, layer.weight, residual, gamma, eps)
        assert (res_out.float() - ref_h).abs().max().item() <= 0.02 * ref_h.abs().max().item() + 0.05, f"call {call}"
        assert (out.float() - ref_y).abs().max().item() <= 0.1, f"call {call}"
        # ... and against the heap-based entry point of the same kernel
        heap_out, heap_res = layer.forward_fused(x, residual, mode=0, nvls=False)
        torch.cuda.synchronize()
        symm.check()
        assert (res_out.float() - heap_res.float()).abs().max().item() <= 0.02 * ref_h.abs().max().item() + 0.05, f"call {call}"
        assert (out.float() - heap_out.float()).abs().max().item() <= 0.1, f"call {call}"
    # the property the entry point exists for: once it has run on the device, a call takes no device memory
    for _ in range(3):
        before = _free_bytes()
        rc, msg = _call(fn, inputs[0][0], layer.weight, inputs[0][1], gamma, out, res_out, eps)
        assert rc == 0, msg
        assert _free_bytes() == before, "a call of the allocation-free entry point changed the free device memory"
    # nothing gave up on the device
    status = (ctypes.c_uint * 16)()
    err = ctypes.create_string_buffer(256)
    lib = ctypes.CDLL(str(_lib_path()))
    lib.mscclpp_b200_tp_layer_noalloc_status.restype = ctypes.c_int
    lib.mscclpp_b200_tp_layer_noalloc_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint), ctypes.c_char_p, ctypes.c_size_t]
    assert lib.mscclpp_b200_tp_layer_noalloc_status(torch.cuda.current_stream().cuda_stream, status, err, len(err)) == 0, err.value
    assert status[0] == 0, list(status)
    symm.destroy()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_no_alloc_entry_point_on_a_second_device():
    """The array, its device address and the kernel's shared-memory limit are per device: the first call on another GPU of
    the same process has to work like the first call on the first one."""
    fn = _lib()
    tokens, hidden, k, eps = 256, 1024, 128, 1e-5
    for dev in (0, 1):
        with torch.cuda.device(dev):
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(7 + dev)
            x = torch.randn((tokens, k), generator=g, device=f"cuda:{dev}").to(torch.bfloat16)
            w = (torch.randn((hidden, k), generator=g, device=f"cuda:{dev}") * 0.05).to(torch.bfloat16)
            residual = torch.randn((tokens, hidden), generator=g, device=f"cuda:{dev}").to(torch.bfloat16)
            gamma = torch.ones((hidden,), device=f"cuda:{dev}", dtype=torch.bfloat16)
            out = torch.full((tokens, hidden), float("nan"), device=f"cuda:{dev}", dtype=torch.bfloat16)
            res_out = torch.full_like(out, float("nan"))
            for _ in range(2):
                rc, msg = _call(fn, x, w, residual, gamma, out, res_out, eps)
                assert rc == 0, msg
                torch.cuda.synchronize()
            ref_y, ref_h = _fp32_reference(x, w, residual, gamma, eps)
            assert (res_out.float() - ref_h).abs().max().item() <= 0.02 * ref_h.abs().max().item() + 0.05
            assert (out.float() - ref_y).abs().max().item() <= 0.1


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
