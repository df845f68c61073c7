"""Test helper: calls the C ABI (``libwush_int4_b200.so``) directly through ctypes with torch
device tensors, the way a foreign-language binding would.  Allocation happens here, in the
test, never inside the library."""
from __future__ import annotations

import torch

from wush_int4_kernel_b200 import capi


def _stream():
    return torch.cuda.current_stream().cuda_stream


def quant_int4(x: torch.Tensor):
    lib = capi.load()
    K = x.shape[-1]
    q = torch.empty(*x.shape[:-1], K // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(*x.shape[:-1], K // 32, dtype=torch.bfloat16, device=x.device)
    capi.check(lib.wush_quant_int4(x.data_ptr(), x.numel() // 32, q.data_ptr(), s.data_ptr(), _stream()), "quant_int4")
    return q, s


def fused_tq(x: torch.Tensor, t: torch.Tensor, variant: int):
    lib = capi.load()
    K = x.shape[-1]
    rows = x.numel() // K
    q = torch.empty(*x.shape[:-1], K // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(*x.shape[:-1], K // 32, dtype=torch.bfloat16, device=x.device)
    capi.check(lib.wush_fused_transform_quant_int4(x.data_ptr(), t.data_ptr(), rows, K, variant, q.data_ptr(),
                                                   s.data_ptr(), _stream()), "fused_tq")
    return q, s


def gemm(xq, xs, wq, ws, variant: int = capi.GEMM_AUTO, misalign: int = 0):
    """`misalign` (a multiple of 16): output and scratch start that many bytes past a 256-byte boundary."""
    lib = capi.load()
    K = wq.shape[1] * 2
    M, N = xq.numel() // (K // 2), wq.shape[0]
    y = torch.empty(M * N + misalign // 2, dtype=torch.float16, device=xq.device)[misalign // 2:].view(M, N)
    nbytes = lib.wush_w4a4_gemm_workspace_bytes(M, N, K, variant)
    work = torch.empty(max(nbytes, 1) + misalign, dtype=torch.uint8, device=xq.device)[misalign:]
    assert y.data_ptr() % 256 == misalign % 256 and work.data_ptr() % 256 == misalign % 256
    capi.check(lib.wush_w4a4_gemm(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K, y.data_ptr(),
                                  variant, work.data_ptr() if nbytes else None, nbytes, _stream()), "w4a4_gemm")
    if nbytes >= 4:                       # the tile kernel reports bounded-wait timeouts in word 0 of its scratch
        torch.cuda.synchronize()
        flag = int(work[:4].view(torch.int32).item())
        assert flag == 0, f"tile GEMM aborted: a bounded wait gave up (role code {flag})"
    return y


def group_partials(xq, wq):
    lib = capi.load()
    K = wq.shape[1] * 2
    M, N = xq.numel() // (K // 2), wq.shape[0]
    P = torch.empty(M, N, K // 32, dtype=torch.int32, device=xq.device)
    capi.check(lib.wush_group_partials(xq.data_ptr(), wq.data_ptr(), M, N, K, P.data_ptr(), _stream()), "group_partials")
    return P


def atom(a, b):
    lib = capi.load()
    c = torch.zeros(8, 8, dtype=torch.int32, device=a.device)
    capi.check(lib.wush_i8_atom_selftest(a.data_ptr(), b.data_ptr(), c.data_ptr(), _stream()), "atom")
    return c


def quant_ts(x, inv_scale: float, inv_dev=None):
    lib = capi.load()
    q = torch.empty(x.numel() // 2, dtype=torch.uint8, device=x.device)
    capi.check(lib.wush_quant_int4_tensor_scale(x.data_ptr(), x.numel(), inv_scale,
                                                inv_dev.data_ptr() if inv_dev is not None else None, q.data_ptr(),
                                                _stream()), "quant_ts")
    return q


def gemm_ts(xq, wq, alpha: float, alpha_dev=None):
    lib = capi.load()
    K = wq.shape[1] * 2
    M, N = xq.numel() // (K // 2), wq.shape[0]
    y = torch.empty(M, N, dtype=torch.float16, device=xq.device)
    capi.check(lib.wush_w4a4_gemm_tensor_scale(xq.data_ptr(), wq.data_ptr(), M, N, K, alpha,
                                               alpha_dev.data_ptr() if alpha_dev is not None else None, y.data_ptr(),
                                               _stream()), "gemm_ts")
    return y


def gemm_ts_ws(xq, wq, alpha: float, alpha_dev=None):
    """Per-tensor product with caller scratch; returns (y, scratch bytes used, error word)."""
    lib = capi.load()
    K = wq.shape[1] * 2
    M, N = xq.numel() // (K // 2), wq.shape[0]
    y = torch.empty(M, N, dtype=torch.float16, device=xq.device)
    nbytes = lib.wush_w4a4_gemm_tensor_scale_workspace_bytes(M, N, K)
    work = torch.full((max(nbytes, 4),), 0x55, dtype=torch.uint8, device=xq.device)
    capi.check(lib.wush_w4a4_gemm_tensor_scale_ws(xq.data_ptr(), wq.data_ptr(), M, N, K, alpha,
                                                  alpha_dev.data_ptr() if alpha_dev is not None else None, y.data_ptr(),
                                                  work.data_ptr() if nbytes else None, nbytes, _stream()), "gemm_ts_ws")
    flag = int(work[:4].view(torch.int32).item()) if nbytes else 0
    return y, nbytes, flag


def tile_selftest(a, b, layout_mode: int = 0):
    lib = capi.load()
    n = b.shape[0]
    d = torch.zeros(128, n, dtype=torch.int32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    capi.check(lib.wush_i8_tile_selftest(a.data_ptr(), b.data_ptr(), d.data_ptr(), n, layout_mode, status.data_ptr(),
                                         _stream()), "tile_selftest")
    return d, int(status.item())


class _RawDeviceMemory:
    """Wraps a raw device pointer so that torch can view it (CUDA array interface, version 2)."""

    def __init__(self, ptr: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 2}


def device_view(ptr: int, count: int, dtype: torch.dtype) -> torch.Tensor:
    """A tensor over `count` elements of device memory at `ptr` (no copy): for tests that look into the
    exchange buffers of a communicator."""
    typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.uint8: "|u1", torch.int32: "<i4"}[dtype]
    return torch.as_tensor(_RawDeviceMemory(ptr, count, typestr), device="cuda")
