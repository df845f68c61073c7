"""The product entry point that brings its own scratch (wush_w4a4_gemm_static_scratch).

It serves hosts that cannot give the library scratch memory and are not allowed to allocate on
the device while running (fixed arenas, fixed memory budgets, loops that cannot take the
implicit synchronisation of an allocation).  Its scratch is one array inside the library, shared
by all calls and never cleared between them, so the check is made on two calls in a row with
different operands: each must equal the regular entry point with caller-provided scratch.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed, dev):
    from oracle import w4a4_oracle as orc

    g = torch.Generator().manual_seed(seed)
    X = torch.randn(M, K, generator=g).to(torch.bfloat16)
    W = (0.05 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    xq, xs = orc.quant_int4(orc.bits(X))
    wq, ws = orc.quant_int4(orc.bits(W))
    to = lambda a, dt=None: (torch.from_numpy(a).to(dev) if dt is None else orc.from_bits(a, dt).to(dev))
    return (to(xq), to(xs, torch.bfloat16), to(wq), to(ws, torch.bfloat16)), orc.gemm_f64(xq, xs, wq, ws)


def test_static_scratch_entry_point_two_calls_in_a_row(monkeypatch):
    assert torch.cuda.is_available(), "needs a CUDA device"
    # with room behind its scratch the caller-scratch entry point cuts tiles into K ranges; the built-in array has
    # no such room, so for the bit-for-bit comparison below the cut is switched off
    monkeypatch.setenv("WUSH_TAIL_SPLIT", "0")
    from tests import cabi
    from wush_int4_kernel_b200 import capi

    dev = torch.device("cuda:0")
    lib = capi.load()
    capi.check(lib.wush_init(), "wush_init")
    limit = lib.wush_w4a4_gemm_static_scratch_limit()
    assert limit == 32 << 20
    stream = torch.cuda.current_stream().cuda_stream

    flag = ctypes.c_int(-1)
    capi.check(lib.wush_device_flag(ctypes.byref(flag)), "device flag")           # clears what earlier tests left

    # Each shape is smaller than the one before: stale bytes of the previous call stay in the array.
    #   (300, 520, 1024)  weights widened inside the GEMM, 256-row tiles
    #   (130, 264, 320)   K % 256 != 0: the route with an fp16 copy of the weights in the array
    #   (130, 264, 512)   weights widened inside the GEMM again
    # Without K ranges in the caller-scratch call the two must agree bit for bit.
    for seed, (M, N, K) in enumerate([(300, 520, 1024), (130, 264, 320), (130, 264, 512)]):
        (xq, xs, wq, ws), y64 = _operands(M, N, K, 100 + seed, dev)
        expect = cabi.gemm(xq, xs, wq, ws, variant=capi.GEMM_TILE_F16)         # caller-provided scratch
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        capi.check(lib.wush_w4a4_gemm_static_scratch(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(),
                                                     M, N, K, y.data_ptr(), stream), "static scratch")
        torch.cuda.synchronize()
        # bits 8-15: the word the kernels of THIS entry point set when a bounded wait gives up
        capi.check(lib.wush_device_flag(ctypes.byref(flag)), "device flag")
        assert flag.value == 0, f"a bounded wait gave up (flag {flag.value:#x})"
        assert torch.equal(y, expect), "differs from the entry point with caller-provided scratch"
        rel = np.linalg.norm(y.double().cpu().numpy() - y64) / np.linalg.norm(y64)
        assert rel <= 1e-3, rel                                               # same bar as the other product tests

    # A narrow layer: with caller scratch K is split over several work units (fp32 partial results in
    # the scratch); the built-in array has no room reserved for them, so this entry point runs the
    # unsplit kernel.  Same arithmetic, different summation order: compared with the fp64 result.
    M, N, K = 256, 512, 4096
    assert lib.wush_w4a4_gemm_workspace_bytes(M, N, K, capi.GEMM_TILE_F16) > 256 + 2 * M * K + 4 * M + 8 * N + 1024
    (xq, xs, wq, ws), y64 = _operands(M, N, K, 200, dev)
    y = torch.empty(M, N, dtype=torch.float16, device=dev)
    capi.check(lib.wush_w4a4_gemm_static_scratch(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(),
                                                 M, N, K, y.data_ptr(), stream), "static scratch")
    torch.cuda.synchronize()
    capi.check(lib.wush_device_flag(ctypes.byref(flag)), "device flag")
    assert flag.value == 0
    rel = np.linalg.norm(y.double().cpu().numpy() - y64) / np.linalg.norm(y64)
    assert rel <= 1e-3, rel

    # Weight scales that are not 16-byte aligned take the route with an fp16 copy of the weights.  Where
    # that copy fits the array the result is still right; where it does not, the call is refused before
    # any launch instead of writing past the array.
    M, N, K = 130, 264, 512
    (xq, xs, wq, ws), y64 = _operands(M, N, K, 300, dev)
    ws_odd = torch.empty(ws.numel() + 1, dtype=torch.bfloat16, device=dev)[1:].view_as(ws)
    ws_odd.copy_(ws)
    assert ws_odd.data_ptr() % 16 == 2
    y = torch.empty(M, N, dtype=torch.float16, device=dev)
    capi.check(lib.wush_w4a4_gemm_static_scratch(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws_odd.data_ptr(),
                                                 M, N, K, y.data_ptr(), stream), "static scratch, odd scales")
    torch.cuda.synchronize()
    rel = np.linalg.norm(y.double().cpu().numpy() - y64) / np.linalg.norm(y64)
    assert rel <= 1e-3, rel
    M, N, K = 128, 8192, 4096                       # 1 MiB of activations fits, 64 MiB of fp16 weights does not
    big = torch.zeros(N * K // 32 + 1, dtype=torch.bfloat16, device=dev)
    z = torch.zeros(max(M, N) * K // 2, dtype=torch.uint8, device=dev)
    y = torch.empty(M, N, dtype=torch.float16, device=dev)
    assert lib.wush_w4a4_gemm_static_scratch(z.data_ptr(), big.data_ptr(), z.data_ptr(), big.data_ptr(), M, N, K,
                                             y.data_ptr(), stream) == capi.WUSH_OK                # aligned: fits
    status = lib.wush_w4a4_gemm_static_scratch(z.data_ptr(), big.data_ptr(), z.data_ptr(), big[1:].data_ptr(), M, N, K,
                                               y.data_ptr(), stream)
    assert status == capi.WUSH_ERR_WORKSPACE, lib.wush_last_error().decode()
    torch.cuda.synchronize()

    # beyond the built-in array: refused with a clear message, nothing launched
    M, N, K = 4096, 8192, 4096
    z = torch.zeros(1, dtype=torch.uint8, device=dev)
    status = lib.wush_w4a4_gemm_static_scratch(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), M, N, K,
                                               z.data_ptr(), stream)
    assert status != capi.WUSH_OK
    msg = lib.wush_last_error().decode()
    assert "scratch" in msg and str(limit) in msg
