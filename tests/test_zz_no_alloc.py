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


def test_static_scratch_entry_point_two_calls_in_a_row():
    assert torch.cuda.is_available(), "needs a CUDA device"
    from tests import cabi
    from wush_int4_kernel_b200 import capi

    dev = torch.device("cuda:0")
    lib = capi.load()
    capi.check(lib.wush_init(), "wush_init")
    limit = lib.wush_w4a4_gemm_static_scratch_limit()
    assert limit == 32 << 20
    stream = torch.cuda.current_stream().cuda_stream

    # second shape is smaller than the first: stale bytes of call 1 stay in the array during call 2
    for seed, (M, N, K) in enumerate([(300, 520, 1024), (130, 264, 512)]):
        (xq, xs, wq, ws), y64 = _operands(M, N, K, 100 + seed, dev)
        expect = cabi.gemm(xq, xs, wq, ws, variant=capi.GEMM_TILE_F16)         # caller-provided scratch
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        capi.check(lib.wush_w4a4_gemm_static_scratch(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(),
                                                     M, N, K, y.data_ptr(), stream), "static scratch")
        torch.cuda.synchronize()
        flag = ctypes.c_int(-1)
        capi.check(lib.wush_device_flag(ctypes.byref(flag)), "device flag")
        assert flag.value == 0
        assert torch.equal(y, expect), "differs from the entry point with caller-provided scratch"
        rel = np.linalg.norm(y.double().cpu().numpy() - y64) / np.linalg.norm(y64)
        assert rel <= 1e-3, rel                                               # same bar as the other product tests

    # beyond the built-in array: refused with a clear message, nothing launched
    M, N, K = 4096, 8192, 4096
    z = torch.zeros(1, dtype=torch.uint8, device=dev)
    status = lib.wush_w4a4_gemm_static_scratch(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), M, N, K,
                                               z.data_ptr(), stream)
    assert status != capi.WUSH_OK
    msg = lib.wush_last_error().decode()
    assert "scratch" in msg and str(limit) in msg
