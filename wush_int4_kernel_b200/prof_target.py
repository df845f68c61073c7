"""Minimal profiling target (the role of the reference's ``bench/prof_target.py``): runs one
operator a few times on synthetic operands so that ``ncu -k regex:<kernel> -c <n>`` has a
small, self-contained process to capture.

    python -m wush_int4_kernel_b200.prof_target gemm  M N K [reps]
    python -m wush_int4_kernel_b200.prof_target gemm_ts M N K [reps]     (per-tensor scale)
    python -m wush_int4_kernel_b200.prof_target gemm_v VARIANT M N K [reps]   (C ABI, variant gemv|decode|decode_tc|tile|tile_f16)
    python -m wush_int4_kernel_b200.prof_target fused M K   [reps]
    python -m wush_int4_kernel_b200.prof_target quant M K   [reps]

Prints the mean time per call measured with CUDA events (never quote a time taken under a
profiler).
"""
from __future__ import annotations

import sys

import torch

from . import _C, timing


def _codes(rows, K, gen, dev):
    q = torch.randint(0, 256, (rows, K // 2), generator=gen, device=dev, dtype=torch.uint8)
    s = (0.01 * (1 + 0.5 * torch.rand(rows, K // 32, generator=gen, device=dev))).to(torch.bfloat16)
    return q, s


def main(argv):
    op = argv[0]
    dev = torch.device("cuda:0")
    _C.init()
    gen = torch.Generator(device=dev).manual_seed(0)
    if op == "gemm":
        M, N, K = map(int, argv[1:4])
        reps = int(argv[4]) if len(argv) > 4 else 5
        xq, xs = _codes(M, K, gen, dev)
        wq, ws = _codes(N, K, gen, dev)
        if M == 1:
            fn = lambda: _C.w4a4_gemv(xq, xs, wq, ws)
        elif M <= 32:
            fn = lambda: _C.w4a4_gemv_multi(xq, xs, wq, ws)
        else:
            fn = lambda: _C.w4a4_gemm_s4(xq, xs, wq, ws)
        work = 2.0 * M * N * K
    elif op == "gemm_v":
        from . import capi
        variant = {"gemv": capi.GEMM_GEMV, "decode": capi.GEMM_DECODE, "tile": capi.GEMM_TILE, "tile_f16": capi.GEMM_TILE_F16,
                   "decode_tc": capi.GEMM_DECODE_TC, "gemv_mma": capi.GEMM_GEMV_MMA}[argv[1]]
        M, N, K = map(int, argv[2:5])
        reps = int(argv[5]) if len(argv) > 5 else 5
        xq, xs = _codes(M, K, gen, dev)
        wq, ws = _codes(N, K, gen, dev)
        lib = capi.load()
        nbytes = lib.wush_w4a4_gemm_workspace_bytes(M, N, K, variant)
        work_buf = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=dev)
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        stream = torch.cuda.current_stream().cuda_stream

        def fn():
            capi.check(lib.wush_w4a4_gemm(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K, y.data_ptr(),
                                          variant, work_buf.data_ptr() if nbytes else None, nbytes, stream), "w4a4_gemm")
        work = 2.0 * M * N * K
    elif op == "gemm_ts":
        M, N, K = map(int, argv[1:4])
        reps = int(argv[4]) if len(argv) > 4 else 5
        xq, _ = _codes(M, K, gen, dev)
        wq, _ = _codes(N, K, gen, dev)
        fn = lambda: _C.w4a4_gemm_cutlass(xq, wq, 1e-3)
        work = 2.0 * M * N * K
    elif op in ("fused", "quant"):
        M, K = map(int, argv[1:3])
        reps = int(argv[3]) if len(argv) > 3 else 5
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        t = (torch.randn(K // 32, 32, 32, generator=gen, device=dev) / 6).to(torch.bfloat16)
        fn = (lambda: _C.fused_transform_quant_int4_v3(x, t)) if op == "fused" else (lambda: _C.quant_int4(x))
        work = 0.0
    else:
        raise SystemExit(__doc__)
    for _ in range(3):
        fn()
    ms = timing.time_events(fn, reps) / reps
    msg = f"{op} {' '.join(argv[1:])}: {ms * 1e3:.1f} us per call"
    if work:
        msg += f", {work / ms / 1e9:.1f} effective TOPS"
    print(msg)


if __name__ == "__main__":
    main(sys.argv[1:])
