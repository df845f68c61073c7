"""ctypes front-end of the CPU oracle (``w4a4_oracle.c``) -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke test and the CPU-baseline leg of the benchmark may
import this module; the shipped CUDA path never does.  Arrays are numpy; bf16 and
fp16 values are carried as ``uint16`` bit patterns.  Helpers at the bottom convert
to and from torch tensors for the tests.

Reference lines each function follows are cited in ``w4a4_oracle.c``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libw4a4_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in ``oracle/Makefile``."""
    src = os.path.join(_HERE, "w4a4_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_abi_version.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


I64 = ctypes.c_int64


def quant_int4(x_bf16: np.ndarray):
    """(…, K) bf16 bits -> (q u8 (…, K/2), s bf16 bits (…, K/32))."""
    x = _c(x_bf16, np.uint16)
    K = x.shape[-1]
    assert K % 32 == 0
    ng = x.size // 32
    q = np.empty(x.shape[:-1] + (K // 2,), np.uint8)
    s = np.empty(x.shape[:-1] + (K // 32,), np.uint16)
    lib().orc_quant_int4(_p(x), I64(ng), _p(q), _p(s))
    return q, s


def quant_int4_f32(x_f32: np.ndarray):
    x = _c(x_f32, np.float32)
    K = x.shape[-1]
    ng = x.size // 32
    q = np.empty(x.shape[:-1] + (K // 2,), np.uint8)
    s = np.empty(x.shape[:-1] + (K // 32,), np.uint16)
    lib().orc_quant_int4_f32(_p(x), I64(ng), _p(q), _p(s))
    return q, s


def transform_f32(x_bf16: np.ndarray, t_bf16: np.ndarray) -> np.ndarray:
    x = _c(x_bf16, np.uint16)
    t = _c(t_bf16, np.uint16)
    K = x.shape[-1]
    C = K // 32
    assert t.shape == (C, 32, 32)
    rows = x.size // K
    out = np.empty(x.shape, np.float32)
    lib().orc_transform_f32(_p(x), _p(t), I64(rows), I64(C), _p(out))
    return out


def fused_tq(x_bf16: np.ndarray, t_bf16: np.ndarray):
    x = _c(x_bf16, np.uint16)
    t = _c(t_bf16, np.uint16)
    K = x.shape[-1]
    C = K // 32
    assert t.shape == (C, 32, 32)
    rows = x.size // K
    q = np.empty(x.shape[:-1] + (K // 2,), np.uint8)
    s = np.empty(x.shape[:-1] + (C,), np.uint16)
    lib().orc_fused_tq(_p(x), _p(t), I64(rows), I64(C), _p(q), _p(s))
    return q, s


def dequant(q: np.ndarray, s: np.ndarray) -> np.ndarray:
    q = _c(q, np.uint8)
    s = _c(s, np.uint16)
    K = q.shape[-1] * 2
    rows = q.size // (K // 2)
    out = np.empty(q.shape[:-1] + (K,), np.float32)
    lib().orc_dequant(_p(q), _p(s), I64(rows), I64(K), _p(out))
    return out


def _mnk(xq, wq):
    K2 = wq.shape[-1]
    M = xq.size // K2
    N = wq.shape[0]
    return M, N, K2 * 2


def group_partials(xq: np.ndarray, wq: np.ndarray) -> np.ndarray:
    xq = _c(xq, np.uint8)
    wq = _c(wq, np.uint8)
    M, N, K = _mnk(xq, wq)
    P = np.empty((M, N, K // 32), np.int32)
    lib().orc_group_partials(_p(xq), _p(wq), I64(M), I64(N), I64(K), _p(P))
    return P


def gemm_f64(xq, xs, wq, ws) -> np.ndarray:
    xq, wq = _c(xq, np.uint8), _c(wq, np.uint8)
    xs, ws = _c(xs, np.uint16), _c(ws, np.uint16)
    M, N, K = _mnk(xq, wq)
    y = np.empty((M, N), np.float64)
    lib().orc_gemm_f64(_p(xq), _p(xs), _p(wq), _p(ws), I64(M), I64(N), I64(K), _p(y))
    return y


def gemm_f16(xq, xs, wq, ws) -> np.ndarray:
    """fp16 bit patterns (M, N) as uint16; use ``.view(np.float16)`` to read them."""
    xq, wq = _c(xq, np.uint8), _c(wq, np.uint8)
    xs, ws = _c(xs, np.uint16), _c(ws, np.uint16)
    M, N, K = _mnk(xq, wq)
    y = np.empty((M, N), np.uint16)
    lib().orc_gemm_f16(_p(xq), _p(xs), _p(wq), _p(ws), I64(M), I64(N), I64(K), _p(y))
    return y


def quant_tensor_scale(x_bf16: np.ndarray, inv_scale: float) -> np.ndarray:
    x = _c(x_bf16, np.uint16)
    q = np.empty(x.size // 2, np.uint8)
    lib().orc_quant_tensor_scale(_p(x), I64(x.size), ctypes.c_float(inv_scale), _p(q))
    return q


def gemm_tensor_scale(xq, wq, alpha: float):
    """Returns (y fp16 bits (M,N), int32 accumulators (M,N))."""
    xq, wq = _c(xq, np.uint8), _c(wq, np.uint8)
    M, N, K = _mnk(xq, wq)
    y = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.int32)
    lib().orc_gemm_tensor_scale(_p(xq), _p(wq), I64(M), I64(N), I64(K), ctypes.c_float(alpha),
                                _p(y), _p(acc))
    return y, acc


def layer(x_bf16, t_bf16, wq, ws) -> np.ndarray:
    """fused transform+quant then W4A4 product; fp16 bits (M, N)."""
    x, t = _c(x_bf16, np.uint16), _c(t_bf16, np.uint16)
    wq, ws = _c(wq, np.uint8), _c(ws, np.uint16)
    K = x.shape[-1]
    M = x.size // K
    N = wq.shape[0]
    xq = np.empty((M, K // 2), np.uint8)
    xs = np.empty((M, K // 32), np.uint16)
    y = np.empty((M, N), np.uint16)
    lib().orc_layer(_p(x), _p(t), _p(wq), _p(ws), I64(M), I64(N), I64(K), _p(xq), _p(xs), _p(y))
    return y


def set_threads(n: int) -> None:
    """OpenMP thread count for the next calls (libgomp reads it per region)."""
    try:
        gomp = ctypes.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(int(n))
    except OSError:
        os.environ["OMP_NUM_THREADS"] = str(int(n))


# ---- torch <-> numpy helpers for the tests (bf16/fp16 as uint16 bits) --------
def bits(t) -> np.ndarray:
    """torch bf16/fp16 tensor (any device) -> numpy uint16 bit patterns."""
    import torch

    assert t.dtype in (torch.bfloat16, torch.float16)
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(a: np.ndarray, dtype):
    """numpy uint16 bit patterns -> torch tensor of ``dtype`` (bf16 or fp16)."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(dtype)
