"""ctypes view of ``libwush_int4_b200.so`` -- the C ABI declared in ``include/wush_int4.h``.

This is the boundary a non-Python host would bind.  Pointers are raw device addresses
(``tensor.data_ptr()``), the stream is a raw ``cudaStream_t``.  Loading fails loudly when the
library has not been built; nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libwush_int4_b200.so")

WUSH_OK = 0
WUSH_ERR_INVALID_ARGUMENT, WUSH_ERR_CUDA, WUSH_ERR_UNSUPPORTED, WUSH_ERR_WORKSPACE, WUSH_ERR_DEVICE_FLAG = 1, 2, 3, 4, 5
TQ_EXACT, TQ_FAST = 0, 1
GEMM_AUTO, GEMM_GEMV, GEMM_DECODE, GEMM_TILE, GEMM_TILE_F16, GEMM_DECODE_TC, GEMM_GEMV_MMA = 0, 1, 2, 3, 4, 5, 6

_vp, _i64, _int, _f32, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes): every symbol include/wush_int4.h declares
SIGNATURES = {
    "wush_abi_version": (_int, []),
    "wush_last_error": (ctypes.c_char_p, []),
    "wush_init": (_int, []),
    "wush_device_flag": (_int, [_vp]),
    "wush_quant_int4": (_int, [_vp, _i64, _vp, _vp, _vp]),
    "wush_fused_transform_quant_int4": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "wush_fused_silu_mul_transform_quant_int4": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "wush_w4a4_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "wush_w4a4_gemm_pick_variant": (_int, [_i64, _i64, _i64]),
    "wush_w4a4_gemm": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _vp, _sz, _vp]),
    "wush_w4a4_gemm_static_scratch_limit": (_sz, []),
    "wush_w4a4_gemm_static_scratch": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "wush_i8_atom_selftest": (_int, [_vp, _vp, _vp, _vp]),
    "wush_i8_tile_selftest": (_int, [_vp, _vp, _vp, _int, _int, _vp, _vp]),
    "wush_group_partials": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "wush_quant_int4_tensor_scale": (_int, [_vp, _i64, _f32, _vp, _vp, _vp]),
    "wush_w4a4_gemm_tensor_scale": (_int, [_vp, _vp, _i64, _i64, _i64, _f32, _vp, _vp, _vp]),
    "wush_comm_create": (_int, [_int, _int, _sz, ctypes.POINTER(ctypes.c_void_p)]),
    "wush_comm_export": (_int, [_vp, _vp]),
    "wush_comm_connect": (_int, [_vp, _int, _vp]),
    "wush_comm_connect_pointer": (_int, [_vp, _int, _vp]),
    "wush_comm_base": (_int, [_vp, ctypes.POINTER(ctypes.c_void_p)]),
    "wush_comm_set_poll_limit": (_int, [_vp, ctypes.c_uint]),
    "wush_comm_allreduce_f16": (_int, [_vp, _vp, _vp, _i64, _vp]),
    "wush_comm_gemv_allreduce": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "wush_comm_allreduce_two_phase_f16": (_int, [_vp, _vp, _vp, _i64, _vp]),
    "wush_comm_allgather_f16": (_int, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "wush_comm_gemv_allgather": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "wush_comm_error": (_int, [_vp, ctypes.POINTER(_int)]),
    "wush_comm_destroy": (_int, [_vp]),
    "wush_debug_stream_tiles": (_int, [_i64]),
    "wush_debug_unit_cover": (_int, [_i64, _int, _int, _int, _int, ctypes.c_double, ctypes.c_double,
                                     ctypes.POINTER(_int), _int, ctypes.POINTER(_int)]),
    "wush_w4a4_gemm_tensor_scale_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "wush_w4a4_gemm_tensor_scale_ws": (_int, [_vp, _vp, _i64, _i64, _i64, _f32, _vp, _vp, _vp, _sz, _vp]),
}

_lib = None


class WushError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m wush_int4_kernel_b200.build`")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if a declared symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != WUSH_OK:
        raise WushError(f"{what}: {load().wush_last_error().decode()} (status {status})")
