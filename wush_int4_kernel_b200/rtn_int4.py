"""Torch statement of the INT4 quantiser semantics (any device; used by tests, offline weight
preparation on CPU and as documentation of the contract the CUDA kernels are bit-exact with).

Same API and bit-identical results as the reference's ``my_int4/rtn_int4.py:33-75``:

* groups of 32 along the last axis; fp32 statistics accumulated element by element in index
  order (a tree reduction would round differently);
* ``scale = sqrt(E[x^2] - E[x]^2) * (2.473650 / 7) + 1e-8`` (1.0 when the variance is negative
  or NaN), stored as bf16, and the codes are computed from the bf16-rounded scale;
* codes ``clamp(round_half_even(x / scale), -7, 7)``, packed two per byte, even element in
  the low nibble, two's complement.

Nothing in the CUDA path calls this module.
"""
from __future__ import annotations

import torch

GROUP = 32
QMAX = 7
C_CLIP = 0.35337862372398376      # 2.473650 / 7


def _ordered_moments(groups: torch.Tensor):
    """sum(x) and sum(x*x) over the last axis, accumulated left to right in fp32."""
    total = torch.zeros_like(groups[..., 0])
    total_sq = torch.zeros_like(total)
    for column in groups.unbind(-1):
        total = total + column
        total_sq = total_sq + column * column
    return total, total_sq


def group_scales(x: torch.Tensor, group_size: int = GROUP) -> torch.Tensor:
    """bf16 sigma-clip scales, shape (..., K/group_size)."""
    assert group_size == GROUP, "the moment normalisation below is written for groups of 32"
    groups = x.float().unflatten(-1, (-1, group_size))
    s1, s2 = _ordered_moments(groups)
    mean = s1 / 32.0
    var = s2 / 32.0 - mean * mean
    scale = torch.where(var >= 0, torch.sqrt(var) * C_CLIP + 1e-8, torch.ones_like(var))
    return scale.to(torch.bfloat16)


def quant_int4(x: torch.Tensor, group_size: int = GROUP):
    """x (..., K) -> (packed uint8 (..., K/2), bf16 scales (..., K/group_size))."""
    groups = x.float().unflatten(-1, (-1, group_size))
    scale = group_scales(x, group_size)
    codes = torch.round(groups / scale.float().unsqueeze(-1)).clamp(-QMAX, QMAX).to(torch.int8)
    nib = (codes.to(torch.uint8) & 0xF).flatten(-2)
    packed = nib[..., 0::2] | (nib[..., 1::2] << 4)
    return packed, scale


def unpack_int4(q_byte: torch.Tensor) -> torch.Tensor:
    """packed uint8 (..., K/2) -> int8 codes (..., K) with sign extension."""
    lo = (q_byte & 0xF).to(torch.int8)
    hi = (q_byte >> 4).to(torch.int8)
    both = torch.stack((lo, hi), dim=-1).flatten(-2)
    return torch.where(both > 7, both - 16, both)


def dequant_int4(q_byte: torch.Tensor, scale: torch.Tensor, group_size: int = GROUP) -> torch.Tensor:
    """(packed uint8 (..., K/2), bf16 scales (..., K/group_size)) -> fp32 (..., K)."""
    codes = unpack_int4(q_byte).float().unflatten(-1, (-1, group_size))
    return (codes * scale.float().reshape(*codes.shape[:-1], 1)).flatten(-2)


def w4a4_matmul_reference(x_q, x_s, w_q, w_s) -> torch.Tensor:
    """Y = dequant(X) @ dequant(W)^T in fp32, returned as fp16."""
    return (dequant_int4(x_q, x_s) @ dequant_int4(w_q, w_s).transpose(-1, -2)).to(torch.float16)
