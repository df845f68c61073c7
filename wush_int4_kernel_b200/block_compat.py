"""Stand-ins for the two modules of the external IST-DASLab/WUSH checkout that the reference's
scripts import by name (``block_transform`` and ``compute_gram``).

The reference resolves them from a sibling checkout (``my_int4/wush_transform.py:15-24``) that is
not part of its repository.  Only the four functions its own code and tests call are provided,
with the keyword names seen at those call sites (``my_int4/wush_transform.py:36-58``,
``tests/test_sw1.py:30-33``); the arithmetic is this package's ``wush_transform``, not upstream's.
``my_int4`` registers them under the upstream names only when no real checkout is importable.
"""
from __future__ import annotations

import torch

from . import wush_transform as _wt


def get_diag_block_gram(x: torch.Tensor, size: int = 32, dtype=torch.float64) -> torch.Tensor:
    """(rows, K) -> (K/size, size, size): un-normalised diagonal blocks of x^T x."""
    return _wt.diag_block_gram(x, size, dtype)


def get_wush_transform(gram_weight: torch.Tensor, gram_activation: torch.Tensor, use_hadamard: bool = True,
                       high_dtype=torch.float64, round_dtype=torch.float64) -> torch.Tensor:
    """Per-block transform from the two second-moment tensors, each (K/G, G, G)."""
    return _wt.solve_from_grams(gram_activation.to(high_dtype), gram_weight.to(high_dtype), use_hadamard).to(round_dtype)


def get_inversed_transposed_transform(transform: torch.Tensor, high_dtype=torch.float64,
                                      round_dtype=torch.float64) -> torch.Tensor:
    """T -> T^-T per block, so that ``apply_block_transform(W, T^-T)`` equals ``W @ T^-1``."""
    return torch.linalg.inv(transform.to(high_dtype)).transpose(-1, -2).contiguous().to(round_dtype)


def apply_block_transform(x: torch.Tensor, transform: torch.Tensor, is_inverse_transpose: bool = False,
                          high_dtype=torch.float64, round_dtype=torch.float64) -> torch.Tensor:
    """Per block of the last dimension: ``x @ transform^T``, or ``x @ transform^-1`` (a solve, not an
    explicit inverse) when ``is_inverse_transpose``."""
    C, G, _ = transform.shape
    lead = x.shape[:-1]
    xb = x.to(high_dtype).reshape(-1, C, G).permute(1, 0, 2)                     # (C, rows, G)
    t = transform.to(high_dtype)
    if is_inverse_transpose:
        yb = torch.linalg.solve(t.transpose(-1, -2), xb.transpose(-1, -2)).transpose(-1, -2)   # y T = x
    else:
        yb = xb @ t.transpose(-1, -2)
    return yb.permute(1, 0, 2).reshape(*lead, C * G).to(round_dtype)
