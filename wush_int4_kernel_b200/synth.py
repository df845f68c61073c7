"""Seeded synthetic layers with the value distributions the benchmark configurations name.

No dataset or checkpoint is involved in the reference's own benchmarks either
(``bench/exp_p13_official.py:42-63`` draws random tensors of the layer shapes):

* activations ``X ~ N(0, 1)`` in bf16 with 0.5 % of the K channels (a seeded random subset)
  scaled by 20 -- the outlier channels;
* weights ``W ~ N(0, 0.02)`` in bf16;
* the transform is solved from 512 calibration rows drawn like X (same outlier channels);
* weights are transformed offline (``W' = W T^-1``), rounded to bf16 and quantised.

Small layers are drawn on the CPU (so the CPU oracle and the GPU see identical bits); big
ones directly on the GPU, block by block, to bound host memory.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import rtn_int4, wush_transform

OUTLIER_FRACTION = 0.005
OUTLIER_GAIN = 20.0
CALIB_ROWS = 512


@dataclass
class Layer:
    K: int
    N: int
    t_bf16: torch.Tensor          # (K/32, 32, 32) bf16
    wq: torch.Tensor              # (N, K/2) uint8
    ws: torch.Tensor              # (N, K/32) bf16
    outliers: torch.Tensor        # indices of the outlier channels
    w_ref: torch.Tensor | None = None     # original bf16 weights (kept for small layers only)


def outlier_channels(K: int, gen: torch.Generator) -> torch.Tensor:
    n = max(1, round(OUTLIER_FRACTION * K))
    return torch.randperm(K, generator=gen, device=gen.device)[:n]


def draw_activations(M: int, K: int, outliers: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
    x = torch.randn(M, K, generator=gen, device=gen.device)
    x[:, outliers] *= OUTLIER_GAIN
    return x.to(torch.bfloat16)


def make_layer(K: int, N: int, seed: int = 0, device: str = "cpu", quantiser=None, keep_weights: bool = False,
               rows_per_block: int = 8192) -> Layer:
    """Builds one quantised layer.  ``quantiser(x_bf16) -> (q, s)`` defaults to the torch
    reference semantics; pass ``my_int4._C.quant_int4`` on a GPU (bit-identical, much faster)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    quantiser = quantiser or rtn_int4.quant_int4
    outliers = outlier_channels(K, gen)
    x_cal = draw_activations(CALIB_ROWS, K, outliers, gen).float()
    # weights block by block; the weight Gram for the solve is accumulated on the fly
    blocks, gram = [], torch.zeros(K // 32, 32, 32, dtype=torch.float64, device=device)
    for r0 in range(0, N, rows_per_block):
        w = (0.02 * torch.randn(min(rows_per_block, N - r0), K, generator=gen, device=device)).to(torch.bfloat16)
        gram += wush_transform.diag_block_gram(w, 32)
        blocks.append(w)
    t64 = wush_transform.solve_from_grams(wush_transform.diag_block_gram(x_cal, 32) / CALIB_ROWS, gram / N)
    wq, ws = [], []
    for w in blocks:
        q, s = quantiser(wush_transform.transform_weights(w, t64).to(torch.bfloat16).contiguous())
        wq.append(q)
        ws.append(s)
    return Layer(K=K, N=N, t_bf16=t64.to(torch.bfloat16).contiguous(), wq=torch.cat(wq).contiguous(),
                 ws=torch.cat(ws).contiguous(), outliers=outliers,
                 w_ref=torch.cat(blocks) if keep_weights else None)
