"""Offline product of the W4A4 path as a file: quantised weights, their scales and the transform.

The reference keeps the result of its offline pipeline -- ``compute_wush_transform`` ->
``transform_weights`` -> ``quant_int4`` -- only as live tensors and rebuilds it in every script
(``tests/test_p13.py:34-38``), which takes minutes of fp64 work at 70B layer sizes and ran out of
memory there (``bench/exp_p13_official.py:52-59``).  Here the triple ``{wq, ws, T}`` is written
once and loaded by whoever runs the layer.

Format (version 1): one ``torch.save`` archive holding a flat dict of tensors and plain values,
loadable with ``torch.load(..., weights_only=True)``:

    format        "wush-w4a4-layer"
    version       1
    K, N          in / out features
    group_size    32 (codes per scale; also the transform's block size)
    clip_sigmas   2.473650 (the sigma-clip constant c*; scale = c* sigma / 7 + 1e-8)
    wq            (N, K/2) uint8   packed codes, even element in the low nibble
    ws            (N, K/32) bfloat16 scales
    t             (K/32, 32, 32) bfloat16, T[g][j][i] multiplies input i into output j
    crc32         {"wq": ..., "ws": ..., "t": ...} of the tensors' bytes
    meta          free-form dict of str -> str / int / float (seed, source, ...)
"""
from __future__ import annotations

import os
import zlib
from dataclasses import dataclass, field

import torch

FORMAT = "wush-w4a4-layer"
VERSION = 1
GROUP_SIZE = 32
CLIP_SIGMAS = 2.473650


@dataclass
class LayerFile:
    K: int
    N: int
    wq: torch.Tensor
    ws: torch.Tensor
    t_bf16: torch.Tensor
    meta: dict = field(default_factory=dict)


def _crc(t: torch.Tensor) -> int:
    raw = t.detach().cpu().contiguous().view(torch.uint8).numpy()
    return zlib.crc32(raw.tobytes()) & 0xFFFFFFFF


def _validate(wq: torch.Tensor, ws: torch.Tensor, t: torch.Tensor) -> tuple[int, int]:
    if wq.dtype != torch.uint8 or wq.dim() != 2:
        raise ValueError("wq must be a 2-D uint8 tensor (N, K/2)")
    N, K = wq.shape[0], wq.shape[1] * 2
    if K % GROUP_SIZE:
        raise ValueError(f"K = {K} is not a multiple of {GROUP_SIZE}")
    if ws.dtype != torch.bfloat16 or tuple(ws.shape) != (N, K // GROUP_SIZE):
        raise ValueError(f"ws must be bfloat16 of shape ({N}, {K // GROUP_SIZE}), got {ws.dtype} {tuple(ws.shape)}")
    if t.dtype != torch.bfloat16 or tuple(t.shape) != (K // GROUP_SIZE, GROUP_SIZE, GROUP_SIZE):
        raise ValueError(f"t must be bfloat16 of shape ({K // GROUP_SIZE}, 32, 32), got {t.dtype} {tuple(t.shape)}")
    return K, N


def save_layer(path: str, wq: torch.Tensor, ws: torch.Tensor, t_bf16: torch.Tensor, meta: dict | None = None) -> None:
    """Writes one layer; the file appears under its final name only when complete."""
    K, N = _validate(wq, ws, t_bf16)
    tensors = {"wq": wq.detach().cpu().contiguous(), "ws": ws.detach().cpu().contiguous(),
               "t": t_bf16.detach().cpu().contiguous()}
    doc = {"format": FORMAT, "version": VERSION, "K": K, "N": N, "group_size": GROUP_SIZE, "clip_sigmas": CLIP_SIGMAS,
           **tensors, "crc32": {k: _crc(v) for k, v in tensors.items()}, "meta": dict(meta or {})}
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(doc, tmp)
    os.replace(tmp, path)


def load_layer(path: str, device="cpu", verify: bool = True) -> LayerFile:
    """Reads a layer written by ``save_layer`` onto ``device``; refuses other formats, newer
    versions, inconsistent shapes and (with ``verify``) tensors whose bytes changed."""
    doc = torch.load(path, map_location="cpu", weights_only=True)
    if not isinstance(doc, dict) or doc.get("format") != FORMAT:
        raise ValueError(f"{path}: not a {FORMAT} file")
    if int(doc.get("version", -1)) != VERSION:
        raise ValueError(f"{path}: format version {doc.get('version')} (this reader knows version {VERSION})")
    if int(doc["group_size"]) != GROUP_SIZE or abs(float(doc["clip_sigmas"]) - CLIP_SIGMAS) > 1e-9:
        raise ValueError(f"{path}: group size / clip constant differ from this build's kernels")
    wq, ws, t = doc["wq"], doc["ws"], doc["t"]
    K, N = _validate(wq, ws, t)
    if (K, N) != (int(doc["K"]), int(doc["N"])):
        raise ValueError(f"{path}: header says K={doc['K']} N={doc['N']}, tensors say K={K} N={N}")
    if verify:
        for name, tensor in (("wq", wq), ("ws", ws), ("t", t)):
            if _crc(tensor) != int(doc["crc32"][name]):
                raise ValueError(f"{path}: checksum of {name} does not match")
    return LayerFile(K=K, N=N, wq=wq.to(device), ws=ws.to(device), t_bf16=t.to(device), meta=dict(doc.get("meta", {})))


def prepare_layer(W: torch.Tensor, X_cal: torch.Tensor, quantiser=None, rows_per_block: int = 8192):
    """The offline pipeline on whatever device ``W`` lives on: transform solve from the calibration
    activations and the weights, ``W' = W T^-1`` rounded to bf16, sigma-clip quantisation.
    ``quantiser(x_bf16) -> (q, s)`` defaults to the torch reference semantics; on a GPU pass
    ``my_int4._C.quant_int4`` (bit-identical).  The weights are processed ``rows_per_block`` rows at
    a time, so only that many fp64 rows exist at once.  Returns ``(wq, ws, t_bf16, t_fp64)``."""
    from . import rtn_int4, wush_transform as wt

    quantiser = quantiser or rtn_int4.quant_int4
    t64 = wt.compute_wush_transform(X_cal, W, group_size=GROUP_SIZE)
    wq, ws = [], []
    for r0 in range(0, W.shape[0], rows_per_block):
        q, s = quantiser(wt.transform_weights(W[r0:r0 + rows_per_block], t64).to(torch.bfloat16).contiguous())
        wq.append(q)
        ws.append(s)
    return torch.cat(wq).contiguous(), torch.cat(ws).contiguous(), t64.to(torch.bfloat16).contiguous(), t64
