"""Regenerates ``tests/golden/*.npz`` by RUNNING THE REFERENCE'S OWN PYTHON on CPU.

Run where the reference checkout is present::

    python tests/golden/make_golden.py /path/to/WUSH_int4_kernel

``my_int4/rtn_int4.py`` of the reference is loaded by file path (its package
``__init__`` imports the compiled extension, which does not exist on a CPU box), and
its ``quant_int4`` / ``dequant_int4`` / ``w4a4_matmul_reference`` produce every
expected output stored here.  The only arithmetic restated in this script is the
32-step transform loop of the reference's ``tests/test_sw2.py:12-24`` (that test
file cannot be imported: it loads the CUDA extension at import time) and the
per-tensor mirror of ``tests/test_p12.py:22-27``.

bf16 / fp16 tensors are stored as uint16 bit patterns.  The files are small (a few
hundred KB in total) and are committed; the GPU box never needs the reference.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    spec = importlib.util.spec_from_file_location("ref_rtn_int4", os.path.join(root, "my_int4", "rtn_int4.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def b16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def transform_mirror(x: torch.Tensor, T: torch.Tensor) -> torch.Tensor:
    """fp32 x' = sum_i x_i * T[g][j][i], i ascending, one rounding per multiply and per add."""
    xf = x.float().reshape(-1, x.size(-1))
    xg = xf.unflatten(-1, (-1, 32))
    acc = torch.zeros_like(xg)
    Tf = T.float()
    for i in range(32):
        acc = acc + xg[:, :, i].unsqueeze(-1) * Tf[:, :, i].unsqueeze(0)
    return acc.flatten(-2)


def main(root: str) -> None:
    ref = load_reference(root)
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16

    # ---------------- a1: quant_int4 ------------------------------------------------
    cases = {}
    x = torch.zeros(1, 32, dtype=bf)
    x[0, 0::2] = 1.0
    x[0, 1::2] = -1.0
    cases["pm1"] = x                                                   # reference tests/test_rtn_int4.py:11-20
    cases["randn"] = torch.randn(256, 128, generator=g).to(bf)
    cases["rank3"] = torch.randn(2, 3, 96, generator=g).to(bf)          # tests/test_s2.py:21
    cases["zeros"] = torch.zeros(4, 32, dtype=bf)                       # tests/test_s2.py:22
    t = torch.zeros(2, 32, dtype=bf)
    t[0, :8] = torch.tensor([7., -7., 2.5, -2.5, 3.5, -3.5, 0.5, -0.5]).to(bf)
    t[1, :8] = (torch.tensor([0.5, 1.5, 2.5, 3.5, 4.5, 5.5, 6.5, -6.5]) * 0.7).to(bf)
    cases["ties"] = t                                                  # tests/test_s2.py:26-29
    cases["overflow"] = torch.full((4, 32), 3.3e38, dtype=bf)          # tests/test_s2.py:32-36
    cases["tiny"] = (torch.randn(8, 64, generator=g) * 1e-30).to(bf)
    wide = torch.randn(32, 256, generator=g) * torch.exp(4 * torch.randn(32, 256, generator=g))
    cases["wide"] = wide.to(bf)
    out = {"pm1_expect_codes": np.array([3, -3] * 16, np.int8)}
    out["names"] = np.array(sorted(cases))
    for name, xin in cases.items():
        q, s = ref.quant_int4(xin)
        s = s.reshape(*xin.shape[:-1], -1)      # the reference squeezes the group axis when K == 32
        d = ref.dequant_int4(q, s)
        out[f"{name}_x"] = b16(xin)
        out[f"{name}_q"] = q.numpy().copy()
        out[f"{name}_s"] = b16(s)
        out[f"{name}_dq"] = d.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "quant_int4.npz"), **out)

    # ---------------- a3/a4: fused transform + quant ---------------------------------
    out = {}
    X = torch.randn(64, 128, generator=g).to(bf)
    X[:, 5::32] *= 12.0
    fcases = {
        "randT": (X, torch.randn(4, 32, 32, generator=g).to(bf)),
        "smallT": (X, (torch.randn(4, 32, 32, generator=g) / 6).to(bf)),
        "rank3": (torch.randn(2, 3, 96, generator=g).to(bf), torch.randn(3, 32, 32, generator=g).to(bf)),
        "zeros": (torch.zeros(4, 64, dtype=bf), torch.randn(2, 32, 32, generator=g).to(bf)),
        "eye": (X, torch.eye(32).repeat(4, 1, 1).to(bf)),
    }
    out["names"] = np.array(sorted(fcases))
    for name, (xin, T) in fcases.items():
        xt = transform_mirror(xin, T)
        q, s = ref.quant_int4(xt)
        out[f"{name}_x"] = b16(xin)
        out[f"{name}_t"] = b16(T)
        out[f"{name}_xt"] = xt.numpy().copy()
        out[f"{name}_q"] = q.reshape(*xin.shape[:-1], -1).numpy().copy()
        out[f"{name}_s"] = b16(s.reshape(*xin.shape[:-1], -1))
    np.savez_compressed(os.path.join(HERE, "fused_tq.npz"), **out)

    # ---------------- a2/a8/a9: W4A4 product ------------------------------------------
    out = {}
    shapes = [(64, 96, 128), (1, 64, 64), (8, 32, 64), (33, 50, 96), (5, 72, 256)]  # tests/test_p13.py:18, test_s3.py:36-43 style
    out["shapes"] = np.array(shapes)
    for (M, N, K) in shapes:
        Xm = torch.randn(M, K, generator=g).to(bf)
        Wm = torch.randn(N, K, generator=g).to(bf)
        xq, xs = ref.quant_int4(Xm)
        wq, ws = ref.quant_int4(Wm)
        y = ref.w4a4_matmul_reference(xq, xs, wq, ws)
        y64 = ref.dequant_int4(xq, xs).double() @ ref.dequant_int4(wq, ws).double().t()
        k = f"{M}x{N}x{K}"
        out[f"{k}_xq"], out[f"{k}_xs"] = xq.numpy().copy(), b16(xs)
        out[f"{k}_wq"], out[f"{k}_ws"] = wq.numpy().copy(), b16(ws)
        out[f"{k}_y16"] = b16(y)
        out[f"{k}_y64"] = y64.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "w4a4_matmul.npz"), **out)

    # ---------------- per-tensor route (tests/test_p12.py:22-27 mirror) -----------------
    out = {}
    Xp = torch.randn(16, 256, generator=g).to(bf)
    sweep = (torch.linspace(-8.5, 8.5, 512) * 0.37).to(bf).reshape(2, 256)
    for name, xin in {"randn": Xp, "sweep": sweep}.items():
        amax = xin.float().abs().max().clamp_min(1e-8)
        scale = (amax / 7.0).item()
        inv = torch.tensor(1.0 / scale, dtype=torch.float32)
        q = torch.round(xin.float() * inv).clamp_(-7, 7).to(torch.int8) & 0xF
        packed = (q[..., 0::2] | (q[..., 1::2] << 4)).to(torch.uint8).reshape(-1)
        out[f"{name}_x"] = b16(xin)
        out[f"{name}_scale"] = np.array(scale, np.float64)
        out[f"{name}_q"] = packed.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "per_tensor.npz"), **out)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
