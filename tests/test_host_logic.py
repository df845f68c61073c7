"""CPU checks of everything above the kernels: torch reference semantics vs the oracle,
transform algebra, sharding arithmetic, and that the C-ABI library loads and exports every
symbol the header declares (no compute calls: there is no GPU here)."""
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_exported():
    from wush_int4_kernel_b200 import capi

    header = open(os.path.join(ROOT, "include", "wush_int4.h")).read()
    declared = set(re.findall(r"\b(wush_[a-z0-9_]+)\s*\(", header))
    declared -= {"wush_status"}
    assert declared == set(capi.SIGNATURES), declared ^ set(capi.SIGNATURES)
    lib = capi.load()                      # AttributeError inside if any symbol is missing
    assert lib.wush_abi_version() == 1


def test_header_constants_match_the_python_binding():
    """Variant, quantiser-mode and status numbers of the header are the ones capi.py passes."""
    from wush_int4_kernel_b200 import capi

    header = open(os.path.join(ROOT, "include", "wush_int4.h")).read()
    enums = {name: int(value) for name, value in re.findall(r"\b(WUSH_[A-Z0-9_]+)\s*=\s*(-?\d+)", header)}
    for name, value in enums.items():
        short = name[len("WUSH_"):]
        mirror = getattr(capi, short, getattr(capi, name, None))
        if mirror is not None:
            assert mirror == value, (name, value, mirror)
    for name in ("GEMM_AUTO", "GEMM_GEMV", "GEMM_DECODE", "GEMM_TILE", "GEMM_TILE_F16", "GEMM_DECODE_TC", "GEMM_GEMV_MMA",
                 "TQ_EXACT", "TQ_FAST"):
        assert enums["WUSH_" + name] == getattr(capi, name), name
    assert enums["WUSH_OK"] == capi.WUSH_OK == 0 and enums["WUSH_ERR_INVALID_ARGUMENT"] == capi.WUSH_ERR_INVALID_ARGUMENT


def test_no_gpu_fails_loudly():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from wush_int4_kernel_b200 import capi

    lib = capi.load()
    assert lib.wush_init() != capi.WUSH_OK
    assert b"CUDA" in lib.wush_last_error() or b"device" in lib.wush_last_error()
    with pytest.raises(capi.WushError):
        capi.check(lib.wush_quant_int4(None, 1, None, None, None), "quant_int4")


def test_operator_surface_matches_reference():
    import my_int4
    from my_int4 import _C

    names = ["quant_int4", "w4a4_gemm", "w4a4_gemm_v1", "w4a4_gemm_v2", "w4a4_gemm_s4", "w4a4_gemv", "w4a4_gemv_multi",
             "s4_atom_selftest", "fused_transform_quant_int4", "fused_transform_quant_int4_wmma",
             "fused_transform_quant_int4_v3", "fused_transform_quant_int4_smallm", "quant_int4_tensor_scale",
             "quant_int4_tensor_scale_dev", "w4a4_gemm_cutlass", "w4a4_gemm_cutlass_dev"]
    for n in names:                         # reference csrc/bindings.cpp:28-68
        assert callable(getattr(_C, n)), n
    assert my_int4.quant_int4 is _C.quant_int4
    from my_int4.rtn_int4 import quant_int4, dequant_int4, w4a4_matmul_reference  # noqa: F401
    from my_int4.wush_transform import compute_wush_transform, transform_weights, transform_activations_reference  # noqa: F401
    # CPU tensors are rejected with RuntimeError, as TORCH_CHECK does in the reference
    with pytest.raises(RuntimeError):
        _C.quant_int4(torch.zeros(4, 32, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        _C.w4a4_gemv(torch.zeros(1, 16, dtype=torch.uint8), torch.zeros(1, 1, dtype=torch.bfloat16),
                     torch.zeros(8, 16, dtype=torch.uint8), torch.zeros(8, 1, dtype=torch.bfloat16))


def test_torch_semantics_equal_oracle(orc):
    from wush_int4_kernel_b200 import rtn_int4

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(128, 256, generator=g) * torch.exp(2 * torch.randn(128, 256, generator=g))).to(torch.bfloat16)
    q, s = rtn_int4.quant_int4(x)
    qo, so = orc.quant_int4(orc.bits(x))
    assert np.array_equal(q.numpy(), qo) and np.array_equal(orc.bits(s), so)
    assert np.array_equal(rtn_int4.dequant_int4(q, s).numpy(), orc.dequant(qo, so))
    w = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    wq, ws = rtn_int4.quant_int4(w)
    y = rtn_int4.w4a4_matmul_reference(q, s, wq, ws).double().numpy()
    y64 = orc.gemm_f64(qo, so, wq.numpy(), orc.bits(ws))
    assert np.linalg.norm(y - y64) / np.linalg.norm(y64) < 1e-3


def test_transform_product_invariance():
    # reference tests/test_sw1.py:12-27
    from wush_int4_kernel_b200 import wush_transform as wt

    torch.manual_seed(0)
    M, N, K, G = 256, 128, 128, 32
    X = torch.randn(M, K, dtype=torch.float64)
    W = torch.randn(N, K, dtype=torch.float64)
    X[:, 5::G] *= 15.0
    W[:, 12::G] *= 8.0
    T = wt.compute_wush_transform(X, W, group_size=G)
    assert T.shape == (K // G, G, G) and T.dtype == torch.float64
    Xp, Wp = wt.transform_activations_reference(X, T), wt.transform_weights(W, T)
    Y = X @ W.t()
    assert ((Xp @ Wp.t() - Y).norm() / Y.norm()).item() < 1e-9
    # the two equivalent routes of the weight transform (tests/test_sw1.py:29-38)
    Wb = torch.einsum("nci,cij->ncj", W.reshape(N, -1, G), torch.linalg.inv(T)).reshape(N, K)
    assert torch.allclose(Wp, Wb, rtol=1e-9, atol=1e-9)


def test_transform_end_to_end_accuracy(orc):
    # reference tests/test_p13.py:29-43 on a quarter of its rows: outlier data, WUSH + INT4
    # G=32 must stay under the 8.2 % gate (the reference measures 7.8 %); bare INT4 is ~53 %.
    from wush_int4_kernel_b200 import rtn_int4, wush_transform as wt

    torch.manual_seed(0)
    M, N, K, G = 512, 512, 4096, 32
    X = torch.randn(M, K).to(torch.bfloat16)
    X[:, 5::G] *= 15.0
    W = torch.randn(N, K).to(torch.bfloat16)
    W[:, 12::G] *= 8.0
    Y = (X.double() @ W.double().t()).numpy()
    Xc = torch.randn(256, K)
    Xc[:, 5::G] *= 15.0
    T = wt.compute_wush_transform(Xc, W.float(), group_size=G)
    wq, ws = rtn_int4.quant_int4(wt.transform_weights(W.double(), T).to(torch.bfloat16).contiguous())
    xq, xs = orc.fused_tq(orc.bits(X), orc.bits(T.to(torch.bfloat16)))
    y = orc.gemm_f64(xq, xs, wq.numpy(), orc.bits(ws))
    err = np.linalg.norm(y - Y) / np.linalg.norm(Y)
    assert err <= 0.082, err
    xq0, xs0 = rtn_int4.quant_int4(X)
    wq0, ws0 = rtn_int4.quant_int4(W)
    bare = orc.gemm_f64(xq0.numpy(), orc.bits(xs0), wq0.numpy(), orc.bits(ws0))
    assert np.linalg.norm(bare - Y) / np.linalg.norm(Y) > 0.3


def test_shard_bounds_cover_exactly():
    from wush_int4_kernel_b200.linear import shard_bounds

    for total, mult in [(57344, 128), (24576, 128), (28672, 32), (8192, 32), (96, 32), (7, 1)]:
        for world in (1, 2, 3, 4, 8):
            if (total // mult) < world:
                continue
            cuts = [shard_bounds(total, world, r, mult) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == total
            for (a, b), (c, d) in zip(cuts, cuts[1:]):
                assert b == c and a < b and a % mult == 0
            sizes = [b - a for a, b in cuts]
            assert max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        shard_bounds(100, 2, 0, 32)
    with pytest.raises(ValueError):
        shard_bounds(64, 2, 2, 32)


def test_synthetic_layer_is_seeded():
    from wush_int4_kernel_b200 import synth

    a = synth.make_layer(256, 64, seed=5)
    b = synth.make_layer(256, 64, seed=5)
    c = synth.make_layer(256, 64, seed=6)
    assert torch.equal(a.wq, b.wq) and torch.equal(a.ws.view(torch.int16), b.ws.view(torch.int16))
    assert not torch.equal(a.wq, c.wq)
    assert a.wq.shape == (64, 128) and a.ws.shape == (64, 8) and a.t_bf16.shape == (8, 32, 32)
    assert len(a.outliers) == max(1, round(0.005 * 256))


def test_block_compat_matches_reference_call_sites():
    """The stand-ins for the external `block_transform` / `compute_gram` modules, exercised the way the
    reference's tests/test_sw1.py:14-38 does: product invariance < 1e-9 and the two routes to W T^-1 agree."""
    import torch
    from wush_int4_kernel_b200 import block_compat as bt, wush_transform as wt
    gen = torch.Generator().manual_seed(0)
    M, N, K = 256, 128, 128
    X = torch.randn(M, K, dtype=torch.float64, generator=gen)
    W = torch.randn(N, K, dtype=torch.float64, generator=gen)
    X[:, 5::32] *= 15.0
    W[:, 12::32] *= 8.0
    hi = torch.float64
    T = bt.get_wush_transform(gram_weight=bt.get_diag_block_gram(x=W, size=32, dtype=hi) / N,
                              gram_activation=bt.get_diag_block_gram(x=X, size=32, dtype=hi) / M,
                              use_hadamard=True, high_dtype=hi, round_dtype=hi)
    assert torch.equal(T, wt.compute_wush_transform(X, W, group_size=32))
    T_w = bt.get_inversed_transposed_transform(T, high_dtype=hi, round_dtype=hi)
    Wa = bt.apply_block_transform(x=W, transform=T, is_inverse_transpose=True)
    Wb = bt.apply_block_transform(x=W, transform=T_w, is_inverse_transpose=False)
    assert torch.allclose(Wa, Wb, rtol=1e-9, atol=1e-9)
    Xp = bt.apply_block_transform(x=X, transform=T, is_inverse_transpose=False)
    Y = X @ W.t()
    assert ((Xp @ Wa.t() - Y).norm() / Y.norm()).item() < 1e-9
