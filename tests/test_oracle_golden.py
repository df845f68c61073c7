"""The CPU oracle against the golden vectors produced by the reference's own Python
(tests/golden/make_golden.py) and against the reference's hand-computed known answers."""
import numpy as np
import pytest


def test_quant_golden(golden, orc):
    z = golden("quant_int4")
    for name in z["names"]:
        q, s = orc.quant_int4(z[f"{name}_x"])
        assert np.array_equal(q, z[f"{name}_q"]), name
        assert np.array_equal(s, z[f"{name}_s"]), name
        assert np.array_equal(orc.dequant(q, s).view(np.uint32), z[f"{name}_dq"].view(np.uint32)), name


def test_known_answer_pm1(golden, orc):
    # reference tests/test_rtn_int4.py:11-20: alternating +-1 -> sigma = 1 -> codes +-3
    z = golden("quant_int4")
    q, s = orc.quant_int4(z["pm1_x"])
    codes = z["pm1_expect_codes"].astype(np.uint8)
    expect = (codes[0::2] & 0xF) | ((codes[1::2] & 0xF) << 4)
    assert np.array_equal(q.reshape(-1), expect)
    d = orc.dequant(q, s).reshape(-1)
    scale = (s.astype(np.uint32) << 16).view(np.float32).reshape(-1)[0]
    assert np.array_equal(d, z["pm1_expect_codes"].astype(np.float32) * scale)


def test_zero_groups(orc):
    # reference tests/test_rtn_int4.py:35-38: sigma = 0 -> scale 1e-8 -> all codes 0
    q, s = orc.quant_int4(np.zeros((4, 32), np.uint16))
    assert (q == 0).all()


def test_fused_golden(golden, orc):
    z = golden("fused_tq")
    for name in z["names"]:
        x, t = z[f"{name}_x"], z[f"{name}_t"]
        xt = orc.transform_f32(x, t)
        assert np.array_equal(xt.view(np.uint32).reshape(-1), z[f"{name}_xt"].view(np.uint32).reshape(-1)), name
        q, s = orc.fused_tq(x, t)
        assert np.array_equal(q, z[f"{name}_q"]), name
        assert np.array_equal(s, z[f"{name}_s"]), name
        q2, s2 = orc.quant_int4_f32(xt)
        assert np.array_equal(q2, q) and np.array_equal(s2, s), name


def test_matmul_golden(golden, orc):
    z = golden("w4a4_matmul")
    for (M, N, K) in z["shapes"]:
        k = f"{M}x{N}x{K}"
        args = (z[k + "_xq"], z[k + "_xs"], z[k + "_wq"], z[k + "_ws"])
        y64 = orc.gemm_f64(*args)
        ref64 = z[k + "_y64"]
        assert np.abs(y64 - ref64).max() <= 1e-12 * max(1.0, np.abs(ref64).max()), k
        # reference's fp32 matmul -> fp16: summation order is not part of the contract, so
        # allow one fp16 ulp; on these vectors the results are in fact identical
        y16 = orc.gemm_f16(*args).view(np.float16).astype(np.float64)
        r16 = z[k + "_y16"].view(np.float16).astype(np.float64)
        assert np.abs(y16 - r16).max() <= 2.0 ** -10 * max(1.0, np.abs(r16).max()), k
        # exact partial sums reproduce the fp64 product
        P = orc.group_partials(args[0], args[2])
        sx = (args[1].astype(np.uint32) << 16).view(np.float32).astype(np.float64).reshape(M, -1)
        sw = (args[3].astype(np.uint32) << 16).view(np.float32).astype(np.float64).reshape(N, -1)
        y_from_p = np.einsum("mng,mg,ng->mn", P.astype(np.float64), sx, sw)
        assert np.abs(y_from_p - ref64).max() <= 1e-12 * max(1.0, np.abs(ref64).max()), k


def test_per_tensor_golden(golden, orc):
    z = golden("per_tensor")
    for name in ("randn", "sweep"):
        inv = np.float32(1.0 / float(z[name + "_scale"]))
        assert np.array_equal(orc.quant_tensor_scale(z[name + "_x"], inv), z[name + "_q"]), name


def test_error_bound(orc):
    # reference tests/test_rtn_int4.py:22-32: |dequant - x| <= 6 * scale
    rng = np.random.default_rng(0)
    x = rng.standard_normal((512, 128)).astype(np.float32)
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)          # truncate to bf16
    xf = (xb.astype(np.uint32) << 16).view(np.float32)
    q, s = orc.quant_int4(xb)
    d = orc.dequant(q, s)
    scale = (s.astype(np.uint32) << 16).view(np.float32)
    err = np.abs(d - xf).reshape(512, 4, 32)
    assert (err <= 6.0 * scale[..., None]).all()
