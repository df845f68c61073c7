"""GPU parity tests: the CUDA path, called through the C ABI (tests/cabi.py) and through the
torch operator module, against the CPU oracle on identical seeded inputs.

Bars (from the hot-path contract):
  * quant_int4 and the EXACT fused op: codes and bf16 scale bit patterns identical;
  * FAST fused op: <= 1e-4 of the nibbles differ from the exact chain, each by +-1 only;
  * per-group int32 partial sums: identical;
  * products: ||y - y64||_F / ||y64||_F <= 1e-3 and max|y - y64| <= 1e-3 * max|y64| against the
    fp64 arbiter (fp16 output rounding alone is ~2.8e-4 rms).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3

if torch.cuda.is_available():
    from tests import cabi  # noqa: E402
    from wush_int4_kernel_b200 import capi  # noqa: E402


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    capi.check(capi.load().wush_init(), "wush_init")
    return torch.device("cuda:0")


def _bf16(a, dev):
    from oracle import w4a4_oracle as o

    return o.from_bits(a, torch.bfloat16).to(dev)


def _nibbles(q: np.ndarray) -> np.ndarray:
    lo = (q & 0xF).astype(np.int8)
    hi = (q >> 4).astype(np.int8)
    both = np.stack((lo, hi), -1).reshape(*q.shape[:-1], -1)
    return np.where(both > 7, both - 16, both)


# ------------------------------------------------------------------------------------------
# a1 quant_int4: bit exact
# ------------------------------------------------------------------------------------------
def _check_quant(x_bits, dev, orc, via_ops=False):
    x = _bf16(x_bits, dev)
    if via_ops:
        from my_int4 import _C
        q, s = _C.quant_int4(x)
    else:
        q, s = cabi.quant_int4(x)
    qo, so = orc.quant_int4(x_bits)
    assert q.shape == qo.shape and s.shape == so.shape
    assert np.array_equal(q.cpu().numpy(), qo)
    assert np.array_equal(orc.bits(s), so)


def test_quant_golden_cases(dev, orc, golden):
    z = golden("quant_int4")
    for name in z["names"]:
        _check_quant(z[f"{name}_x"], dev, orc)
        _check_quant(z[f"{name}_x"], dev, orc, via_ops=True)


def test_quant_random_and_stress(dev, orc):
    g = torch.Generator().manual_seed(0)
    cases = [torch.randn(4096, 32, generator=g), torch.randn(2, 3, 96, generator=g), torch.randn(1000, 64, generator=g),
             torch.randn(300, 160, generator=g) * torch.exp(3 * torch.randn(300, 160, generator=g)),
             torch.randn(1 << 17, 128, generator=g)]                      # 2^24 elements
    for c in cases:
        _check_quant(orc.bits(c.to(torch.bfloat16)), dev, orc)


def test_quant_empty(dev):
    from my_int4 import _C
    q, s = _C.quant_int4(torch.empty(0, 64, dtype=torch.bfloat16, device=dev))
    assert q.shape == (0, 32) and s.shape == (0, 2)


# ------------------------------------------------------------------------------------------
# a4..a7 fused transform + quantisation
# ------------------------------------------------------------------------------------------
def _wush_t(K, gen):
    from wush_int4_kernel_b200 import wush_transform as wt
    xc = torch.randn(256, K, generator=gen)
    xc[:, 5::32] *= 12.0
    w = torch.randn(64, K, generator=gen)
    return wt.compute_wush_transform(xc, w).to(torch.bfloat16)


def _fused_cases():
    g = torch.Generator().manual_seed(0)
    X = torch.randn(256, 128, generator=g).to(torch.bfloat16)
    X[:, 5::32] *= 12.0
    T = _wush_t(128, g)
    yield "wush-T", X, T
    yield "rand-T", X, torch.randn(4, 32, 32, generator=g).to(torch.bfloat16)
    yield "rank3", torch.randn(2, 3, 96, generator=g).to(torch.bfloat16), torch.randn(3, 32, 32, generator=g).to(torch.bfloat16)
    yield "zeros", torch.zeros(4, 64, dtype=torch.bfloat16), T[:2].contiguous()
    yield "odd-rows", torch.randn(37, 256, generator=g).to(torch.bfloat16), _wush_t(256, g)
    yield "one-row", torch.randn(1, 4096, generator=g).to(torch.bfloat16), _wush_t(4096, g)
    yield "stress", torch.randn(1 << 14, 64, generator=g).to(torch.bfloat16), T[:2].contiguous()


def test_fused_exact_bit_exact(dev, orc, golden):
    z = golden("fused_tq")
    for name in z["names"]:
        q, s = cabi.fused_tq(_bf16(z[f"{name}_x"], dev), _bf16(z[f"{name}_t"], dev), capi.TQ_EXACT)
        assert np.array_equal(q.cpu().numpy(), z[f"{name}_q"]), name
        assert np.array_equal(orc.bits(s), z[f"{name}_s"]), name
    for name, X, T in _fused_cases():
        q, s = cabi.fused_tq(X.to(dev), T.to(dev), capi.TQ_EXACT)
        qo, so = orc.fused_tq(orc.bits(X), orc.bits(T))
        assert np.array_equal(q.cpu().numpy(), qo), name
        assert np.array_equal(orc.bits(s), so), name


def test_fused_fast_flip_rate(dev, orc):
    total = flips = big = scale_mismatch = groups = 0
    for name, X, T in _fused_cases():
        q, s = cabi.fused_tq(X.to(dev), T.to(dev), capi.TQ_FAST)
        qo, so = orc.fused_tq(orc.bits(X), orc.bits(T))
        d = _nibbles(q.cpu().numpy()).astype(np.int32) - _nibbles(qo).astype(np.int32)
        total += d.size
        flips += int((d != 0).sum())
        big += int((np.abs(d) > 1).sum())
        sm = orc.bits(s).astype(np.int32) - so.astype(np.int32)
        scale_mismatch += int((sm != 0).sum())
        groups += sm.size
        assert np.abs(sm).max(initial=0) <= 1, name           # at most one bf16 ulp
    assert big == 0
    assert flips <= 1e-4 * total, (flips, total)
    assert scale_mismatch <= 2e-3 * groups, (scale_mismatch, groups)


def test_fused_names_and_shapes(dev, orc):
    from my_int4 import _C
    g = torch.Generator().manual_seed(1)
    X = torch.randn(2, 5, 128, generator=g).to(torch.bfloat16).to(dev)
    T = torch.randn(4, 32, 32, generator=g).to(torch.bfloat16).to(dev)
    qe, se = _C.fused_transform_quant_int4(X, T)
    assert qe.shape == (2, 5, 64) and se.shape == (2, 5, 4) and qe.dtype == torch.uint8 and se.dtype == torch.bfloat16
    qo, so = orc.fused_tq(orc.bits(X), orc.bits(T))
    assert np.array_equal(qe.cpu().numpy(), qo)
    for fn in (_C.fused_transform_quant_int4_wmma, _C.fused_transform_quant_int4_v3, _C.fused_transform_quant_int4_smallm):
        q, s = fn(X, T)
        assert q.shape == qe.shape and s.shape == se.shape
        assert (q != qe).float().mean().item() < 1e-2
    with pytest.raises(RuntimeError):
        _C.fused_transform_quant_int4(X, T[:3].contiguous())
    with pytest.raises(RuntimeError):
        _C.fused_transform_quant_int4(X.float(), T)


# ------------------------------------------------------------------------------------------
# a8..a10 products
# ------------------------------------------------------------------------------------------
def _operands(M, N, K, seed, orc):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(M, K, generator=g).to(torch.bfloat16)
    W = torch.randn(N, K, generator=g).to(torch.bfloat16)
    xq, xs = orc.quant_int4(orc.bits(X))
    wq, ws = orc.quant_int4(orc.bits(W))
    return xq, xs, wq, ws


def _to_dev(dev, xq, xs, wq, ws):
    return (torch.from_numpy(xq).to(dev), _bf16(xs, dev), torch.from_numpy(wq).to(dev), _bf16(ws, dev))


def _assert_close(y: torch.Tensor, y64: np.ndarray, tag):
    yd = y.double().cpu().numpy().reshape(y64.shape)
    ref = max(np.linalg.norm(y64), 1e-30)
    rel = np.linalg.norm(yd - y64) / ref
    mx = np.abs(yd - y64).max() / max(np.abs(y64).max(), 1e-30)
    assert rel <= REL_TOL, (tag, "frobenius", rel)
    assert mx <= REL_TOL, (tag, "max", mx)


TILE_SHAPES = [(128, 128, 256), (256, 384, 512), (300, 504, 512), (130, 512, 4096), (33, 64, 256), (129, 8, 256),
               (1000, 1000, 1024), (512, 4096, 4096), (2100, 264, 512), (200, 520, 8192), (300, 1000, 4096), (100, 520, 8192)]


@pytest.mark.parametrize("shape", TILE_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_tile_tcgen05_vs_fp64(dev, orc, shape):
    M, N, K = shape
    ops = _operands(M, N, K, seed=M + 3 * N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    y = cabi.gemm(*_to_dev(dev, *ops), variant=capi.GEMM_TILE)
    _assert_close(y, y64, shape)
    y2 = cabi.gemm(*_to_dev(dev, *ops), variant=capi.GEMM_DECODE)       # streaming kernel on the same data
    _assert_close(y2, y64, shape)
    y3 = cabi.gemm(*_to_dev(dev, *ops), variant=capi.GEMM_TILE_F16)     # scales folded into fp16 operands
    _assert_close(y3, y64, shape)


@pytest.mark.parametrize("shape", [(8, 264, 8192), (32, 1000, 8192), (20, 2048, 2048), (5, 520, 1024), (70, 776, 4096)],
                         ids=lambda s: "x".join(map(str, s)))
def test_decode_split_k_vs_fp64(dev, orc, shape):
    """Narrow layers: the streaming kernel splits K over a cluster of 8 / 8 / 2 / 1 / 4 CTAs and sums
    the partial results through distributed shared memory; ragged rows and row blocks included."""
    M, N, K = shape
    ops = _operands(M, N, K, seed=7 * M + N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    y = cabi.gemm(*_to_dev(dev, *ops), variant=capi.GEMM_DECODE)
    _assert_close(y, y64, shape)
    y2 = cabi.gemm(*_to_dev(dev, *ops), variant=capi.GEMM_DECODE)
    assert torch.equal(y, y2)                                              # fixed summation order


DECODE_TC_SHAPES = [(1, 128, 256), (5, 264, 256), (8, 264, 8192), (16, 1000, 2048), (17, 520, 1024), (32, 1000, 8192),
                    (32, 4096, 4096), (20, 19072, 512), (31, 776, 4096), (24, 2048, 2048), (9, 8, 256), (12, 130, 7168)]


@pytest.mark.parametrize("shape", DECODE_TC_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_decode_tcgen05_swapped_vs_fp64(dev, orc, shape):
    """The tcgen05 decode kernel (weights as the 128-row operand, 16 / 32 activation columns): ragged
    activation rows and weight rows, one stage per tile up to 32, tiles split over several CTAs (narrow
    layers: every tile is split) and unsplit ones, against the fp64 arbiter and against the streaming
    kernel on the same operands; repeatable bit for bit (the pieces of a split tile are added in K order)."""
    M, N, K = shape
    ops = _operands(M, N, K, seed=11 * M + N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    dops = _to_dev(dev, *ops)
    y = cabi.gemm(*dops, variant=capi.GEMM_DECODE_TC)
    _assert_close(y, y64, shape)
    y2 = cabi.gemm(*dops, variant=capi.GEMM_DECODE_TC)
    assert torch.equal(y, y2)
    y_stream = cabi.gemm(*dops, variant=capi.GEMM_DECODE)
    assert (y.float() - y_stream.float()).abs().max().item() <= 2e-3 * max(np.abs(y64).max(), 1e-30)


@pytest.mark.parametrize("shape", [(2100, 264, 512), (2304, 520, 1024), (300, 1000, 320)], ids=lambda s: "x".join(map(str, s)))
def test_pair_tile_kernel_equals_single_cta_kernel(dev, orc, shape, monkeypatch):
    """The pre-widened fp16-folded route on CTA pairs (tcgen05 cta_group::2: each CTA holds 128 activation rows
    and half of the weight rows of a 256 x 256 tile) against the single-CTA tile kernel: same operands, same
    accumulation order over K, so the results must agree bit for bit -- and with the fp64 arbiter."""
    M, N, K = shape
    ops = _operands(M, N, K, seed=M + N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    dops = _to_dev(dev, *ops)
    monkeypatch.setenv("WUSH_TAIL_SPLIT", "0")        # the single-CTA kernel otherwise sums the last wave's tiles in K ranges
    monkeypatch.setenv("WUSH_TILE_KERNEL", "pair")
    y_pair = cabi.gemm(*dops, variant=capi.GEMM_TILE_F16)
    monkeypatch.setenv("WUSH_TILE_KERNEL", "single")
    y_single = cabi.gemm(*dops, variant=capi.GEMM_TILE_F16)
    _assert_close(y_pair, y64, shape)
    assert torch.equal(y_pair, y_single)


@pytest.mark.parametrize("mode", ["1", "2"])
@pytest.mark.parametrize("shape", [(2100, 264, 512), (2304, 2048, 1024), (4096, 1536, 2048), (2100, 9472, 256),
                                   (260, 4096, 2048), (520, 2048, 4096), (300, 520, 1024)])
def test_last_wave_in_k_ranges(dev, orc, shape, mode, monkeypatch):
    """The tiles of the last, partly filled wave are cut along K and summed afterwards: mode 1 = equal ranges that
    fit one round, mode 2 = their stages dealt to all CTAs as contiguous runs (a run may end one tile and begin the
    next).  Both tile kernels (weights pre-widened: M > 2048; widened in the kernel: M <= 2048), forced by the
    environment switch where the mode applies at all.  Against the fp64 arbiter, and against the same product
    without the cut: the operands' products are exact in fp32, only the order of the additions differs."""
    M, N, K = shape
    ops = _operands(M, N, K, seed=M + K, orc=orc)
    dops = _to_dev(dev, *ops)
    monkeypatch.setenv("WUSH_TILE_KERNEL", "single")
    monkeypatch.setenv("WUSH_TAIL_SPLIT", mode)
    y_cut = cabi.gemm(*dops, variant=capi.GEMM_TILE_F16)
    monkeypatch.setenv("WUSH_TAIL_SPLIT", "0")
    y_whole = cabi.gemm(*dops, variant=capi.GEMM_TILE_F16)
    if M * N * K <= 2304 * 2048 * 1024:
        _assert_close(y_cut, orc.gemm_f64(*ops), shape)
    d = (y_cut.float() - y_whole.float()).abs()
    assert float(d.max()) <= 2e-3 * float(y_whole.float().abs().max())
    assert float((d > 0).float().mean()) < 0.2


@pytest.mark.parametrize("M,N,K", [(2100, 264, 512), (2100, 512, 512), (256, 520, 512), (130, 264, 320), (300, 512, 1024)])
def test_output_and_scratch_on_16_byte_boundaries(M, N, K):
    """The tile kernels and their pre-passes store 32 bytes per lane where the addresses allow it.  A caller may
    hand over an output and a scratch that are only 16-byte aligned, and N need not be a multiple of 16: the
    result must be the same bit for bit as with 256-byte-aligned buffers."""
    from tests import cabi
    from wush_int4_kernel_b200 import capi
    gen = torch.Generator(device="cuda").manual_seed(77)
    xq = torch.randint(0, 256, (M, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    wq = torch.randint(0, 256, (N, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    xs = (0.02 * (1 + torch.rand(M, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    ws = (0.01 * (1 + torch.rand(N, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    for variant in (capi.GEMM_AUTO, capi.GEMM_TILE_F16):
        want = cabi.gemm(xq, xs, wq, ws, variant)
        got = cabi.gemm(xq, xs, wq, ws, variant, misalign=16)
        assert torch.equal(got, want), variant
    y_ts, _, flag = cabi.gemm_ts_ws(xq, wq, 0.001)
    assert flag == 0 and torch.equal(y_ts, cabi.gemm_ts(xq, wq, 0.001))
