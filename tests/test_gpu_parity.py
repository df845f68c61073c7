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
                                   (260, 4096, 2048), (520, 2048, 4096), (300, 520, 1024),
                                   (100, 19456, 512), (100, 38400, 512)])      # the 128-row kernel: 76 and 150 tiles
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


def test_decode_tcgen05_exact_group_sums(dev, orc):
    """One group per row with unit scales: the fp16 result IS the integer group sum (|P| <= 2048 is exact
    in fp16), so the tensor-core path's per-group sums are checked exactly -- including code -8."""
    M, N, K = 32, 256, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    xq = torch.randint(0, 256, (M, K // 2), generator=g, device=dev, dtype=torch.uint8)
    wq = torch.randint(0, 256, (N, K // 2), generator=g, device=dev, dtype=torch.uint8)
    # only group 0 carries a non-zero scale: Y = P_0
    xs = torch.zeros(M, K // 32, dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(N, K // 32, dtype=torch.bfloat16, device=dev)
    for grp in range(K // 32):
        xs.zero_(); ws.zero_()
        xs[:, grp] = 1.0
        ws[:, grp] = 1.0
        y = cabi.gemm(xq, xs, wq, ws, variant=capi.GEMM_DECODE_TC)
        P = orc.group_partials(xq.cpu().numpy(), wq.cpu().numpy())[:, :, grp]
        assert np.array_equal(y.float().cpu().numpy(), P.astype(np.float32)), grp


def test_decode_tcgen05_needs_scratch(dev):
    """The explicit variant refuses to run without its scratch; AUTO (the streaming kernel here) needs none."""
    lib = capi.load()
    M, N, K = 8, 512, 1024
    z = torch.zeros(N * K // 2, dtype=torch.uint8, device=dev)
    s = torch.zeros(N * K // 32, dtype=torch.bfloat16, device=dev)
    y = torch.empty(M, N, dtype=torch.float16, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.wush_w4a4_gemm_workspace_bytes(M, N, K, capi.GEMM_DECODE_TC) > 256
    assert lib.wush_w4a4_gemm(z.data_ptr(), s.data_ptr(), z.data_ptr(), s.data_ptr(), M, N, K, y.data_ptr(),
                              capi.GEMM_DECODE_TC, None, 0, st) == capi.WUSH_ERR_WORKSPACE
    assert lib.wush_w4a4_gemm(z.data_ptr(), s.data_ptr(), z.data_ptr(), s.data_ptr(), M, N, K, y.data_ptr(),
                              capi.GEMM_AUTO, None, 0, st) == capi.WUSH_OK
    torch.cuda.synchronize()
    assert (y == 0).all()


def test_auto_variant_by_shape(dev):
    """What AUTO stands for: the GEMV for up to three rows (four on all but the widest layers), the streaming kernel for decode batches and for
    mid-size M on narrow layers, the fp16 route where its tiles (or K ranges) fill the machine."""
    lib = capi.load()
    pick = lib.wush_w4a4_gemm_pick_variant
    assert pick(1, 57344, 8192) == capi.GEMM_GEMV and pick(2, 8192, 8192) == capi.GEMM_GEMV
    assert pick(4, 57344, 8192) == capi.GEMM_DECODE and pick(4, 8192, 8192) == capi.GEMM_GEMV
    assert pick(3, 57344, 8192) == capi.GEMM_GEMV and pick(4, 24576, 4096) == capi.GEMM_GEMV
    assert pick(16, 57344, 8192) == capi.GEMM_DECODE and pick(32, 24576, 4096) == capi.GEMM_DECODE
    assert pick(64, 8192, 8192) == capi.GEMM_DECODE and pick(128, 8192, 3584) == capi.GEMM_DECODE
    assert pick(128, 57344, 8192) == capi.GEMM_TILE_F16 and pick(256, 8192, 8192) == capi.GEMM_TILE_F16
    assert pick(4096, 57344, 8192) == capi.GEMM_TILE_F16
    assert pick(48, 64, 96) == capi.GEMM_DECODE                   # K no tile kernel takes: the generic decode path
    for shape in [(1, 64, 64), (300, 1000, 4096), (96, 24576, 4096)]:
        v = pick(*shape)
        assert lib.wush_w4a4_gemm_workspace_bytes(*shape, capi.GEMM_AUTO) == lib.wush_w4a4_gemm_workspace_bytes(*shape, v)


def test_f16_route_wide_scale_range(dev, orc):
    """Rows whose group scales span many octaves (and exact-zero groups) through the fp16-folded route."""
    g = torch.Generator().manual_seed(5)
    M, N, K = 160, 264, 512
    X = (torch.randn(M, K, generator=g) * torch.exp2(torch.randint(-12, 8, (M, K // 32), generator=g).float()).repeat_interleave(32, 1))
    W = (torch.randn(N, K, generator=g) * torch.exp2(torch.randint(-14, 2, (N, K // 32), generator=g).float()).repeat_interleave(32, 1))
    X[3] = 0
    W[:, 64:96] = 0
    xq, xs = orc.quant_int4(orc.bits(X.to(torch.bfloat16)))
    wq, ws = orc.quant_int4(orc.bits(W.to(torch.bfloat16)))
    y64 = orc.gemm_f64(xq, xs, wq, ws)
    y = cabi.gemm(*_to_dev(dev, xq, xs, wq, ws), variant=capi.GEMM_TILE_F16)
    assert torch.isfinite(y.float()).all()
    _assert_close(y, y64, "wide")
    assert (y[3] == 0).all()


SHAPES = [(64, 96, 128), (1, 64, 64), (300, 500, 512), (130, 512, 4096), (8, 4096, 4096),   # reference tests/test_p13.py:18
          (257, 33, 96), (8, 8, 32), (4, 100, 256), (2, 77, 512), (3, 64, 96), (17, 130, 768), (32, 256, 1024),
          (5, 129, 256), (33, 64, 256)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_auto_vs_fp64(dev, orc, shape):
    M, N, K = shape
    ops = _operands(M, N, K, seed=M * 7 + N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    y = cabi.gemm(*_to_dev(dev, *ops))
    _assert_close(y, y64, shape)


def test_gemm_every_variant(dev, orc):
    for (M, N, K) in [(1, 200, 512), (4, 130, 256), (3, 64, 96)]:
        ops = _operands(M, N, K, seed=11, orc=orc)
        y64 = orc.gemm_f64(*ops)
        d = _to_dev(dev, *ops)
        for v in (capi.GEMM_GEMV, capi.GEMM_DECODE, capi.GEMM_TILE, capi.GEMM_AUTO):
            _assert_close(cabi.gemm(*d, variant=v), y64, (M, N, K, v))
    for (M, N, K) in [(16, 300, 512), (32, 128, 256), (100, 260, 768)]:
        ops = _operands(M, N, K, seed=12, orc=orc)
        y64 = orc.gemm_f64(*ops)
        d = _to_dev(dev, *ops)
        for v in (capi.GEMM_DECODE, capi.GEMM_TILE, capi.GEMM_AUTO):
            _assert_close(cabi.gemm(*d, variant=v), y64, (M, N, K, v))
    with pytest.raises(capi.WushError):
        cabi.gemm(*_to_dev(dev, *_operands(8, 16, 64, 1, orc)), variant=capi.GEMM_GEMV)


@pytest.mark.parametrize("shape", [(1, 77, 8192), (2, 130, 8192), (3, 67, 28672), (4, 50, 2048), (2, 33, 1024), (3, 20, 4096),
                                   (4, 9, 320), (1, 5, 12288)], ids=lambda s: "x".join(map(str, s)))
def test_gemv_rows_per_trip(dev, orc, shape, monkeypatch):
    """The GEMV takes two or four weight rows per trip and reloads a slot as soon as it is consumed: rows that
    end inside a unit, rows of one, several and a fractional number of trips, and both row counts -- which add
    every row's groups in the same order, so their results are the same bits."""
    M, N, K = shape
    ops = _operands(M, N, K, seed=3 * M + N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    d = _to_dev(dev, *ops)
    ys = []
    for rows in ("2", "4"):
        monkeypatch.setenv("WUSH_GEMV_ROWS", rows)
        ys.append(cabi.gemm(*d, variant=capi.GEMM_GEMV))
        _assert_close(ys[-1], y64, (shape, rows))
    assert torch.equal(ys[0], ys[1])


GEMV_MMA_SHAPES = [(1, 16, 512), (2, 77, 128), (3, 130, 1152), (4, 50, 2048), (5, 264, 640), (6, 33, 4096), (7, 1000, 1024),
                   (8, 264, 8192), (8, 2400, 512), (9, 40, 1024), (12, 520, 2048), (13, 17, 4096), (16, 300, 8192), (16, 5000, 512)]


@pytest.mark.parametrize("shape", GEMV_MMA_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemv_mma_vs_fp64(dev, orc, shape):
    """Weights streamed straight into mma.sync fragments (variant GEMV_MMA): every chain count (M = 1..16, odd M
    padded with a zero row), row blocks that end inside a unit of 16, one to sixteen ring rounds per row, more
    units than resident warps (several units per warp, loads crossing from one unit to the next)."""
    M, N, K = shape
    ops = _operands(M, N, K, seed=5 * M + N, orc=orc)
    y64 = orc.gemm_f64(*ops)
    y = cabi.gemm(*_to_dev(dev, *ops), variant=capi.GEMM_GEMV_MMA)
    _assert_close(y, y64, shape)


def test_gemv_mma_exact_against_streaming_kernel(dev, orc):
    """Group sums are exact integers in both kernels and both apply the scales with the same two FMAs; only the
    order in which a row's groups are added differs, so the results agree to fp32 summation order -- and zero rows
    of activations give exact zeros."""
    M, N, K = 8, 520, 2048
    xq, xs, wq, ws = _operands(M, N, K, seed=21, orc=orc)
    xq = xq.copy()
    xq[3] = 0
    d = _to_dev(dev, xq, xs, wq, ws)
    a = cabi.gemm(*d, variant=capi.GEMM_GEMV_MMA).float()
    b = cabi.gemm(*d, variant=capi.GEMM_DECODE).float()
    assert (a[3] == 0).all()
    assert (a - b).abs().max() <= 2e-3 * b.abs().max()
    with pytest.raises(capi.WushError):
        cabi.gemm(*_to_dev(dev, *_operands(4, 16, 96, 1, orc)), variant=capi.GEMM_GEMV_MMA)      # K not a multiple of 128
    with pytest.raises(capi.WushError):
        cabi.gemm(*_to_dev(dev, *_operands(17, 16, 512, 1, orc)), variant=capi.GEMM_GEMV_MMA)    # more than 16 rows


def test_gemm_golden(dev, orc, golden):
    z = golden("w4a4_matmul")
    for (M, N, K) in z["shapes"]:
        k = f"{M}x{N}x{K}"
        d = _to_dev(dev, z[k + "_xq"], z[k + "_xs"], z[k + "_wq"], z[k + "_ws"])
        _assert_close(cabi.gemm(*d), z[k + "_y64"], k)


def test_zero_activations_give_exact_zero(dev, orc):
    # reference tests/test_s3.py:43-48
    g = torch.Generator().manual_seed(0)
    for M, N, K in [(4, 16, 64), (1, 64, 256), (16, 128, 256), (40, 130, 512)]:
        xq, xs = orc.quant_int4(np.zeros((M, K), np.uint16))
        wq, ws = orc.quant_int4(orc.bits(torch.randn(N, K, generator=g).to(torch.bfloat16)))
        y = cabi.gemm(*_to_dev(dev, xq, xs, wq, ws))
        assert (y == 0).all()


def test_code_minus_eight_is_sign_extended(dev, orc):
    # the sigma path never emits -8, but consumers must handle it (reference tests/test_s4c.py:13)
    rng = np.random.default_rng(0)
    for M, N, K in [(1, 64, 128), (8, 64, 256), (40, 64, 256)]:
        xq = rng.integers(0, 256, (M, K // 2), dtype=np.uint8)
        wq = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
        ones = np.full((M, K // 32), 0x3F80, np.uint16)
        onesw = np.full((N, K // 32), 0x3F80, np.uint16)
        y64 = orc.gemm_f64(xq, ones, wq, onesw)
        _assert_close(cabi.gemm(*_to_dev(dev, xq, ones, wq, onesw)), y64, (M, N, K))
        P = cabi.group_partials(torch.from_numpy(xq).to(dev), torch.from_numpy(wq).to(dev))
        assert np.array_equal(P.cpu().numpy(), orc.group_partials(xq, wq))


def test_group_partials_exact(dev, orc):
    # the last three shapes run on the tcgen05 tile path (M > 32, K % 256 == 0, N % 8 == 0)
    for (M, N, K) in [(8, 16, 64), (33, 130, 256), (5, 64, 1024), (64, 96, 128), (130, 136, 512), (128, 256, 256),
                      (200, 72, 768)]:
        xq, _, wq, _ = _operands(M, N, K, seed=5, orc=orc)
        P = cabi.group_partials(torch.from_numpy(xq).to(dev), torch.from_numpy(wq).to(dev))
        assert np.array_equal(P.cpu().numpy(), orc.group_partials(xq, wq)), (M, N, K)


def test_atom_selftest(dev):
    rng = np.random.default_rng(1)
    a = rng.integers(-8, 8, (8, 32), dtype=np.int8)
    b = rng.integers(-8, 8, (32, 8), dtype=np.int8)
    c = cabi.atom(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev))
    assert np.array_equal(c.cpu().numpy(), a.astype(np.int32) @ b.astype(np.int32))
    from my_int4 import _C
    c2 = _C.s4_atom_selftest(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev))
    assert np.array_equal(c2.cpu().numpy(), a.astype(np.int32) @ b.astype(np.int32))


def test_operator_shapes_and_errors(dev, orc):
    from my_int4 import _C
    ops = _operands(6, 40, 128, seed=3, orc=orc)
    xq, xs, wq, ws = _to_dev(dev, *ops)
    y64 = orc.gemm_f64(*ops)
    y = _C.w4a4_gemm(xq.reshape(2, 3, -1), xs.reshape(2, 3, -1), wq, ws)
    assert y.shape == (2, 3, 40) and y.dtype == torch.float16        # v0 keeps leading dims
    _assert_close(y, y64, "v0")
    for fn in (_C.w4a4_gemm_v1, _C.w4a4_gemm_v2, _C.w4a4_gemm_s4, _C.w4a4_gemv_multi):
        y = fn(xq.reshape(2, 3, -1), xs.reshape(2, 3, -1), wq, ws)
        assert y.shape == (6, 40)
        _assert_close(y, y64, fn.__name__)
    y1 = _C.w4a4_gemv(xq[:1], xs[:1], wq, ws)
    assert y1.shape == (40,)
    _assert_close(y1, y64[:1], "gemv")
    with pytest.raises(RuntimeError):
        _C.w4a4_gemv(xq, xs, wq, ws)                                   # more than one row
    with pytest.raises(RuntimeError):
        _C.w4a4_gemm_s4(xq, xs, wq[:, :32].contiguous(), ws)           # K mismatch
    with pytest.raises(RuntimeError):
        _C.w4a4_gemm_s4(xq, xs.float(), wq, ws)                        # wrong scale dtype
    big = _operands(33, 16, 64, seed=4, orc=orc)
    with pytest.raises(RuntimeError):
        _C.w4a4_gemv_multi(*_to_dev(dev, *big))                        # more than 32 rows


# ------------------------------------------------------------------------------------------
# per-tensor route
# ------------------------------------------------------------------------------------------
def test_per_tensor_route(dev, orc, golden):
    from my_int4 import _C
    z = golden("per_tensor")
    for name in ("randn", "sweep"):
        x = _bf16(z[name + "_x"], dev)
        scale = float(z[name + "_scale"])
        q = _C.quant_int4_tensor_scale(x, scale)
        assert q.dim() == 1 and np.array_equal(q.cpu().numpy(), z[name + "_q"]), name
        inv = torch.tensor([1.0 / scale], dtype=torch.float32, device=dev)
        q2 = _C.quant_int4_tensor_scale_dev(x, inv)
        assert torch.equal(q, q2)
    rng = np.random.default_rng(2)
    for (M, N, K) in [(64, 96, 128), (1, 64, 256), (30, 50, 512)]:
        xq = rng.integers(0, 256, (M, K // 2), dtype=np.uint8)
        wq = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
        alpha = 0.0123
        yo, _ = orc.gemm_tensor_scale(xq, wq, alpha)
        y = _C.w4a4_gemm_cutlass(torch.from_numpy(xq).to(dev), torch.from_numpy(wq).to(dev), alpha)
        assert y.shape == (M, N) and np.array_equal(orc.bits(y), yo), (M, N, K)
        a = torch.tensor([alpha], dtype=torch.float32, device=dev)
        y2 = _C.w4a4_gemm_cutlass_dev(torch.from_numpy(xq).reshape(-1).to(dev), torch.from_numpy(wq).to(dev), a)
        assert torch.equal(y, y2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (200, 264, 384), (512, 1000, 1024), (4096, 4096, 4096)])
def test_per_tensor_tile_route(dev, orc, M, N, K):
    """tcgen05 kind::i8 tiles for the per-tensor product: same bits as the scratch-free kernel
    (and as the oracle where the oracle finishes quickly), error word clean."""
    from tests import cabi
    gen = torch.Generator(device=dev).manual_seed(M + N + K)
    xq = torch.randint(0, 256, (M, K // 2), generator=gen, device=dev, dtype=torch.uint8)
    wq = torch.randint(0, 256, (N, K // 2), generator=gen, device=dev, dtype=torch.uint8)
    alpha = 3.1e-4
    y, nbytes, flag = cabi.gemm_ts_ws(xq, wq, alpha)
    assert nbytes > 0 and flag == 0
    assert torch.equal(y, cabi.gemm_ts(xq, wq, alpha))
    a = torch.tensor([alpha], dtype=torch.float32, device=dev)
    y2, _, flag2 = cabi.gemm_ts_ws(xq, wq, 0.0, a)
    assert flag2 == 0 and torch.equal(y, y2)
    if M * N * K <= 1 << 28:
        yo, _ = orc.gemm_tensor_scale(xq.cpu().numpy(), wq.cpu().numpy(), alpha)
        assert np.array_equal(orc.bits(y), yo)
    # the binding allocates the scratch itself
    from my_int4 import _C
    assert torch.equal(_C.w4a4_gemm_cutlass(xq, wq, alpha), y)


# ------------------------------------------------------------------------------------------
# CUDA Graph safety (reference tests/test_p13.py:45-66, tests/test_p12.py:142-152)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M", [1, 8, 48])
def test_graph_replay_equals_eager(dev, M):
    from my_int4 import _C
    from wush_int4_kernel_b200 import synth
    from wush_int4_kernel_b200.linear import W4A4Linear

    _C.init()
    layer = synth.make_layer(512, 384, seed=2, device="cuda", quantiser=_C.quant_int4)
    lin = W4A4Linear(layer.t_bf16, layer.wq, layer.ws)
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = synth.draw_activations(M, 512, layer.outliers, gen)
    y0 = lin(x).clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            lin(x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = lin(x)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, y0)                     # deterministic kernels: bit identical
    x.copy_(synth.draw_activations(M, 512, layer.outliers, gen))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, lin(x))


# ------------------------------------------------------------------------------------------
# the reference's end-to-end accuracy gate on outlier data (tests/test_p13.py:29-43)
# ------------------------------------------------------------------------------------------
def test_end_to_end_outlier_gate(dev):
    from my_int4 import _C
    from my_int4.wush_transform import compute_wush_transform, transform_weights

    torch.manual_seed(0)
    M, N, K, G = 2048, 512, 4096, 32
    X = torch.randn(M, K, dtype=torch.bfloat16, device=dev)
    X[:, 5::G] *= 15.0
    W = torch.randn(N, K, dtype=torch.bfloat16, device=dev)
    W[:, 12::G] *= 8.0
    Yt = X.double() @ W.double().t()
    Xc = torch.randn(256, K, device=dev)
    Xc[:, 5::G] *= 15.0
    T64 = compute_wush_transform(Xc, W.float(), group_size=G)
    Ww = transform_weights(W.double(), T64).to(torch.bfloat16).contiguous()
    wq, ws = _C.quant_int4(Ww)
    xq, xs = _C.fused_transform_quant_int4_v3(X, T64.to(torch.bfloat16))
    err = ((_C.w4a4_gemm_s4(xq, xs, wq, ws).double() - Yt).norm() / Yt.norm()).item()
    assert err <= 0.082, err
    xq0, xs0 = _C.quant_int4(X)
    wq0, ws0 = _C.quant_int4(W)
    bare = ((_C.w4a4_gemm_s4(xq0, xs0, wq0, ws0).double() - Yt).norm() / Yt.norm()).item()
    assert bare > 0.3                                # the transform is what brings 53 % down to 7.8 %


# ------------------------------------------------------------------------------------------
# full benchmark sizes: size-independent properties instead of a full CPU product
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("K,N", [(4096, 24576), (8192, 57344)])
@pytest.mark.parametrize("M", [1, 8, 32])
def test_full_size_decode_sampled_columns(dev, orc, K, N, M):
    """Random weights at the benchmark shapes; a seeded sample of output columns must agree
    with the oracle, a zeroed activation row must give an exactly zero output row, and a
    permutation of the weight rows must permute the output columns bit for bit."""
    g = torch.Generator(device="cuda").manual_seed(K + M)
    wq = torch.randint(0, 256, (N, K // 2), generator=g, device=dev, dtype=torch.uint8)
    ws = (0.01 * (1 + 0.2 * torch.rand(N, K // 32, generator=g, device=dev))).to(torch.bfloat16)
    xq = torch.randint(0, 256, (M, K // 2), generator=g, device=dev, dtype=torch.uint8)
    xs = (0.5 * (1 + torch.rand(M, K // 32, generator=g, device=dev))).to(torch.bfloat16)
    if M > 1:
        xq[M - 1].zero_()
    y = cabi.gemm(xq, xs, wq, ws)
    cols = torch.randperm(N, generator=g, device=dev)[:256].sort().values
    y64 = orc.gemm_f64(xq.cpu().numpy(), orc.bits(xs), wq[cols].cpu().numpy(), orc.bits(ws[cols]))
    _assert_close(y[:, cols], y64, (M, N, K))
    if M > 1:
        assert (y[M - 1] == 0).all()
    perm = torch.randperm(N, generator=g, device=dev)
    y_perm = cabi.gemm(xq, xs, wq[perm].contiguous(), ws[perm].contiguous())
    assert torch.equal(y_perm, y[:, perm])


def test_full_size_prefill_sampled(dev, orc):
    K, N, M = 8192, 57344, 512
    g = torch.Generator(device="cuda").manual_seed(9)
    wq = torch.randint(0, 256, (N, K // 2), generator=g, device=dev, dtype=torch.uint8)
    ws = (0.01 * (1 + 0.2 * torch.rand(N, K // 32, generator=g, device=dev))).to(torch.bfloat16)
    xq = torch.randint(0, 256, (M, K // 2), generator=g, device=dev, dtype=torch.uint8)
    xs = (0.5 * (1 + torch.rand(M, K // 32, generator=g, device=dev))).to(torch.bfloat16)
    y = cabi.gemm(xq, xs, wq, ws)
    cols = torch.randperm(N, generator=g, device=dev)[:64].sort().values
    rows = torch.randperm(M, generator=g, device=dev)[:64].sort().values
    y64 = orc.gemm_f64(xq[rows].cpu().numpy(), orc.bits(xs[rows]), wq[cols].cpu().numpy(), orc.bits(ws[cols]))
    _assert_close(y[rows][:, cols], y64, "prefill")


def test_full_size_fused_tq_roundtrip(dev, orc):
    """M=4096, K=8192 activations: FAST vs EXACT flip rate at full size, and EXACT vs the
    oracle on a sample of rows."""
    from wush_int4_kernel_b200 import synth
    from my_int4 import _C
    layer = synth.make_layer(8192, 256, seed=4, device="cuda", quantiser=_C.quant_int4)
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = synth.draw_activations(4096, 8192, layer.outliers, gen)
    qe, se = cabi.fused_tq(x, layer.t_bf16, capi.TQ_EXACT)
    qf, sf = cabi.fused_tq(x, layer.t_bf16, capi.TQ_FAST)
    ne, nf = _nibbles(qe.cpu().numpy()).astype(np.int32), _nibbles(qf.cpu().numpy()).astype(np.int32)
    d = ne - nf
    assert np.abs(d).max() <= 1 and (d != 0).mean() <= 1e-4
    rows = torch.arange(0, 4096, 257, device=dev)
    qo, so = orc.fused_tq(orc.bits(x[rows]), orc.bits(layer.t_bf16))
    assert np.array_equal(qe[rows].cpu().numpy(), qo) and np.array_equal(orc.bits(se[rows]), so)


# ------------------------------------------------------------------------------------------
# tcgen05 plumbing: one kind::i8 instruction tile (descriptor / TMEM / tcgen05.ld mapping)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [16, 64, 128, 256])
def test_tcgen05_i8_tile(dev, n):
    rng = np.random.default_rng(n)
    a = rng.integers(-128, 128, (128, 32), dtype=np.int8)
    b = rng.integers(-128, 128, (n, 32), dtype=np.int8)
    d, status = cabi.tile_selftest(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev))
    assert status == 0, "bounded wait on the MMA barrier gave up"
    assert np.array_equal(d.cpu().numpy(), a.astype(np.int32) @ b.astype(np.int32).T)


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
