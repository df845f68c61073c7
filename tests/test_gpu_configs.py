"""GPU parity tests at the benchmark configurations themselves (sizes, value distributions and
entry points the throughput figures are quoted on), against the CPU oracle and its fp64 arbiter.

A full CPU product at these sizes would take minutes, so the large shapes are checked on a
seeded sample of rows x columns plus size-independent properties (an all-zero activation row gives
an exactly zero output row; the kernels' error word stays clear).  Tolerances follow the hot-path
contract: codes and scales bit-exact, products within 1e-3 (Frobenius and max) of the fp64 result.
The reference gates its GEMM the same way, against an fp64 product of the dequantised operands
(tests/test_p13.py:17-27 of the reference), with the looser bound 0.05 * max|y64|.
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


def _close(y, y64, tag):
    yd = y.double().cpu().numpy().reshape(y64.shape)
    rel = np.linalg.norm(yd - y64) / max(np.linalg.norm(y64), 1e-30)
    mx = np.abs(yd - y64).max() / max(np.abs(y64).max(), 1e-30)
    assert rel <= REL_TOL, (tag, "frobenius", rel)
    assert mx <= REL_TOL, (tag, "max", mx)


def _random_operands(M, N, K, seed, dev):
    """Uniform random codes (every nibble value, -8 included) and scales spread over a factor of two
    (weights) / two (activations): what the large-shape tests of the decode family use as well."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    wq = torch.randint(0, 256, (N, K // 2), generator=g, device=dev, dtype=torch.uint8)
    ws = (0.01 * (1 + 0.2 * torch.rand(N, K // 32, generator=g, device=dev))).to(torch.bfloat16)
    xq = torch.randint(0, 256, (M, K // 2), generator=g, device=dev, dtype=torch.uint8)
    xs = (0.5 * (1 + torch.rand(M, K // 32, generator=g, device=dev))).to(torch.bfloat16)
    return g, xq, xs, wq, ws


def _sampled_check(y, xq, xs, wq, ws, g, orc, n_rows, n_cols, tag):
    M, N = y.shape
    rows = torch.randperm(M, generator=g, device=y.device)[:min(n_rows, M)].sort().values
    cols = torch.randperm(N, generator=g, device=y.device)[:min(n_cols, N)].sort().values
    # always include the corners of the tile grid: first / last rows and columns
    rows = torch.unique(torch.cat((rows, torch.tensor([0, M - 1], device=y.device))))
    cols = torch.unique(torch.cat((cols, torch.tensor([0, N - 1], device=y.device))))
    y64 = orc.gemm_f64(xq[rows].cpu().numpy(), orc.bits(xs[rows]), wq[cols].cpu().numpy(), orc.bits(ws[cols]))
    _close(y[rows][:, cols], y64, tag)


# ------------------------------------------------------------------------------------------
# prefill: K = 8192, N = 57344 at M = 2048 and 4096; group-scaled 4096^3
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M", [2048, 4096])
def test_prefill_llama70b_gate_up(dev, orc, M):
    """The shapes the prefill throughput is quoted on, through wush_w4a4_gemm with AUTO (what the
    benchmark and my_int4._C.w4a4_gemm_s4 call).  cabi.gemm also asserts that word 0 of the scratch,
    the kernels' bounded-wait error word, is still zero."""
    K, N = 8192, 57344
    g, xq, xs, wq, ws = _random_operands(M, N, K, 40 + M, dev)
    xq[M // 2].zero_()
    assert capi.load().wush_w4a4_gemm_pick_variant(M, N, K) == capi.GEMM_TILE_F16
    y = cabi.gemm(xq, xs, wq, ws)
    _sampled_check(y, xq, xs, wq, ws, g, orc, 96, 96, ("prefill", M))
    assert (y[M // 2] == 0).all()
    assert torch.isfinite(y).all()
    # every 256 x 256 tile of the output was written: no tile keeps the fill pattern
    y2 = torch.full_like(y, float("nan"))
    lib = capi.load()
    nbytes = lib.wush_w4a4_gemm_workspace_bytes(M, N, K, capi.GEMM_AUTO)
    work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    capi.check(lib.wush_w4a4_gemm(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K, y2.data_ptr(),
                                  capi.GEMM_AUTO, work.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream), "gemm")
    torch.cuda.synchronize()
    assert int(work[:4].view(torch.int32).item()) == 0
    assert torch.equal(y2, y), "a second call on the same operands differs (or left part of the output unwritten)"


def test_prefill_square_4096_group_scaled(dev, orc):
    M = N = K = 4096
    g, xq, xs, wq, ws = _random_operands(M, N, K, 77, dev)
    y = cabi.gemm(xq, xs, wq, ws)
    _sampled_check(y, xq, xs, wq, ws, g, orc, 128, 128, "4096^3")
    # the exact-group-sum tile kernel on the same operands (int32 sums per group, fp32 scaling)
    y_tile = cabi.gemm(xq, xs, wq, ws, variant=capi.GEMM_TILE)
    _sampled_check(y_tile, xq, xs, wq, ws, g, orc, 64, 64, "4096^3 tile")


# ------------------------------------------------------------------------------------------
# the CPU-runnable configuration exactly as stated: M = 16, K = N = 4096, 512 calibration rows
# ------------------------------------------------------------------------------------------
def test_single_layer_m16_k4096_n4096_cpu_drawn(dev, orc):
    """The whole layer (fused transform + quantisation, then the product) on a layer drawn on the CPU
    with the benchmark's distributions -- identical bits for the oracle and the GPU.  The bit-exact
    name must reproduce the oracle's codes and scales; the layer output must agree with the fp64
    arbiter on the FULL 16 x 4096 result."""
    from my_int4 import _C
    from wush_int4_kernel_b200 import synth
    from wush_int4_kernel_b200.linear import W4A4Linear

    assert synth.CALIB_ROWS == 512
    M, K, N = 16, 4096, 4096
    layer = synth.make_layer(K, N, seed=0)                       # CPU draw and CPU quantiser (reference semantics)
    x = synth.draw_activations(M, K, layer.outliers, torch.Generator().manual_seed(1))
    t_bits, x_bits = orc.bits(layer.t_bf16), orc.bits(x)
    xq_o, xs_o = orc.fused_tq(x_bits, t_bits)
    # weights: the GPU quantiser on the same transformed weights gives the CPU result bit for bit
    xq, xs = _C.fused_transform_quant_int4(x.to(dev), layer.t_bf16.to(dev))
    assert np.array_equal(xq.cpu().numpy(), xq_o) and np.array_equal(orc.bits(xs), xs_o)
    lin = W4A4Linear(layer.t_bf16.to(dev), layer.wq.to(dev), layer.ws.to(dev))
    y = lin(x.to(dev))                                            # production names: _smallm + w4a4_gemv_multi
    xq_f, xs_f = _C.fused_transform_quant_int4_smallm(x.to(dev), lin.t)
    flips = (xq_f.cpu().numpy() != xq_o)
    assert flips.mean() <= 2e-4                                   # <= 1e-4 of the nibbles = 2e-4 of the bytes
    y64 = orc.gemm_f64(xq_f.cpu().numpy(), orc.bits(xs_f), layer.wq.numpy(), orc.bits(layer.ws))
    _close(y, y64, "config 1 layer")
    # and through the exact codes: the product alone against the arbiter of the oracle's own codes
    y_exact = cabi.gemm(xq, xs, lin.wq, lin.ws)
    _close(y_exact, orc.gemm_f64(xq_o, xs_o, layer.wq.numpy(), orc.bits(layer.ws)), "config 1 product")


# ------------------------------------------------------------------------------------------
# one rank's shard of the tensor-parallel FFN block at full dimensions
# ------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def ffn_shard(dev):
    """Rank 0's shard of hidden 8192 / intermediate 28672 over 8 ranks: gate+up 7168 x 8192 (gate rows
    then up rows of the local 3584 intermediate channels), down 8192 x 3584."""
    from my_int4 import _C
    from wush_int4_kernel_b200 import synth
    from wush_int4_kernel_b200.linear import TensorParallelFFN

    hidden, inter_local = 8192, 28672 // 8
    gu = synth.make_layer(hidden, 2 * inter_local, seed=21, device="cuda", quantiser=_C.quant_int4)
    dn = synth.make_layer(inter_local, hidden, seed=22, device="cuda", quantiser=_C.quant_int4)
    ffn = TensorParallelFFN.from_local_shards((gu.t_bf16, gu.wq, gu.ws), (dn.t_bf16, dn.wq, dn.ws), world=8, rank=0)
    ffn.down.reduce_output = False                                # this rank's partial product, no exchange
    return _C, synth, gu, dn, ffn


@pytest.mark.parametrize("M", [1, 32, 2048])
def test_ffn_block_shard_full_dimensions(dev, orc, ffn_shard, M):
    _C, synth, gu, dn, ffn = ffn_shard
    hidden, inter = 8192, 3584
    x = synth.draw_activations(M, hidden, gu.outliers, torch.Generator(device="cuda").manual_seed(100 + M))
    y = ffn(x)                                                    # fused SiLU*up -> transform -> quantise in one kernel
    assert y.shape == (M, hidden) and y.dtype == torch.float16 and torch.isfinite(y).all()
    assert torch.equal(y, ffn.reference_call(x)), "fused activation kernel differs from the separate ops"
    # each product of the chain against the fp64 arbiter of its own quantised inputs (sampled)
    g = torch.Generator(device="cuda").manual_seed(M)
    xq, xs = (_C.fused_transform_quant_int4_smallm if M <= 32 else _C.fused_transform_quant_int4_v3)(x, gu.t_bf16)
    y1 = ffn.gate_up(x)
    _sampled_check(y1, xq, xs, gu.wq, gu.ws, g, orc, 64, 128, ("gate+up", M))
    hq, hs = _C.fused_silu_mul_transform_quant_int4(y1, dn.t_bf16)
    _sampled_check(y, hq, hs, dn.wq, dn.ws, g, orc, 64, 128, ("down", M))
    # the activation stage against the oracle's bit-exact chain on a few rows: <= 1e-4 of the nibbles
    rows = torch.unique(torch.tensor([0, M // 2, M - 1]))
    h = (torch.nn.functional.silu(y1[rows, :inter].float()) * y1[rows, inter:].float()).to(torch.bfloat16)
    hq_o, _ = orc.fused_tq(orc.bits(h.cpu()), orc.bits(dn.t_bf16.cpu()))
    assert (hq[rows.to(dev)].cpu().numpy() != hq_o).mean() <= 2e-4
