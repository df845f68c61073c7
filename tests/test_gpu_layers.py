"""GPU tests of the layer level: M-dispatch, column / row parallel shards and the FFN block.

The reference has no multi-GPU code, so the sharded results are pinned as compositions of the
single-op semantics: shards computed one after the other on ONE GPU must reproduce the
unsharded layer (column parallel: bit for bit; row parallel: to fp32 summation order)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    assert torch.cuda.is_available()
    from my_int4 import _C
    from wush_int4_kernel_b200 import synth
    _C.init()
    layer = synth.make_layer(1024, 768, seed=3, device="cuda", quantiser=_C.quant_int4)
    gen = torch.Generator(device="cuda").manual_seed(4)
    return _C, synth, layer, gen


@pytest.mark.parametrize("M", [1, 2, 5, 32, 40, 200])
def test_layer_dispatch_matches_oracle(setup, orc, M):
    _C, synth, layer, gen = setup
    from wush_int4_kernel_b200.linear import W4A4Linear
    lin = W4A4Linear(layer.t_bf16, layer.wq, layer.ws)
    x = synth.draw_activations(M, 1024, layer.outliers, gen)
    y = lin(x)
    assert y.shape == (M, 768) and y.dtype == torch.float16
    xq, xs = _C.fused_transform_quant_int4_v3(x, layer.t_bf16) if M > 32 else _C.fused_transform_quant_int4_smallm(x, layer.t_bf16)
    y64 = orc.gemm_f64(xq.cpu().numpy(), orc.bits(xs), layer.wq.cpu().numpy(), orc.bits(layer.ws))
    rel = np.linalg.norm(y.double().cpu().numpy() - y64) / np.linalg.norm(y64)
    assert rel <= 1e-3, rel
    y3 = lin(x.reshape(1, M, 1024))
    assert y3.shape == (1, M, 768) and torch.equal(y3[0], y)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_parallel_shards_compose(setup, world):
    _C, synth, layer, gen = setup
    from wush_int4_kernel_b200.linear import ColumnParallelW4A4Linear, W4A4Linear
    x = synth.draw_activations(3, 1024, layer.outliers, gen)
    full = W4A4Linear(layer.t_bf16, layer.wq, layer.ws)(x)
    parts = [ColumnParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, r, multiple=32)(x) for r in range(world)]
    assert sum(p.shape[1] for p in parts) == 768
    assert torch.equal(torch.cat(parts, dim=1), full)


@pytest.mark.parametrize("world", [2, 4])
def test_row_parallel_partials_sum(setup, orc, world):
    _C, synth, layer, gen = setup
    from wush_int4_kernel_b200.linear import RowParallelW4A4Linear, W4A4Linear, shard_bounds
    x = synth.draw_activations(40, 1024, layer.outliers, gen)
    full = W4A4Linear(layer.t_bf16, layer.wq, layer.ws)(x).float()
    acc = torch.zeros_like(full)
    for r in range(world):
        shard = RowParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, r, reduce_output=False)
        k0, k1 = shard_bounds(1024, world, r, 32)
        acc += shard(x[:, k0:k1].contiguous()).float()
    rel = ((acc - full).norm() / full.norm()).item()
    assert rel <= 2e-3, rel            # each partial is rounded to fp16 before the sum


def test_ffn_block_single_rank_equals_composition(setup):
    _C, synth, layer, gen = setup
    from wush_int4_kernel_b200.linear import TensorParallelFFN, W4A4Linear
    hidden, inter = 512, 1024
    gu = synth.make_layer(hidden, 2 * inter, seed=7, device="cuda", quantiser=_C.quant_int4)
    dn = synth.make_layer(inter, hidden, seed=8, device="cuda", quantiser=_C.quant_int4)
    ffn = TensorParallelFFN((gu.t_bf16, gu.wq, gu.ws), (dn.t_bf16, dn.wq, dn.ws), world=1, rank=0)
    x = synth.draw_activations(24, hidden, gu.outliers, gen)
    y = ffn(x)
    assert torch.equal(y, ffn.reference_call(x))          # fused activation kernel == separate torch kernels, bit for bit
    g = W4A4Linear(gu.t_bf16, gu.wq, gu.ws)(x)
    h = (torch.nn.functional.silu(g[:, :inter].float()) * g[:, inter:].float()).to(torch.bfloat16)
    expect = W4A4Linear(dn.t_bf16, dn.wq, dn.ws)(h)
    assert y.shape == (24, hidden) and torch.equal(y, expect)
    # two ranks' worth of shards, run one after the other: partial products add up to the block
    parts = []
    for r in range(2):
        shard = TensorParallelFFN((gu.t_bf16, gu.wq, gu.ws), (dn.t_bf16, dn.wq, dn.ws), world=2, rank=r)
        shard.down.reduce_output = False
        parts.append(shard(x).float())
    rel = ((parts[0] + parts[1] - expect.float()).norm() / expect.float().norm()).item()
    assert rel <= 5e-3, rel


def test_two_process_nccl_if_available():
    """torchrun with two ranks when the box has two GPUs: column-parallel all-gather and
    row-parallel all-reduce against the unsharded layer (skipped on single-GPU boxes)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import socket
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with socket.socket() as sock:                      # a port nobody is using right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(root, "tests", "nccl_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout


@pytest.mark.parametrize("rows,K", [(1, 256), (7, 1024), (33, 512), (300, 2048)])
def test_fused_silu_mul_transform_quant(setup, rows, K):
    """One kernel for SiLU(gate) * up -> bf16 -> transform -> quantise against the composition
    `fused_transform_quant_int4_v3((silu(gate.float()) * up.float()).bfloat16(), t)`."""
    _C, synth, layer, gen = setup
    gate_up = (2.0 * torch.randn(rows, 2 * K, generator=gen, device="cuda")).to(torch.float16)
    t = (torch.randn(K // 32, 32, 32, generator=gen, device="cuda") / 6).to(torch.bfloat16)
    q, s = _C.fused_silu_mul_transform_quant_int4(gate_up, t)
    h = (torch.nn.functional.silu(gate_up[:, :K].float()) * gate_up[:, K:].float()).to(torch.bfloat16).contiguous()
    q_ref, s_ref = _C.fused_transform_quant_int4_v3(h, t)
    assert q.shape == (rows, K // 2) and s.shape == (rows, K // 32) and s.dtype == torch.bfloat16
    assert torch.equal(s, s_ref) and torch.equal(q, q_ref)
    with pytest.raises(RuntimeError):
        _C.fused_silu_mul_transform_quant_int4(gate_up.float(), t)


def test_peer_allreduce_single_rank():
    """World of one through the C ABI: the kernel's copy / publish / wait / reduce path with no
    peers -- the result is the input, step after step, eager and replayed from a graph."""
    import ctypes
    from wush_int4_kernel_b200 import capi
    lib = capi.load()
    comm = ctypes.c_void_p()
    capi.check(lib.wush_comm_create(0, 1, 256 * 1024, ctypes.byref(comm)), "comm_create")
    try:
        gen = torch.Generator(device="cuda").manual_seed(0)
        stream = torch.cuda.current_stream().cuda_stream
        for n in (8, 8192, 131072, 8192):
            part = torch.randn(n, generator=gen, device="cuda").to(torch.float16)
            out = torch.zeros_like(part)
            capi.check(lib.wush_comm_allreduce_f16(comm, part.data_ptr(), out.data_ptr(), n, stream), "allreduce")
            assert torch.equal(out, part)
        assert lib.wush_comm_allreduce_f16(comm, part.data_ptr(), out.data_ptr(), 12, stream) != 0       # not a multiple of 8
        big = torch.zeros(256 * 1024, dtype=torch.float16, device="cuda")
        assert lib.wush_comm_allreduce_f16(comm, big.data_ptr(), big.data_ptr(), big.numel(), stream) != 0  # larger than a slot
        err = ctypes.c_int(-1)
        capi.check(lib.wush_comm_error(comm, ctypes.byref(err)), "comm_error")
        assert err.value == 0
    finally:
        capi.check(lib.wush_comm_destroy(comm), "comm_destroy")


def test_peer_allreduce_wait_runs_out():
    """Failure detection without a fault: rank 0 of a world of two whose peer never publishes.
    The peer's buffer is a second communicator of this process that never runs; the wait of the
    kernel is bounded (set to ~2 ms here), it records the error word and returns, and the
    context stays usable."""
    import ctypes
    from wush_int4_kernel_b200 import capi
    lib = capi.load()
    mine, other = ctypes.c_void_p(), ctypes.c_void_p()
    capi.check(lib.wush_comm_create(0, 2, 64 * 1024, ctypes.byref(mine)), "comm_create")
    capi.check(lib.wush_comm_create(1, 2, 64 * 1024, ctypes.byref(other)), "comm_create")
    try:
        base = ctypes.c_void_p()
        capi.check(lib.wush_comm_base(other, ctypes.byref(base)), "comm_base")
        capi.check(lib.wush_comm_connect_pointer(mine, 1, base), "comm_connect_pointer")
        capi.check(lib.wush_comm_set_poll_limit(mine, 4096), "comm_set_poll_limit")
        part = torch.ones(4096, dtype=torch.float16, device="cuda")
        out = torch.zeros_like(part)
        stream = torch.cuda.current_stream().cuda_stream
        capi.check(lib.wush_comm_allreduce_f16(mine, part.data_ptr(), out.data_ptr(), part.numel(), stream), "allreduce")
        torch.cuda.synchronize()                                  # returns: nothing hangs
        err = ctypes.c_int(0)
        capi.check(lib.wush_comm_error(mine, ctypes.byref(err)), "comm_error")
        assert err.value == 1
        assert float((part * 2).sum().item()) == 8192.0           # the device still computes
    finally:
        capi.check(lib.wush_comm_destroy(mine), "comm_destroy")
        capi.check(lib.wush_comm_destroy(other), "comm_destroy")


@pytest.mark.parametrize("M,N,K", [(1, 768, 1024), (2, 1000, 4096), (1, 8192, 3584), (2, 264, 256),
                                   (3, 768, 1024), (8, 1000, 4096), (13, 264, 256), (24, 776, 512), (32, 768, 2048)])
def test_pushed_gemv_allreduce_single_rank(setup, M, N, K):
    """World of one: the product kernel writes into the exchange buffer instead of y, publishes,
    and the reduction returns it -- byte-identical to the plain product, several steps in a row
    (both slots), mixed with plain all-reduce steps."""
    import ctypes
    from tests import cabi
    from wush_int4_kernel_b200 import capi
    _C, synth, layer, gen = setup
    lib = capi.load()
    xq = torch.randint(0, 256, (M, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    wq = torch.randint(0, 256, (N, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    xs = (0.02 * (1 + torch.rand(M, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    ws = (0.01 * (1 + torch.rand(N, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    expect = cabi.gemm(xq, xs, wq, ws, capi.GEMM_GEMV if M <= 2 else capi.GEMM_DECODE)   # the kernel that pushes
    comm = ctypes.c_void_p()
    capi.check(lib.wush_comm_create(0, 1, 64 * 1024, ctypes.byref(comm)), "comm_create")
    try:
        stream = torch.cuda.current_stream().cuda_stream
        for step in range(3):
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            capi.check(lib.wush_comm_gemv_allreduce(comm, xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K,
                                                    out.data_ptr(), stream), "gemv_allreduce")
            assert torch.equal(out, expect), step
            plain = torch.zeros_like(expect)
            capi.check(lib.wush_comm_allreduce_f16(comm, expect.data_ptr(), plain.data_ptr(), expect.numel(), stream), "allreduce")
            assert torch.equal(plain, expect)
        x33 = torch.zeros(33, K // 2, dtype=torch.uint8, device="cuda")
        assert lib.wush_comm_gemv_allreduce(comm, x33.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), 33, N, K,
                                            out.data_ptr(), stream) == 3          # WUSH_ERR_UNSUPPORTED: more than 32 rows
        err = ctypes.c_int(-1)
        capi.check(lib.wush_comm_error(comm, ctypes.byref(err)), "comm_error")
        assert err.value == 0
    finally:
        capi.check(lib.wush_comm_destroy(comm), "comm_destroy")


def _widths(values):
    import ctypes
    return (ctypes.c_int64 * len(values))(*values)


@pytest.mark.parametrize("M,N,K", [(1, 768, 1024), (2, 1000, 4096), (8, 1000, 4096), (32, 768, 2048)])
def test_peer_allgather_single_rank(setup, M, N, K):
    """World of one: the gather is a copy through the slot (pull form) and the product's pushed
    block comes back unchanged (pushed form); bad widths are refused before any launch."""
    import ctypes
    from tests import cabi
    from wush_int4_kernel_b200 import capi
    _C, synth, layer, gen = setup
    lib = capi.load()
    xq = torch.randint(0, 256, (M, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    wq = torch.randint(0, 256, (N, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    xs = (0.02 * (1 + torch.rand(M, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    ws = (0.01 * (1 + torch.rand(N, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    expect = cabi.gemm(xq, xs, wq, ws, capi.GEMM_GEMV if M <= 2 else capi.GEMM_DECODE)
    comm = ctypes.c_void_p()
    capi.check(lib.wush_comm_create(0, 1, 64 * 1024, ctypes.byref(comm)), "comm_create")
    try:
        stream = torch.cuda.current_stream().cuda_stream
        for step in range(3):
            out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
            capi.check(lib.wush_comm_gemv_allgather(comm, xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, K,
                                                    _widths([N]), out.data_ptr(), stream), "gemv_allgather")
            assert torch.equal(out, expect), step
            plain = torch.zeros_like(expect)
            capi.check(lib.wush_comm_allgather_f16(comm, expect.data_ptr(), plain.data_ptr(), M, _widths([N]), stream), "allgather")
            assert torch.equal(plain, expect)
        assert lib.wush_comm_allgather_f16(comm, expect.data_ptr(), plain.data_ptr(), M, _widths([N - 4]), stream) != 0   # not a multiple of 8
        assert lib.wush_comm_allgather_f16(comm, expect.data_ptr(), plain.data_ptr(), 64, _widths([N]), stream) != 0     # larger than a slot
        err = ctypes.c_int(-1)
        capi.check(lib.wush_comm_error(comm, ctypes.byref(err)), "comm_error")
        assert err.value == 0
    finally:
        capi.check(lib.wush_comm_destroy(comm), "comm_destroy")


@pytest.mark.parametrize("M", [1, 2, 8, 32])
def test_peer_allgather_two_ranks_one_after_the_other(setup, M):
    """World of two in one process, blocks of unequal width.  The two ranks' kernels never run at
    the same time: rank 1 goes first with a wait of ~2 ms that runs out (nobody has published for
    rank 0 yet) -- its block and its flag are in place by then --, then rank 0 runs and finds
    everything there.  Checks the slot / offset arithmetic of both forms against the plain products."""
    import ctypes
    from tests import cabi
    from wush_int4_kernel_b200 import capi
    _C, synth, layer, gen = setup
    lib = capi.load()
    K, widths = 1024, [512, 256]
    xq = torch.randint(0, 256, (M, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    xs = (0.02 * (1 + torch.rand(M, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16)
    wq = [torch.randint(0, 256, (w, K // 2), generator=gen, device="cuda", dtype=torch.uint8) for w in widths]
    ws = [(0.01 * (1 + torch.rand(w, K // 32, generator=gen, device="cuda"))).to(torch.bfloat16) for w in widths]
    blocks = [cabi.gemm(xq, xs, wq[r], ws[r], capi.GEMM_GEMV if M <= 2 else capi.GEMM_DECODE) for r in range(2)]
    expect = torch.cat(blocks, dim=1)
    stream = torch.cuda.current_stream().cuda_stream
    for pushed in (False, True):
        comms = [ctypes.c_void_p(), ctypes.c_void_p()]
        for r in range(2):
            capi.check(lib.wush_comm_create(r, 2, 64 * 1024, ctypes.byref(comms[r])), "comm_create")
        try:
            for r in range(2):
                base = ctypes.c_void_p()
                capi.check(lib.wush_comm_base(comms[1 - r], ctypes.byref(base)), "comm_base")
                capi.check(lib.wush_comm_connect_pointer(comms[r], 1 - r, base), "comm_connect_pointer")
            capi.check(lib.wush_comm_set_poll_limit(comms[1], 4096), "comm_set_poll_limit")
            outs = [torch.zeros(M, sum(widths), dtype=torch.float16, device="cuda") for _ in range(2)]
            for r in (1, 0):
                if pushed:
                    capi.check(lib.wush_comm_gemv_allgather(comms[r], xq.data_ptr(), xs.data_ptr(), wq[r].data_ptr(), ws[r].data_ptr(),
                                                            M, K, _widths(widths), outs[r].data_ptr(), stream), "gemv_allgather")
                else:
                    capi.check(lib.wush_comm_allgather_f16(comms[r], blocks[r].data_ptr(), outs[r].data_ptr(), M, _widths(widths),
                                                           stream), "allgather")
                torch.cuda.synchronize()
            errs = []
            for r in range(2):
                e = ctypes.c_int(-1)
                capi.check(lib.wush_comm_error(comms[r], ctypes.byref(e)), "comm_error")
                errs.append(e.value)
            assert errs == [0, 1]                                # rank 1 gave up as planned, rank 0 saw both blocks
            assert torch.equal(outs[0], expect), pushed
        finally:
            for c in comms:
                capi.check(lib.wush_comm_destroy(c), "comm_destroy")


def test_peer_allreduce_two_phase_single_rank_and_sequential_ranks():
    """The two-phase sum (reduce-scatter + all-gather in one kernel).  World of one: the result is the
    input.  World of two in one process, the ranks' kernels run one after the other: rank 1 first, whose
    waits (~2 ms) run out with its partial and its flag in place; rank 0 then finds rank 1's partial,
    reduces its own half exactly -- the half rank 1 would have delivered stays untouched -- and gives up
    at the second wait (nobody publishes the second step for rank 1).  Checks addressing and bounded waits."""
    import ctypes
    from wush_int4_kernel_b200 import capi
    lib = capi.load()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(5)
    comm = ctypes.c_void_p()
    capi.check(lib.wush_comm_create(0, 1, 4 << 20, ctypes.byref(comm)), "comm_create")
    try:
        for n in (8, 1 << 20, 8192, 2 << 20):
            part = torch.randn(n, generator=gen, device="cuda").to(torch.float16)
            out = torch.zeros_like(part)
            capi.check(lib.wush_comm_allreduce_two_phase_f16(comm, part.data_ptr(), out.data_ptr(), n, stream), "two_phase")
            assert torch.equal(out, part)
            plain = torch.zeros_like(part)
            capi.check(lib.wush_comm_allreduce_f16(comm, part.data_ptr(), plain.data_ptr(), n, stream), "allreduce")
            assert torch.equal(plain, part)
        err = ctypes.c_int(-1)
        capi.check(lib.wush_comm_error(comm, ctypes.byref(err)), "comm_error")
        assert err.value == 0
    finally:
        capi.check(lib.wush_comm_destroy(comm), "comm_destroy")

    comms = [ctypes.c_void_p(), ctypes.c_void_p()]
    for r in range(2):
        capi.check(lib.wush_comm_create(r, 2, 1 << 20, ctypes.byref(comms[r])), "comm_create")
    try:
        for r in range(2):
            base = ctypes.c_void_p()
            capi.check(lib.wush_comm_base(comms[1 - r], ctypes.byref(base)), "comm_base")
            capi.check(lib.wush_comm_connect_pointer(comms[r], 1 - r, base), "comm_connect_pointer")
            capi.check(lib.wush_comm_set_poll_limit(comms[r], 4096), "comm_set_poll_limit")
        n = 1 << 18
        parts = [torch.randn(n, generator=gen, device="cuda").to(torch.float16) for _ in range(2)]
        outs = [torch.full((n,), 7.0, dtype=torch.float16, device="cuda") for _ in range(2)]
        for r in (1, 0):
            capi.check(lib.wush_comm_allreduce_two_phase_f16(comms[r], parts[r].data_ptr(), outs[r].data_ptr(), n, stream), "two_phase")
            torch.cuda.synchronize()
        errs = []
        for r in range(2):
            e = ctypes.c_int(-1)
            capi.check(lib.wush_comm_error(comms[r], ctypes.byref(e)), "comm_error")
            errs.append(e.value)
        assert errs == [1, 1]
        assert bool((outs[0] == 7.0).all())                          # a sum that was not completed is not delivered
        # rank 0's half of the sum reached rank 1's buffer: slot (1, 1) of rank 1, vectors [0, n/2)
        base1 = ctypes.c_void_p()
        capi.check(lib.wush_comm_base(comms[1], ctypes.byref(base1)), "comm_base")
        expect = (parts[0].float() + parts[1].float()).to(torch.float16)[: n // 2]
        from tests import cabi
        got = cabi.device_view(base1.value + (1 * 2 + 1) * (1 << 20), n // 2, torch.float16)
        assert torch.equal(got, expect)
        assert torch.isfinite((parts[0] * 2).sum()).item()            # the device still computes
    finally:
        for c in comms:
            capi.check(lib.wush_comm_destroy(c), "comm_destroy")


@pytest.mark.parametrize("rows", [1, 8])
def test_host_streamed_layer_equals_plain_layer(setup, rows):
    """Requests from pinned host memory through the three-stream pipeline (uploads, kernels and downloads of
    consecutive requests overlap): every result equals the plain layer's, eagerly and replayed from one graph,
    with more requests than device buffers and alternating weights."""
    from wush_int4_kernel_b200.host_pipeline import HostStreamedLayer
    from wush_int4_kernel_b200.linear import W4A4Linear
    _C, synth, layer, gen = setup
    other = synth.make_layer(1024, 768, seed=11, device="cuda", quantiser=_C.quant_int4)
    weights = [(layer.wq, layer.ws), (other.wq, other.ws)]
    xs = [synth.draw_activations(rows, 1024, layer.outliers, gen) for _ in range(7)]
    want = [W4A4Linear(layer.t_bf16, *weights[i % 2])(x).cpu() for i, x in enumerate(xs)]
    x_hosts = [x.cpu().pin_memory() for x in xs]
    y_hosts = [torch.zeros(rows, 768, dtype=torch.float16).pin_memory() for _ in xs]
    pipe = HostStreamedLayer(layer.t_bf16, rows)
    pipe.run(x_hosts, y_hosts, weights)
    torch.cuda.synchronize()
    for i, (y, w) in enumerate(zip(y_hosts, want)):
        assert torch.equal(y, w), f"eager, request {i}"
    for y in y_hosts:
        y.zero_()
    from wush_int4_kernel_b200 import timing
    graph, _ = timing.capture(lambda: pipe.run(x_hosts, y_hosts, weights))
    for y in y_hosts:
        y.zero_()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for i, (y, w) in enumerate(zip(y_hosts, want)):
        assert torch.equal(y, w), f"graph, request {i}"
    with pytest.raises(ValueError):
        pipe.run([xs[0].cpu()], [y_hosts[0]], weights)          # not pinned
