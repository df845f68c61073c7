#!/usr/bin/env python
"""Benchmark of the W4A4 linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows M]

Workload (``config.workload``): the Llama-70B-style fused gate+up decode layer, K=8192,
N=57344, M=1 activation row per step (``--rows`` changes M).  One step = one layer call as
the reference times it (bench/exp_p13_official.py:31-39): fused WUSH transform+quantisation
of the activations, then the group-scaled W4A4 product, replayed from a CUDA Graph.  At
N GPUs the layer is column parallel: each rank holds N/p output columns (no data-path
collective; the consumer of a fused gate+up projection is column-local).  Total work is
fixed, so scaling is "strong".

Prints ONE JSON line: metric effective TOPS (2*M*N*K / time), plus
  roofline      the weight-streaming product kernel against the measured HBM copy bandwidth
  cpu_baseline  the CPU oracle port of the same layer on this box's host cores
  e2e           the same metric through the public ops with HOST activations and results
  clocks        SM clock / throttle reasons sampled with nvidia-smi while the step runs
  prefill       the other half of the metric, measured in the same run: M=4096 rows through the same
                layer (this rank's column shard at N GPUs), against the tensor-core peak
  ffn_block     (N > 1 only) the tensor-parallel FFN block 8192 -> 2 x 28672 -> 8192 at M = 1 / 32 / 2048:
                with the exchange over NVLink peer memory and with the NCCL all-reduce
``config`` names the workload only and is key-for-key the same in both arms; how this arm lays the
work out (sharding, L2 policy, timing method) is under ``setup``.

``--impl reference`` times the CPU port alone (rank 0 only): the reference's own kernels are
sm_75-only CUDA and cannot run here, its Python path is what the oracle restates.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM, N_DIM = 8192, 57344
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the product kernel, from the ncu
# capture summarised in profiles/gemv_row_decode_m1_k8192_n57344.md (264.27 MB read + 3.37 / 4.76 MB
# written in the two captured launches; their mean).
PRODUCT_KERNEL_DRAM_BYTES = 268_330_000
PRODUCT_KERNEL_DRAM_SOURCE = ("constant from an earlier ncu capture, not measured in this run: "
                              "profiles/gemv_row_decode_m1_k8192_n57344.md (scaled by the shard's share of N)")
INT8_NOMINAL_TOPS = 4500.0
PREFILL_ROWS = 4096


def workload_config(M: int) -> dict:
    """The workload, named the same way by both arms."""
    return {"workload": f"llama70b_gate_up_decode K={K_DIM} N={N_DIM} M={M}", "K": K_DIM, "N": N_DIM, "M": M}


def algorithmic_bytes_product(M: int, N: int, K: int) -> int:
    """codes + scales of the weights and of the activations, fp16 output."""
    return 9 * N * K // 16 + 9 * M * K // 16 + 2 * M * N


def algorithmic_bytes_layer(M: int, N: int, K: int) -> int:
    """fused transform+quant (x in, T in, codes+scales out) followed by the product."""
    return 2 * M * K + 64 * K + 2 * (9 * M * K // 16) + 9 * N * K // 16 + 2 * M * N


def measured_peak(key: str, fallback: float):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)[key]), "measured"
    except (OSError, KeyError, ValueError):
        return fallback, "fallback"


def measured_hbm_peak():
    return measured_peak("hbm_gbs", 6650.0)


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the layer (test infrastructure, the only place outside tests and
# the smoke check where oracle/ is executed)
# ---------------------------------------------------------------------------------------------
CPU_BLOCK_ROWS = 4096


def cpu_layer_inputs(M: int, n_rows: int, seed: int = 1234):
    """The seeded synthetic layer of synth.py, drawn on the CPU: activations N(0,1) with 0.5 % of the
    channels x 20, weights N(0, 0.02), transform solved from 512 calibration rows, weights transformed
    and sigma-clip quantised.  One block of CPU_BLOCK_ROWS weight rows is built this way and repeated
    up to n_rows (building all 57344 rows in fp64 on the host would take longer than the timed
    sample itself; the CPU path's time does not depend on the values)."""
    import numpy as np
    import torch

    from oracle import w4a4_oracle as orc
    from wush_int4_kernel_b200 import synth, wush_transform as wt

    gen = torch.Generator().manual_seed(seed)
    outliers = synth.outlier_channels(K_DIM, torch.Generator().manual_seed(7))
    x_cal = synth.draw_activations(synth.CALIB_ROWS, K_DIM, outliers, gen).float()
    block = min(CPU_BLOCK_ROWS, n_rows)
    w = (0.02 * torch.randn(block, K_DIM, generator=gen)).to(torch.bfloat16)
    t64 = wt.solve_from_grams(wt.diag_block_gram(x_cal) / synth.CALIB_ROWS, wt.diag_block_gram(w) / block)
    wq_b, ws_b = orc.quant_int4(orc.bits(wt.transform_weights(w, t64).to(torch.bfloat16).contiguous()))
    reps = -(-n_rows // block)
    wq = np.ascontiguousarray(np.tile(wq_b, (reps, 1))[:n_rows])
    ws = np.ascontiguousarray(np.tile(ws_b, (reps, 1))[:n_rows])
    x = orc.bits(synth.draw_activations(M, K_DIM, outliers, gen))
    t = orc.bits(t64.to(torch.bfloat16).contiguous())
    return x, t, wq, ws


def cpu_model() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def time_cpu_layer(M: int, n_rows: int, steps: int, warmup: int, inputs=None):
    from oracle import w4a4_oracle as orc
    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    x, t, wq, ws = inputs if inputs is not None else cpu_layer_inputs(M, n_rows)
    for _ in range(warmup):
        orc.layer(x, t, wq, ws)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        orc.layer(x, t, wq, ws)
        times.append(time.perf_counter() - t0)
    return times, cores


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M = args.rows
    n_rows = N_DIM                                   # the whole layer: ~0.5 G MAC per row of X
    times, cores = time_cpu_layer(M, n_rows, args.steps, args.warmup)
    med = statistics.median(times)                   # the same statistic as the GPU arm's cpu_baseline leg
    tops = 2.0 * M * n_rows * K_DIM / med / 1e12
    line = {
        "impl": "reference", "metric": "w4a4_layer_eff_tops", "value": tops, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * med, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4", "data": "synthetic",
        "config": workload_config(M),
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "cpu": cpu_model(), "kind": "port",
                         "sample": f"whole layer (N={n_rows} rows of W: a seeded synthetic block of {CPU_BLOCK_ROWS} rows repeated), "
                                   f"median of {len(times)} steps (mean {1e3 * sum(times) / len(times):.3f} ms), OpenMP over output columns"},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def measure_prefill(weights, t_bf16, outliers, gen, dev, world, n_local, barrier):
    """M = PREFILL_ROWS rows through the same layer (this rank's column shard): transform+quantise, then
    the product through the public op (my_int4._C.w4a4_gemm_s4).  Median of 5 batches of 4 graph replays
    over the rotating weight copies (layer and product batches alternating), max over ranks."""
    import torch
    import torch.distributed as dist

    from wush_int4_kernel_b200 import synth, timing
    from wush_int4_kernel_b200.linear import quantise_activations, w4a4_product

    M = PREFILL_ROWS
    x = synth.draw_activations(M, K_DIM, outliers, gen)
    xq, xs = quantise_activations(x, t_bf16)
    use = weights[:2]

    def batch_ms(graphs):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(4):
            graphs[i % len(graphs)].replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 4

    def across_ranks(ms):
        if world > 1:
            tmax = torch.tensor([ms], device=dev)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            ms = float(tmax.item())
        return ms

    layer_graphs = [timing.capture(lambda wq=wq, ws=ws: w4a4_product(*quantise_activations(x, t_bf16), wq, ws))[0]
                    for (wq, ws) in use]
    prod_graphs = [timing.capture(lambda wq=wq, ws=ws: w4a4_product(xq, xs, wq, ws))[0] for (wq, ws) in use]
    for i in range(3):
        layer_graphs[i % len(layer_graphs)].replay()
    # batches of the two graphs alternate, so both medians see the same power / clock state of the part
    layer_t, prod_t = [], []
    for _ in range(5):
        layer_t.append(batch_ms(layer_graphs))
        prod_t.append(batch_ms(prod_graphs))
    layer_ms, prod_ms = across_ranks(statistics.median(layer_t)), across_ranks(statistics.median(prod_t))
    torch.cuda.empty_cache()
    tpeak, tkind = measured_peak("bf16_tflops", 1590.0)
    per_gpu = 2.0 * M * n_local * K_DIM / (prod_ms * 1e-3) / 1e12
    return {"M": M, "K": K_DIM, "N": N_DIM, "columns_per_gpu": n_local, "us_per_layer": layer_ms * 1e3,
            "product_us": prod_ms * 1e3, "eff_tops": 2.0 * M * N_DIM * K_DIM / (layer_ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tpeak, "unit": "TFLOP/s", "frac": per_gpu / tpeak,
                         "peak_kind": f"of {tkind} (cuBLAS bf16 burst; the product runs tcgen05 kind::f16 on exactly "
                                      f"folded operands, so the dense-f16 rate is its ceiling)",
                         "frac_of_nominal_int8": per_gpu / INT8_NOMINAL_TOPS, "kernel": "w4a4 product (per GPU)"}}


def measure_ffn_block(world, rank, dev):
    """hidden 8192, intermediate 28672, one rank per GPU: fused gate+up (column parallel) -> SiLU*up ->
    transform+quantise -> down (row parallel) -> sum over ranks; once with the exchange over NVLink peer
    memory (decode sizes; larger results fall back to NCCL inside it) and once with the NCCL all-reduce."""
    import torch

    from wush_int4_kernel_b200 import bench_matrix
    from wush_int4_kernel_b200.peer_reduce import PeerAllReduce

    layers = bench_matrix.build_ffn_layers(world, rank, dev, copies=3)
    peer = PeerAllReduce(max_elements=2048 * 8192)   # the block's output at every M measured (two-phase sum beyond a megabyte); 32-row blocks of the gate+up shard
    out = {}
    for m in (1, 32, 2048):
        with_peer = bench_matrix.measure_ffn(m, world, rank, dev, True, peer, layers=layers)
        with_nccl = bench_matrix.measure_ffn(m, world, rank, dev, True, None, layers=layers)
        out[str(m)] = {"us_peer_memory": with_peer["us_per_block"], "exchange": with_peer["all_reduce"],
                       "us_nccl": with_nccl["us_per_block"], "graph": with_peer["graph"] and with_nccl["graph"],
                       "eff_tops_whole_block": with_peer["eff_tops_whole_block"]}
        torch.cuda.empty_cache()
    # the gate+up layer alone, column parallel, full row gathered on every rank (decode sizes)
    gather = {}
    for m in (1, 32):
        with_peer = bench_matrix.measure_column_gather(m, world, rank, dev, peer, layers)
        with_nccl = bench_matrix.measure_column_gather(m, world, rank, dev, None, layers)
        gather[str(m)] = {"us_peer_memory": with_peer["us_per_layer"], "us_nccl": with_nccl["us_per_layer"],
                          "gather": with_peer["gather"], "graph": with_peer["graph"] and with_nccl["graph"]}
    out["column_gather"] = gather
    err = peer.error()
    peer.close()
    out["peer_wait_timeout"] = bool(err)
    out["block"] = "ffn 8192 -> 2 x 28672 -> 8192, tensor parallel over %d GPUs" % world
    return out


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from wush_int4_kernel_b200 import _C, synth, timing
    from wush_int4_kernel_b200.linear import quantise_activations, shard_bounds, w4a4_product

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _C.init()

    M = args.rows
    n0, n1 = shard_bounds(N_DIM, world, rank, 128)
    n_local = n1 - n0

    # ---- synthetic layer shard (seeded; distributions of synth.py).  Built on the GPU once and kept as
    # layer files (layer_file.py) in the temporary directory: later runs on the same box -- the other
    # arm, the next N of a scaling series -- load the {wq, ws, T} triples instead of re-quantising them.
    from wush_int4_kernel_b200 import layer_file, wush_transform as wt
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    outliers = synth.outlier_channels(K_DIM, torch.Generator(device=dev).manual_seed(7))
    shard_bytes = n_local * (K_DIM // 2 + K_DIM // 16)
    copies = max(2, -(-(2 * L2_BYTES + shard_bytes) // shard_bytes))   # consecutive steps never touch the same bytes
    cache_dir = os.path.join(tempfile.gettempdir(), "wush_w4a4_bench_layers")
    os.makedirs(cache_dir, exist_ok=True)
    paths = [os.path.join(cache_dir, f"gate_up_K{K_DIM}_cols{n0}-{n1}_of{N_DIM}_copy{c}_v1.pt") for c in range(copies)]
    weights, t_bf16, from_cache = [], None, 0
    if all(os.path.exists(pth) for pth in paths):
        try:
            loaded = [layer_file.load_layer(pth, device=dev) for pth in paths]
            t_bf16 = loaded[0].t_bf16
            weights = [(l.wq, l.ws) for l in loaded]
            from_cache = copies
        except (ValueError, RuntimeError, OSError):
            weights = []
    if not weights:
        x_cal = synth.draw_activations(synth.CALIB_ROWS, K_DIM, outliers, gen).float()
        w0 = (0.02 * torch.randn(4096, K_DIM, generator=torch.Generator(device=dev).manual_seed(99), device=dev)).to(torch.bfloat16)
        t64 = wt.solve_from_grams(wt.diag_block_gram(x_cal) / synth.CALIB_ROWS, wt.diag_block_gram(w0) / 4096)
        t_bf16 = t64.to(torch.bfloat16).contiguous()
        for c in range(copies):
            wq_parts, ws_parts = [], []
            for r0 in range(0, n_local, 8192):
                w = (0.02 * torch.randn(min(8192, n_local - r0), K_DIM, generator=gen, device=dev)).to(torch.bfloat16)
                q, s_ = _C.quant_int4(wt.transform_weights(w, t64).to(torch.bfloat16).contiguous())
                wq_parts.append(q)
                ws_parts.append(s_)
            weights.append((torch.cat(wq_parts).contiguous(), torch.cat(ws_parts).contiguous()))
            try:
                layer_file.save_layer(paths[c], weights[-1][0], weights[-1][1], t_bf16, meta={"seed": 1234 + rank, "copy": c})
            except OSError:
                pass                                                   # no room in the temporary directory: keep going uncached
    x = synth.draw_activations(M, K_DIM, outliers, gen)

    def make_step(wq, ws):
        def step():
            xq, xs = quantise_activations(x, t_bf16)
            return w4a4_product(xq, xs, wq, ws)
        return step

    graphs = [timing.capture(make_step(wq, ws))[0] for (wq, ws) in weights]
    launches_per_step = 2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: W warm-ups, exactly K timed steps, max over ranks -----------
    sampler = timing.ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.__enter__()
    for i in range(max(args.warmup, 3)):
        graphs[i % copies].replay()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        graphs[i % copies].replay()
    stop.record()
    barrier()
    ms_total = start.elapsed_time(stop)
    # keep the same load running long enough for nvidia-smi to see it (not part of any number)
    t_end = time.perf_counter() + 1.0
    while time.perf_counter() < t_end:
        for i in range(200):
            graphs[i % copies].replay()
        torch.cuda.synchronize()
    if sampler:
        sampler.__exit__(None, None, None)
    if world > 1:
        tmax = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms_total = float(tmax.item())
    ms_per_step = ms_total / args.steps
    tops = 2.0 * M * N_DIM * K_DIM / (ms_per_step * 1e-3) / 1e12

    # ---- dominant kernel alone (roofline): the product kernel over the same shard -----------
    xq, xs = quantise_activations(x, t_bf16)
    prod_graphs = [timing.capture(lambda wq=wq, ws=ws: w4a4_product(xq, xs, wq, ws))[0] for (wq, ws) in weights]
    for i in range(5):
        prod_graphs[i % copies].replay()
    reps = max(20, min(args.steps, 400))
    samples = []
    for _ in range(5):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            prod_graphs[i % copies].replay()
        e1.record()
        torch.cuda.synchronize()
        samples.append(e0.elapsed_time(e1) / reps)
    kernel_ms = statistics.median(samples)
    alg_bytes = algorithmic_bytes_product(M, n_local, K_DIM)
    peak, peak_kind = measured_hbm_peak()
    achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
    if M <= 32:
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": (PRODUCT_KERNEL_DRAM_BYTES * n_local // N_DIM) if M == 1 else None,
                    "traffic_source": PRODUCT_KERNEL_DRAM_SOURCE if M == 1 else None,
                    "peak_kind": f"of {peak_kind} (a read+write copy; this kernel only reads, so a little above 1.0 is possible)",
                    "kernel": "w4a4 product", "kernel_us": kernel_ms * 1e3, "algorithmic_bytes": alg_bytes}
    else:                                                              # --rows beyond the decode range: the tensor cores bound it
        tpeak, tkind = measured_peak("bf16_tflops", 1590.0)
        tflops = 2.0 * M * n_local * K_DIM / (kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": tflops, "peak": tpeak, "unit": "TFLOP/s", "frac": tflops / tpeak,
                    "traffic": None, "peak_kind": f"of {tkind} (cuBLAS bf16; the product runs tcgen05 kind::f16)",
                    "frac_of_nominal_int8": tflops / INT8_NOMINAL_TOPS, "kernel": "w4a4 product", "kernel_us": kernel_ms * 1e3}

    # ---- end to end through the public ops: host activations in, host result out -------------
    # Requests arrive in pinned host memory and their results return there.  Consecutive requests are
    # independent, so the public helper host_pipeline.HostStreamedLayer overlaps the upload of request i + 1 and
    # the download of request i - 1 with the kernels of request i (three streams, double-buffered device
    # tensors); every request makes its own host -> device -> host trip inside the timed region.  A block of
    # E2E_BLOCK requests is one CUDA Graph; args.steps requests are timed exactly (whole blocks + a remainder).
    from wush_int4_kernel_b200.host_pipeline import HostStreamedLayer
    E2E_BLOCK = 16
    x_host = [synth.draw_activations(M, K_DIM, outliers, gen).cpu().pin_memory() for _ in range(4)]
    y_host = [torch.empty(M, n_local, dtype=torch.float16).pin_memory() for _ in range(E2E_BLOCK)]
    pipe = HostStreamedLayer(t_bf16, M)

    def e2e_block(first, count):
        pipe.run([x_host[(first + k) % 4] for k in range(count)], y_host[:count],
                 [weights[(first + k) % copies] for k in range(count)])

    # block b starts at request b * E2E_BLOCK; inputs repeat with period 4 and weights with period `copies`
    period = (4 * copies // math.gcd(4, copies))
    block_period = period // math.gcd(period, E2E_BLOCK)
    e2e_graphs = [timing.capture(lambda b=b: e2e_block(b * E2E_BLOCK, E2E_BLOCK))[0] for b in range(block_period)]
    whole, rest = divmod(args.steps, E2E_BLOCK)
    rest_graph = timing.capture(lambda: e2e_block(whole * E2E_BLOCK, rest))[0] if rest else None

    # the same request handled alone (upload -> kernels -> download, nothing overlapped): its latency
    x_dev = torch.empty(M, K_DIM, dtype=torch.bfloat16, device=dev)
    y_one = torch.empty(M, n_local, dtype=torch.float16).pin_memory()

    def e2e_single(i):
        x_dev.copy_(x_host[i % 4], non_blocking=True)
        a, b = quantise_activations(x_dev, t_bf16)
        y_one.copy_(w4a4_product(a, b, *weights[i % copies]), non_blocking=True)

    single_graphs = [timing.capture(lambda i=i: e2e_single(i))[0] for i in range(period)]
    for i in range(8):
        single_graphs[i % period].replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(64):
        single_graphs[i % period].replay()
    e1.record()
    torch.cuda.synchronize()
    latency_us = 1e3 * e0.elapsed_time(e1) / 64

    for b in range(max(1, -(-max(args.warmup, 3) // E2E_BLOCK))):
        e2e_graphs[b % block_period].replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in range(whole):
        e2e_graphs[b % block_period].replay()
    if rest_graph is not None:
        rest_graph.replay()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        tmax = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    # the host buffers of the last replay must hold the products of their inputs
    torch.cuda.synchronize()
    last_first, last_count = (whole * E2E_BLOCK, rest) if rest else ((whole - 1) * E2E_BLOCK, E2E_BLOCK)
    e2e_check = True
    for k in range(last_count):
        a, b = quantise_activations(x_host[(last_first + k) % 4].to(dev), t_bf16)
        expect = w4a4_product(a, b, *weights[(last_first + k) % copies]).cpu()
        e2e_check = e2e_check and bool(torch.equal(expect, y_host[k]))
    e2e_tops = 2.0 * M * N_DIM * K_DIM / (e2e_ms / args.steps * 1e-3) / 1e12
    e2e = {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": 2 * M * K_DIM * world,
           "d2h_bytes_per_step": 2 * M * N_DIM, "us_per_step": 1e3 * e2e_ms / args.steps,
           "latency_us_one_request_alone": latency_us,
           "form": f"requests in pinned host memory; per request: H2D copy -> transform+quant -> product -> D2H copy; "
                   f"{E2E_BLOCK} requests per CUDA Graph on three streams (upload of the next and download of the previous "
                   f"request overlap the kernels of the current one: host_pipeline.HostStreamedLayer); "
                   f"`latency_us_one_request_alone` is the same chain with nothing overlapped"}

    # ---- the other half of the metric in the same run: M = 4096 through the same layer --------
    prefill = None
    if not args.no_prefill:
        prefill = measure_prefill(weights, t_bf16, outliers, gen, dev, world, n_local, barrier)

    # ---- tensor-parallel FFN block with its exchange (N > 1) -----------------------------------
    ffn_block = None
    if world > 1 and not args.no_ffn:
        del graphs, prod_graphs, e2e_graphs, single_graphs, rest_graph
        ffn_block = measure_ffn_block(world, rank, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- CPU baseline beside it (rank 0, N=1 only): bounded sample of the same layer ---------
    cpu = None
    if world == 1 and not args.no_cpu:
        t0 = time.perf_counter()
        times, cores = [], os.cpu_count() or 1
        first, cores = time_cpu_layer(M, N_DIM, 1, 1)
        n_rep = int(max(3, min(2000, 12.0 / max(first[0], 1e-3))))
        times, cores = time_cpu_layer(M, N_DIM, n_rep, 0)
        med = statistics.median(times)
        cpu = {"value": 2.0 * M * N_DIM * K_DIM / med / 1e12, "unit": "TOPS", "cores": cores, "cpu": cpu_model(), "kind": "port",
               "sample": f"whole layer M={M}, median of {n_rep} calls ({time.perf_counter() - t0:.1f} s of CPU work)",
               "us_per_step": med * 1e6}

    clocks = sampler.summary() if sampler else None
    line = {
        "metric": "w4a4_layer_eff_tops", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4", "data": "synthetic",
        "config": workload_config(M),
        "setup": {"sharding": f"column parallel, {n_local} columns per GPU" if world > 1 else "single GPU",
                  "l2": f"{copies} rotating copies of the weight shard ({shard_bytes >> 20} MiB each), together > 2x L2",
                  "timing": "CUDA Graph replay of transform+quant -> product, CUDA events, max over ranks",
                  "layer_files": f"{from_cache} of {copies} weight copies loaded from {cache_dir}"},
        "us_per_layer": ms_per_step * 1e3,
        "layer_hbm_frac": algorithmic_bytes_layer(M, n_local, K_DIM) / (ms_per_step * 1e-3) / 1e9 / peak,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "e2e_check": e2e_check, "prefill": prefill, "ffn_block": ffn_block,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--rows", type=int, default=1, help="activation rows M per step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the M=4096 sub-record")
    ap.add_argument("--no-ffn", action="store_true", help="skip the FFN-block sub-record (N > 1)")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 20
        args.warmup = args.warmup if args.warmup is not None else 3
        run_reference_arm(args)
    else:
        args.steps = args.steps if args.steps is not None else 2000
        args.warmup = args.warmup if args.warmup is not None else 20
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
