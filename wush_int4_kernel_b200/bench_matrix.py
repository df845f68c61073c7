"""Measurement matrix over the layer shapes the reference quotes (``bench/exp_p13_official.py:42-63``
draws random tensors of the same shapes; no dataset or checkpoint is involved).

    python -m wush_int4_kernel_b200.bench_matrix [--configs qwen,llama,mid,square,prefill,ffn] [--tp P]
    torchrun --nproc-per-node P -m wush_int4_kernel_b200.bench_matrix --configs ffn

For every (K, N, M) one JSON line with the time of the fused transform+quantisation, of the
product and of the whole layer (each replayed from a CUDA Graph over rotating copies of the
weights so no step finds its weights in L2), the effective TOPS ``2MNK / t`` and the fraction of
the bounding peak: HBM copy bandwidth for M <= 32, dense int8 tensor throughput for M >= 128.
Protocol of the reference (``bench/exp_p13_official.py:15-29,65``): 20 warm-ups, median of 5
batches of 100 (M <= 4), 30 (M <= 256) or 8 replays.

``ffn`` times the Llama-70B FFN block (hidden 8192, intermediate 28672) of ONE tensor-parallel
rank: under torchrun with P ranks including the all-reduce of the down projection, otherwise
(``--tp P``) the compute of rank 0's shard alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

L2_BYTES = 126 << 20
HBM_NOMINAL_GBS = 8000.0
INT8_NOMINAL_TOPS = 4500.0
F16_MEASURED_TFLOPS = 1684.0       # cuBLAS bf16 burst measured on this pool: the ceiling of the fp16-folded product

SHAPES = {                      # name -> (K, N, rows per step)
    "qwen": (4096, 24576, (1, 2, 4, 8, 24, 32)),
    "llama": (8192, 57344, (1, 2, 3, 4, 8, 16, 24, 32)),
    "mid": (8192, 57344, (64, 128, 256)),
    "square": (4096, 4096, (4096,)),
    "prefill": (8192, 57344, (512, 2048, 4096)),
}


def _hbm_peak():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def _reps(M: int) -> int:
    return 100 if M <= 4 else (30 if M <= 256 else 8)


def _median_us(graphs, reps: int) -> float:
    n = len(graphs)
    for i in range(20):
        graphs[i % n].replay()
    out = []
    for _ in range(5):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            graphs[i % n].replay()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / reps * 1e3)
    return statistics.median(out)


def make_copies(K: int, N: int, dev) -> list:
    """Enough independently drawn copies of the layer that consecutive steps never find their
    weights in L2 (at most 8: small layers are L2-resident in any real deployment too)."""
    from . import _C, synth

    shard = N * (K // 2 + K // 16)
    copies = max(2, min(8, -(-(2 * L2_BYTES + shard) // shard)))
    return [synth.make_layer(K, N, seed=11 + c, device=str(dev), quantiser=_C.quant_int4) for c in range(copies)]


def measure_layer(layers: list, M: int, dev) -> dict:
    from . import synth, timing
    from .linear import quantise_activations, w4a4_product

    K, N, copies = layers[0].K, layers[0].N, len(layers)
    gen = torch.Generator(device=dev).manual_seed(5)
    x = synth.draw_activations(M, K, layers[0].outliers, gen)
    xq, xs = quantise_activations(x, layers[0].t_bf16)
    reps = _reps(M)
    t_fused = _median_us([timing.capture(lambda l=l: quantise_activations(x, l.t_bf16))[0] for l in layers], reps)
    t_prod = _median_us([timing.capture(lambda l=l: w4a4_product(xq, xs, l.wq, l.ws))[0] for l in layers], reps)
    t_layer = _median_us(
        [timing.capture(lambda l=l: w4a4_product(*quantise_activations(x, l.t_bf16), l.wq, l.ws))[0] for l in layers], reps)
    ops = 2.0 * M * N * K
    layer_bytes = 2 * M * K + 64 * K + 2 * (9 * M * K // 16) + 9 * N * K // 16 + 2 * M * N
    peak, kind = _hbm_peak()
    line = {"K": K, "N": N, "M": M, "fused_tq_us": round(t_fused, 2), "product_us": round(t_prod, 2),
            "layer_us": round(t_layer, 2), "eff_tops": round(ops / t_layer / 1e6, 2), "weight_copies": copies, "reps": reps}
    if M <= 32:
        gbs = layer_bytes / t_layer / 1e3
        line.update(bound="hbm", layer_bytes=layer_bytes, layer_gbs=round(gbs, 1),
                    frac_of_hbm=round(gbs / peak, 3), hbm_peak_kind=kind, frac_of_nominal_hbm=round(gbs / HBM_NOMINAL_GBS, 3))
    else:
        tops = ops / t_prod / 1e6
        line.update(bound="tensor", product_tops=round(tops, 1), frac_of_measured_f16=round(tops / F16_MEASURED_TFLOPS, 3),
                    frac_of_nominal_int8=round(tops / INT8_NOMINAL_TOPS, 3))
    return line


def build_ffn_layers(tp: int, rank: int, dev, copies: int) -> list:
    """``copies`` independently drawn (gate+up, down) shard pairs of rank ``rank`` of ``tp``: rotating
    copies, so consecutive steps stream different weights."""
    from . import _C, synth
    from .linear import shard_bounds

    hidden, inter = 8192, 28672
    i0, i1 = shard_bounds(inter, tp, rank, 32)
    il = i1 - i0
    return [(synth.make_layer(hidden, 2 * il, seed=100 + 10 * c + rank, device=str(dev), quantiser=_C.quant_int4),
             synth.make_layer(il, hidden, seed=200 + 10 * c + rank, device=str(dev), quantiser=_C.quant_int4))
            for c in range(copies)]


def measure_ffn(M: int, tp: int, rank: int, dev, distributed: bool, peer=None, layers=None) -> dict:
    from . import synth, timing
    from .linear import TensorParallelFFN, shard_bounds

    hidden, inter = 8192, 28672
    i0, i1 = shard_bounds(inter, tp, rank, 32)
    il = i1 - i0
    blocks = []
    for gu, dn in (layers if layers is not None else build_ffn_layers(tp, rank, dev, 3 if tp > 1 else 2)):
        ffn = TensorParallelFFN.from_local_shards((gu.t_bf16, gu.wq, gu.ws), (dn.t_bf16, dn.wq, dn.ws), tp, rank)
        ffn.down.reduce_output = distributed
        if peer is not None:
            ffn.use_peer_reduce(peer)
        blocks.append((ffn, gu))
    gen = torch.Generator(device=dev).manual_seed(9)
    x = synth.draw_activations(M, hidden, blocks[0][1].outliers, gen)
    captured = True
    try:
        graphs = [timing.capture(lambda f=f: f(x))[0] for f, _ in blocks]
        t = _median_us(graphs, _reps(M))
    except RuntimeError:                       # a collective that cannot be captured: time eager launches
        captured = False
        torch.cuda.synchronize()
        fns = [f for f, _ in blocks]
        t = timing.median_of(lambda: [f(x) for f in fns], max(2, _reps(M) // len(fns))) / len(fns)
    if distributed:
        import torch.distributed as dist
        tt = torch.tensor([t], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t = float(tt.item())
    ops_total = 2.0 * M * hidden * (2 * inter) + 2.0 * M * inter * hidden
    wbytes = (2 * il * hidden + il * hidden) * 9 // 16
    if not distributed:
        reduce_kind = "none"
    elif peer is None or M * hidden > peer.max_elements:
        reduce_kind = "nccl fp32"
    else:
        pushed = M <= 2 or (M <= 32 and (il) % 256 == 0)
        reduce_kind = ("peer memory, pushed from the product kernel" if pushed else
                       "peer memory, reduce-scatter + all-gather in one kernel" if M * hidden * 2 >= peer.TWO_PHASE_BYTES else
                       "peer memory, one kernel")
    return {"block": "ffn 8192 -> 2 x 28672 -> 8192", "M": M, "tp": tp, "all_reduce": reduce_kind, "graph": captured,
            "us_per_block": round(t, 2), "eff_tops_whole_block": round(ops_total / t / 1e6, 2),
            "weight_bytes_per_rank": wbytes, "weight_stream_gbs_per_rank": round(wbytes / t / 1e3, 1)}


def measure_column_gather(M: int, tp: int, rank: int, dev, peer, layers) -> dict:
    """The gate+up layer column parallel with the full row gathered on every rank (what a caller
    outside an FFN block needs): the product pushing its block into every rank's buffer (``peer``) or
    the library all-gather (``peer`` None).  ``layers``: the pairs of ``build_ffn_layers``."""
    import torch.distributed as dist

    from . import synth, timing
    from .linear import ColumnParallelW4A4Linear

    cols = []
    for gu, _ in layers:
        col = ColumnParallelW4A4Linear.__new__(ColumnParallelW4A4Linear)    # from tensors that already are this rank's shard
        n_loc = gu.wq.shape[0]
        col.world, col.rank, col.group, col.gather_output, col.peer_gather = tp, rank, None, True, peer
        col.full_out, col.widths = n_loc * tp, [n_loc] * tp
        col.bounds = [(r * n_loc, (r + 1) * n_loc) for r in range(tp)]
        from .linear import W4A4Linear
        col.local = W4A4Linear(gu.t_bf16, gu.wq, gu.ws)
        cols.append(col)
    x = synth.draw_activations(M, 8192, layers[0][0].outliers, torch.Generator(device=dev).manual_seed(9))
    captured = True
    try:
        graphs = [timing.capture(lambda c=c: c(x))[0] for c in cols]
        t = _median_us(graphs, _reps(M))
    except RuntimeError:
        captured = False
        torch.cuda.synchronize()
        t = timing.median_of(lambda: [c(x) for c in cols], max(2, _reps(M) // len(cols))) / len(cols)
    tt = torch.tensor([t], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    return {"M": M, "tp": tp, "us_per_layer": round(float(tt.item()), 2), "graph": captured,
            "gather": "library all-gather" if peer is None else
                      ("peer memory, pushed from the product kernel" if M <= 32 else "peer memory, one kernel")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="qwen,llama,square,prefill")
    ap.add_argument("--tp", type=int, default=8, help="tensor-parallel degree emulated by `ffn` on one GPU")
    ap.add_argument("--ffn-rows", default="1,32,2048")
    ap.add_argument("--nccl-only", action="store_true", help="finish the FFN block with the library all-reduce at every size")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from . import _C
    _C.init()
    peer = None
    if world > 1 and not args.nccl_only and "ffn" in args.configs.split(","):
        from .peer_reduce import PeerAllReduce
        peer = PeerAllReduce(max_elements=64 * 8192)           # decode-size results; larger ones go through NCCL
    for name in args.configs.split(","):
        if name == "ffn":
            for m in map(int, args.ffn_rows.split(",")):
                line = measure_ffn(m, world if world > 1 else args.tp, rank if world > 1 else 0, dev, world > 1, peer)
                if rank == 0:
                    print(json.dumps(line), flush=True)
        elif world == 1:
            K, N, rows = SHAPES[name]
            layers = make_copies(K, N, dev)
            for M in rows:
                print(json.dumps(measure_layer(layers, M, dev)), flush=True)
                torch.cuda.empty_cache()
            del layers
    if peer is not None:
        err = peer.error()
        peer.close()
        if err:
            raise SystemExit("peer all-reduce: a bounded wait ran out")
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
