"""Worker of tests/test_gpu_layers.py::test_two_process_nccl_if_available (run under torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from my_int4 import _C
    from wush_int4_kernel_b200 import synth
    from wush_int4_kernel_b200.linear import ColumnParallelW4A4Linear, RowParallelW4A4Linear, W4A4Linear, shard_bounds

    _C.init()
    layer = synth.make_layer(1024, 768, seed=3, device="cuda", quantiser=_C.quant_int4)     # same seed on every rank
    gen = torch.Generator(device="cuda").manual_seed(4)
    x = synth.draw_activations(6, 1024, layer.outliers, gen)
    full = W4A4Linear(layer.t_bf16, layer.wq, layer.ws)(x)
    col = ColumnParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, rank, multiple=32, gather_output=True)
    assert torch.equal(col(x), full), "all-gathered columns differ"
    k0, k1 = shard_bounds(1024, world, rank, 32)
    row = RowParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, rank)
    y = row(x[:, k0:k1].contiguous())
    rel = ((y.float() - full.float()).norm() / full.float().norm()).item()
    assert rel <= 2e-3, rel
    # one-shot all-reduce over peer memory: bit-identical to the fp32 sum of the fp16 partials in rank order,
    # eager and replayed from a CUDA Graph, several steps in a row (the two slots alternate)
    from wush_int4_kernel_b200.peer_reduce import PeerAllReduce
    peer = PeerAllReduce(max_elements=64 * 768)
    gen_r = torch.Generator(device="cuda").manual_seed(100 + rank)
    for step, rows in enumerate([1, 6, 64, 6, 1]):
        part = torch.randn(rows, 768, generator=gen_r, device="cuda").to(torch.float16)
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part)
        acc = torch.zeros(rows, 768, device="cuda")
        for g in gathered:
            acc = acc + g.float()
        got = peer(part)
        assert torch.equal(got, acc.to(torch.float16)), f"peer all-reduce differs at step {step}"
    # results of megabytes take the two-phase kernel (reduce-scatter + all-gather): same bits, mixed with small steps
    big = PeerAllReduce(max_elements=1024 * 768)
    for step, rows in enumerate([1024, 6, 1000, 1024]):
        part = torch.randn(rows, 768, generator=gen_r, device="cuda").to(torch.float16)
        gathered = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(gathered, part)
        acc = torch.zeros(rows, 768, device="cuda")
        for g in gathered:
            acc = acc + g.float()
        assert torch.equal(big(part), acc.to(torch.float16)), f"two-phase all-reduce differs at step {step}"
    assert big.error() == 0
    big.close()
    part = torch.randn(8, 768, generator=gen_r, device="cuda").to(torch.float16)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        warm = peer(part)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        out = peer(part)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, warm), "graph replay differs from the eager call"
    assert peer.error() == 0
    # fused product + exchange (decode rows): equals product followed by the pull all-reduce, bit for bit
    from wush_int4_kernel_b200.linear import quantise_activations, w4a4_product
    for rows in (1, 2, 1, 8, 32, 5):
        xr = synth.draw_activations(rows, 1024, layer.outliers, gen)[:, k0:k1].contiguous()
        shard = RowParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, rank, reduce_output=False)
        xq_l, xs_l = quantise_activations(xr, shard.local.t)
        fused = peer.product_allreduce(xq_l, xs_l, shard.local.wq, shard.local.ws)
        assert fused is not None
        plain = peer(w4a4_product(xq_l, xs_l, shard.local.wq, shard.local.ws))
        assert torch.equal(fused, plain), f"pushed product differs at rows={rows}"
    assert peer.error() == 0
    # all-gather of column blocks over peer memory, equal and unequal widths: the pull kernel and the product that
    # pushes its block, against the library all-gather of the same blocks (bit for bit); several steps, mixed with sums
    for multiple in (32, 256):
        colp = ColumnParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, rank, multiple=multiple, gather_output=True,
                                        peer_gather=peer)
        coln = ColumnParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, rank, multiple=multiple, gather_output=True)
        for rows in (1, 2, 8, 32, 5, 40):
            xr = synth.draw_activations(rows, 1024, layer.outliers, gen)
            want = coln(xr)
            got = colp(xr)
            assert torch.equal(got, want), f"peer all-gather differs at rows={rows}, multiple={multiple}"
            xq_f, xs_f = quantise_activations(xr, layer.t_bf16)
            assert torch.equal(want, w4a4_product(xq_f, xs_f, layer.wq, layer.ws)), "sharded columns differ from the unsharded product"
            blk = w4a4_product(xq_f, xs_f, colp.local.wq, colp.local.ws)
            assert torch.equal(peer.allgather(blk, colp.widths), want), f"pull all-gather differs at rows={rows}"
            assert torch.equal(peer(blk), peer(blk)), "sum between gathers"
    assert peer.error() == 0
    row2 = RowParallelW4A4Linear(layer.t_bf16, layer.wq, layer.ws, world, rank, peer_reduce=peer)
    y2 = row2(x[:, k0:k1].contiguous())
    assert ((y2.float() - full.float()).norm() / full.float().norm()).item() <= 2e-3
    peer.close()
    dist.barrier()
    print(f"rank {rank} ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
