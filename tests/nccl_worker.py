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
    dist.barrier()
    print(f"rank {rank} ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
