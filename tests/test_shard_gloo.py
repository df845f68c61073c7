"""Two CPU ranks over gloo: the column-parallel all-gather and the row-parallel all-reduce
compositions reproduce the unsharded product.  The per-rank products come from the CPU
oracle (test infrastructure); what is under test is the host-side sharding logic of
wush_int4_kernel_b200.linear (bounds, gather order, reduction)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import w4a4_oracle as orc
        from wush_int4_kernel_b200 import synth
        from wush_int4_kernel_b200.linear import gather_columns, shard_bounds

        orc.set_threads(1)
        K, N, M = 256, 320, 5
        layer = synth.make_layer(K, N, seed=1)
        gen = torch.Generator().manual_seed(2)
        x = synth.draw_activations(M, K, layer.outliers, gen)
        xq, xs = orc.fused_tq(orc.bits(x), orc.bits(layer.t_bf16))
        full = orc.gemm_f16(xq, xs, layer.wq.numpy(), orc.bits(layer.ws))

        # column parallel: unequal shards (320 = 3 + 2 units of 64) and an all-gather
        bounds = [shard_bounds(N, world, r, 64) for r in range(world)]
        n0, n1 = bounds[rank]
        local = orc.gemm_f16(xq, xs, layer.wq[n0:n1].numpy(), orc.bits(layer.ws[n0:n1]))
        y = gather_columns(orc.from_bits(local, torch.float16), bounds)
        ok_col = np.array_equal(orc.bits(y), full)
        # equal shards (the first 256 columns as 2 + 2 units of 64): the gather without the padding pass
        eq_bounds = [shard_bounds(256, world, r, 64) for r in range(world)]
        e0, e1 = eq_bounds[rank]
        y_eq = gather_columns(orc.from_bits(full[:, e0:e1].copy(), torch.float16), eq_bounds)
        ok_col = ok_col and np.array_equal(orc.bits(y_eq), full[:, :256])

        # row parallel: K split on whole groups, partial products summed in fp32
        k0, k1 = shard_bounds(K, world, rank, 32)
        part = orc.gemm_f64(xq[:, k0 // 2:k1 // 2], xs[:, k0 // 32:k1 // 32],
                            layer.wq[:, k0 // 2:k1 // 2].contiguous().numpy(),
                            orc.bits(layer.ws[:, k0 // 32:k1 // 32].contiguous()))
        acc = torch.from_numpy(part).float()
        dist.all_reduce(acc)
        y64 = orc.gemm_f64(xq, xs, layer.wq.numpy(), orc.bits(layer.ws))
        rel = float(np.linalg.norm(acc.double().numpy() - y64) / np.linalg.norm(y64))
        ret[rank] = (ok_col, rel)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_sharding():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        ok_col, rel = ret[rank]
        assert ok_col, f"rank {rank}: gathered columns differ from the unsharded product"
        assert rel < 1e-6, (rank, rel)
