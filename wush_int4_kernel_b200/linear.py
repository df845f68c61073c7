"""W4A4 linear layer on top of the ``_C`` operators: the M-dispatch the reference leaves to its
callers (``bench/exp_p13_official.py:31-39``, ``scripts/run_sm100.py:78-89``) and the
column- / row-parallel variants for 1/2/4/8 GPUs of one node.

Sharding (none exists in the reference; the composition is pinned by the single-op semantics):

* column parallel -- the rows of ``wq`` / ``ws`` (= columns of Y) are split; X, T and the
  activation quantisation are replicated; no collective unless the caller asks for the full
  row (``gather_output=True`` -> one all-gather of ``(M, N/p)`` fp16 blocks: with a peer
  communicator attached the decode product stores its block straight into every rank's buffer,
  otherwise the library all-gather);
* row parallel -- K is split on multiples of 32 so each rank keeps whole transform blocks and
  whole scale groups; every rank produces a partial ``(M, N)`` product and one all-reduce
  (sum, fp32) finishes it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def shard_bounds(total: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """[start, stop) of ``rank``'s share of ``total`` items, cut on multiples of ``multiple``;
    the first ``rem`` ranks get one extra unit.  Covers ``total`` exactly and in order."""
    if total % multiple:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    units = total // multiple
    base, rem = divmod(units, world)
    start = rank * base + min(rank, rem)
    stop = start + base + (1 if rank < rem else 0)
    return start * multiple, stop * multiple


def _ops():
    from . import _C          # ImportError when the extension is not built: no fallback
    return _C


def quantise_activations(x: torch.Tensor, t: torch.Tensor):
    """bf16 activations -> (codes, scales) through the fused transform+quantisation op."""
    ops = _ops()
    rows = x.numel() // x.shape[-1]
    if rows <= 32:
        return ops.fused_transform_quant_int4_smallm(x, t)
    return ops.fused_transform_quant_int4_v3(x, t)


def w4a4_product(xq, xs, wq, ws):
    """Shape-dispatched product with the reference's per-shape entry points."""
    ops = _ops()
    rows = xq.numel() // xq.shape[-1]
    if rows == 1:
        return ops.w4a4_gemv(xq.reshape(1, -1), xs.reshape(1, -1), wq, ws).reshape(1, -1)
    if rows <= 32:
        return ops.w4a4_gemv_multi(xq, xs, wq, ws)
    return ops.w4a4_gemm_s4(xq, xs, wq, ws)


@dataclass
class W4A4Linear:
    """y = W4A4(x): fused transform+quantisation of x, then the group-scaled product."""
    t: torch.Tensor        # (K/32, 32, 32) bf16
    wq: torch.Tensor       # (N, K/2) uint8
    ws: torch.Tensor       # (N, K/32) bf16

    @property
    def in_features(self) -> int:
        return self.wq.shape[1] * 2

    @property
    def out_features(self) -> int:
        return self.wq.shape[0]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        xq, xs = quantise_activations(x2, self.t)
        return w4a4_product(xq, xs, self.wq, self.ws).reshape(*lead, self.out_features)

    def to(self, device) -> "W4A4Linear":
        return W4A4Linear(self.t.to(device), self.wq.to(device), self.ws.to(device))


class ColumnParallelW4A4Linear:
    """Rank ``rank`` of ``world`` holds output columns ``shard_bounds(N, world, rank, multiple)``."""

    def __init__(self, t, wq, ws, world: int, rank: int, multiple: int = 1, gather_output: bool = False,
                 group=None, peer_gather=None):
        self.full_out = wq.shape[0]
        self.world, self.rank, self.group, self.gather_output = world, rank, group, gather_output
        self.peer_gather = peer_gather          # optional peer_reduce.PeerAllReduce for decode-size results
        self.n0, self.n1 = shard_bounds(self.full_out, world, rank, multiple)
        self.local = W4A4Linear(t, wq[self.n0:self.n1].contiguous(), ws[self.n0:self.n1].contiguous())
        self.bounds = [shard_bounds(self.full_out, world, r, multiple) for r in range(world)]
        self.widths = [b - a for a, b in self.bounds]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if not self.gather_output or self.world == 1:
            return self.local(x)
        lead = x.shape[:-1]
        peer = self.peer_gather
        if peer is not None:
            # at most 32 rows: the product pushes its block into every rank's buffer and the gather is local;
            # larger results that fit a slot: one gather kernel over peer memory
            xq, xs = quantise_activations(x.reshape(-1, x.shape[-1]), self.local.t)
            y = peer.product_allgather(xq, xs, self.local.wq, self.local.ws, self.widths)
            if y is None:
                y = w4a4_product(xq, xs, self.local.wq, self.local.ws)
                y = peer.allgather(y, self.widths) if peer.fits_gather(y.shape[0], self.widths) else \
                    gather_columns(y, self.bounds, self.group)
            return y.reshape(*lead, self.full_out)
        return gather_columns(self.local(x), self.bounds, self.group)


def gather_columns(y_local: torch.Tensor, bounds, group=None) -> torch.Tensor:
    """All-gather of column blocks of unequal width into the full ``(…, N)`` tensor."""
    import torch.distributed as dist

    width = max(b - a for a, b in bounds)
    lead = y_local.shape[:-1]
    if all(b - a == width for a, b in bounds):               # equal blocks: no padding pass
        parts = [torch.empty_like(y_local) for _ in bounds]
        dist.all_gather(parts, y_local.contiguous(), group=group)
        return torch.cat(parts, dim=-1)
    padded = y_local.new_zeros(*lead, width)
    padded[..., : y_local.shape[-1]] = y_local
    parts = [torch.empty_like(padded) for _ in bounds]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[..., : b - a] for p, (a, b) in zip(parts, bounds)], dim=-1)


class RowParallelW4A4Linear:
    """Rank ``rank`` holds K-slice ``shard_bounds(K, world, rank, 32)`` of the weights and the
    matching transform blocks; ``__call__`` takes the local slice of the activations and
    returns the all-reduced product (fp16, summed in fp32)."""

    def __init__(self, t, wq, ws, world: int, rank: int, group=None, reduce_output: bool = True, peer_reduce=None):
        K = wq.shape[1] * 2
        self.world, self.rank, self.group, self.reduce_output = world, rank, group, reduce_output
        self.peer_reduce = peer_reduce          # optional peer_reduce.PeerAllReduce for decode-size results
        self.k0, self.k1 = shard_bounds(K, world, rank, 32)
        self.local = W4A4Linear(t[self.k0 // 32:self.k1 // 32].contiguous(),
                                wq[:, self.k0 // 2:self.k1 // 2].contiguous(),
                                ws[:, self.k0 // 32:self.k1 // 32].contiguous())

    def __call__(self, x_local: torch.Tensor) -> torch.Tensor:
        lead = x_local.shape[:-1]
        xq, xs = quantise_activations(x_local.reshape(-1, x_local.shape[-1]), self.local.t)
        return self.product_and_reduce(xq, xs).reshape(*lead, self.local.out_features)

    def product_and_reduce(self, xq: torch.Tensor, xs: torch.Tensor) -> torch.Tensor:
        """Local product of already quantised activations, then the sum over ranks; at most 32
        rows with a peer communicator attached run as the fused product + exchange chain."""
        peer = getattr(self, "peer_reduce", None)
        if peer is not None and self.reduce_output and self.world > 1:
            y = peer.product_allreduce(xq, xs, self.local.wq, self.local.ws)
            if y is not None:
                return y
        return self.reduce(w4a4_product(xq, xs, self.local.wq, self.local.ws))

    def reduce(self, y: torch.Tensor) -> torch.Tensor:
        """All-reduce (sum in fp32) of this rank's partial product."""
        if not self.reduce_output or self.world == 1:
            return y
        peer = getattr(self, "peer_reduce", None)
        if peer is not None and peer.fits(y):
            return peer(y)                      # one kernel over NVLink peer memory (same fp32 sum of the fp16 partials)
        import torch.distributed as dist

        acc = y.float()
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        return acc.to(torch.float16)


class TensorParallelFFN:
    """Llama-style FFN block: fused gate+up (column parallel, gate and up halves of the same
    intermediate index on the same rank) -> SiLU(gate) * up -> bf16 -> down (row parallel)."""

    def __init__(self, gate_up: tuple, down: tuple, world: int, rank: int, group=None):
        t_gu, wq_gu, ws_gu = gate_up           # rows [0, I) = gate, [I, 2I) = up
        t_d, wq_d, ws_d = down                 # (hidden, I/2) codes
        inter = wq_gu.shape[0] // 2
        self.i0, self.i1 = shard_bounds(inter, world, rank, 32)
        rows = torch.cat((torch.arange(self.i0, self.i1), torch.arange(inter + self.i0, inter + self.i1)))
        rows = rows.to(wq_gu.device)
        self.gate_up = W4A4Linear(t_gu, wq_gu[rows].contiguous(), ws_gu[rows].contiguous())
        self.down = RowParallelW4A4Linear.__new__(RowParallelW4A4Linear)
        self.down.world, self.down.rank, self.down.group, self.down.reduce_output = world, rank, group, True
        self.down.peer_reduce = None
        self.down.k0, self.down.k1 = self.i0, self.i1
        self.down.local = W4A4Linear(t_d[self.i0 // 32:self.i1 // 32].contiguous(),
                                     wq_d[:, self.i0 // 2:self.i1 // 2].contiguous(),
                                     ws_d[:, self.i0 // 32:self.i1 // 32].contiguous())

    @classmethod
    def from_local_shards(cls, gate_up: tuple, down: tuple, world: int, rank: int, group=None) -> "TensorParallelFFN":
        """Builds the block from tensors that are ALREADY this rank's shards (gate rows then up
        rows of the local intermediate slice; down-projection columns of the same slice), so a
        rank never has to hold the unsharded layer."""
        self = cls(gate_up, down, world=1, rank=0, group=group)
        self.down.world, self.down.rank = world, rank
        return self

    def use_peer_reduce(self, peer_reduce) -> None:
        """Finish small results with ``peer_reduce.PeerAllReduce`` instead of the library all-reduce."""
        self.down.peer_reduce = peer_reduce

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        gu = self.gate_up(x)
        # SiLU(gate) * up -> bf16 -> transform -> quantise in one kernel: h never goes to HBM
        lead = gu.shape[:-1]
        hq, hs = _ops().fused_silu_mul_transform_quant_int4(gu.reshape(-1, gu.shape[-1]), self.down.local.t)
        return self.down.product_and_reduce(hq, hs).reshape(*lead, self.down.local.out_features)

    def reference_call(self, x: torch.Tensor) -> torch.Tensor:
        """The same block as a composition of the single ops (separate activation kernels)."""
        gu = self.gate_up(x)
        half = gu.shape[-1] // 2
        h = (torch.nn.functional.silu(gu[..., :half].float()) * gu[..., half:].float()).to(torch.bfloat16)
        return self.down(h.contiguous())
