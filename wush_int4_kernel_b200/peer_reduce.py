"""One-shot all-reduce and all-gather of small fp16 products over NVLink peer memory: the Python face
of the ``wush_comm_*`` entry points (``csrc/peer_reduce.cu``).  The reference is single-GPU and has
nothing like it; here the sum finishes the row-parallel down projection of the tensor-parallel FFN
block and the gather a column-parallel layer whose caller needs the full row, at decode sizes,
where a library collective costs several times the sharded product.

One process per GPU of ONE node.  Construction is collective over ``group`` (it exchanges CUDA IPC
handles through ``torch.distributed``); calls are one kernel launch on the current stream and
may be captured in a CUDA Graph.  Every rank must make the same sequence of calls.
"""
from __future__ import annotations

import ctypes

import torch

from . import capi


class PeerAllReduce:
    TWO_PHASE_BYTES = 1 << 20

    def __init__(self, max_elements: int, group=None):
        import torch.distributed as dist

        self.lib = capi.load()
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.slot_bytes = (2 * max_elements + 255) // 256 * 256
        self.max_elements = max_elements
        comm = ctypes.c_void_p()
        capi.check(self.lib.wush_comm_create(self.rank, self.world, self.slot_bytes, ctypes.byref(comm)), "comm_create")
        self.comm = comm
        handle = ctypes.create_string_buffer(64)
        capi.check(self.lib.wush_comm_export(self.comm, handle), "comm_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        for r, h in enumerate(handles):
            if r != self.rank:
                capi.check(self.lib.wush_comm_connect(self.comm, r, ctypes.create_string_buffer(h, 64)), "comm_connect")
        dist.barrier(group=group)                   # nobody publishes before everybody has mapped everybody

    def fits(self, y: torch.Tensor) -> bool:
        return (y.dtype == torch.float16 and y.is_cuda and y.is_contiguous() and y.numel() % 8 == 0
                and y.numel() <= self.max_elements)

    def __call__(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum over ranks (fp32 accumulation in rank order, fp16 result) of ``partial``."""
        if not self.fits(partial):
            raise ValueError("PeerAllReduce: needs a contiguous CUDA fp16 tensor of a multiple of 8 elements that fits the slot")
        out = torch.empty_like(partial)
        # a megabyte and more: reduce-scatter + all-gather in one kernel instead of every rank reading everything
        two_phase = self.world > 1 and partial.numel() * 2 >= self.TWO_PHASE_BYTES
        fn = self.lib.wush_comm_allreduce_two_phase_f16 if two_phase else self.lib.wush_comm_allreduce_f16
        capi.check(fn(self.comm, partial.data_ptr(), out.data_ptr(), partial.numel(), torch.cuda.current_stream().cuda_stream),
                   "comm_allreduce_f16")
        return out

    def product_allreduce(self, xq, xs, wq, ws):
        """Decode product (at most 32 activation rows) and the sum over ranks in one chain: the
        product kernel pushes its result into every rank's buffer (the CUDA-core GEMV up to two
        rows, the tensor-core streaming kernel up to 32 where K % 256 == 0).  Returns ``None`` for
        shapes outside those kernels' range (the caller then uses the product op followed by
        ``__call__``)."""
        K = wq.shape[1] * 2
        rows, n = xq.numel() // (K // 2), wq.shape[0]
        by_gemv = rows <= 2 and rows * (K // 32) * 36 <= 200 * 1024
        by_stream = rows <= 32 and K % 256 == 0 and xs.data_ptr() % 16 == 0 and ws.data_ptr() % 16 == 0
        if not (by_gemv or by_stream) or (rows * n) % 8 or rows * n > self.max_elements:
            return None
        out = torch.empty(rows, n, dtype=torch.float16, device=xq.device)
        capi.check(self.lib.wush_comm_gemv_allreduce(self.comm, xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(),
                                                     rows, n, K, out.data_ptr(), torch.cuda.current_stream().cuda_stream),
                   "comm_gemv_allreduce")
        return out

    def _widths(self, widths):
        if len(widths) != self.world:
            raise ValueError(f"PeerAllReduce: {len(widths)} widths for a world of {self.world}")
        return (ctypes.c_int64 * self.world)(*[int(w) for w in widths])

    def fits_gather(self, rows: int, widths) -> bool:
        return all(w > 0 and w % 8 == 0 and rows * w <= self.max_elements for w in widths)

    def allgather(self, y_local: torch.Tensor, widths) -> torch.Tensor:
        """All-gather of column blocks: ``y_local`` is this rank's contiguous ``(rows, widths[rank])``
        fp16 block, the result the ``(rows, sum(widths))`` matrix with all ranks' blocks in rank order."""
        rows = y_local.numel() // y_local.shape[-1]
        if (y_local.dtype != torch.float16 or not y_local.is_cuda or not y_local.is_contiguous()
                or y_local.shape[-1] != widths[self.rank] or not self.fits_gather(rows, widths)):
            raise ValueError("PeerAllReduce.allgather: needs contiguous CUDA fp16 blocks whose widths are multiples of 8 and fit the slot")
        out = torch.empty(*y_local.shape[:-1], sum(widths), dtype=torch.float16, device=y_local.device)
        capi.check(self.lib.wush_comm_allgather_f16(self.comm, y_local.data_ptr(), out.data_ptr(), rows, self._widths(widths),
                                                    torch.cuda.current_stream().cuda_stream), "comm_allgather_f16")
        return out

    def product_allgather(self, xq, xs, wq, ws, widths):
        """Column-parallel decode product (at most 32 activation rows) and the all-gather of its column
        blocks in one chain: the product kernel pushes this rank's block into every rank's buffer.
        Returns ``None`` for shapes outside the pushed kernels' range."""
        K = wq.shape[1] * 2
        rows = xq.numel() // (K // 2)
        by_gemv = rows <= 2 and rows * (K // 32) * 36 <= 200 * 1024
        by_stream = rows <= 32 and K % 256 == 0 and xs.data_ptr() % 16 == 0 and ws.data_ptr() % 16 == 0
        if not (by_gemv or by_stream) or wq.shape[0] != widths[self.rank] or not self.fits_gather(rows, widths):
            return None
        out = torch.empty(rows, sum(widths), dtype=torch.float16, device=xq.device)
        capi.check(self.lib.wush_comm_gemv_allgather(self.comm, xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(),
                                                     rows, K, self._widths(widths), out.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream), "comm_gemv_allgather")
        return out

    def error(self) -> int:
        """1 if a bounded wait for a peer ever ran out on this rank (synchronises the device)."""
        torch.cuda.synchronize()
        e = ctypes.c_int(0)
        capi.check(self.lib.wush_comm_error(self.comm, ctypes.byref(e)), "comm_error")
        return int(e.value)

    def close(self) -> None:
        if self.comm is not None:
            import torch.distributed as dist

            torch.cuda.synchronize()
            dist.barrier(group=self.group)          # no peer may still be reading this rank's slots
            self.lib.wush_comm_destroy(self.comm)
            self.comm = None
