"""A W4A4 layer fed from and drained to pinned host memory, request after request.

The reference's scripts keep activations and results on the device (``bench/exp_p13_official.py:42-63``); a
caller whose requests arrive in host memory pays, per request, an upload of the activations, the two kernels
(transform + quantisation, product) and a download of the result.  Done one after the other that is three
dependent hops per request -- at decode sizes the two copies and their hand-overs cost half as much again as
the kernels.  Here consecutive, independent requests overlap: the upload of request i + 1 and the download of
request i - 1 run on the two copy engines while the kernels of request i run, on three streams with
double-buffered device tensors.  Every request still makes its own host -> device -> host trip.

``run`` forks from the current stream and joins it again, so it can be called eagerly or captured whole into
one CUDA Graph (``torch.cuda.graph``) and replayed.
"""
from __future__ import annotations

import torch

from .linear import quantise_activations, w4a4_product


class HostStreamedLayer:
    """``y_hosts[i] = W4A4(x_hosts[i])`` with the weights ``weights[i]`` (``(wq, ws)`` pairs; one pair serves all
    requests if the list has one entry).  ``depth`` device buffers per direction (2 = double buffering)."""

    def __init__(self, t_bf16: torch.Tensor, rows: int, depth: int = 2):
        if depth < 2:
            raise ValueError("depth must be at least 2")
        self.t = t_bf16
        self.depth = depth
        dev = t_bf16.device
        K = t_bf16.shape[0] * 32
        self.x_dev = [torch.empty(rows, K, dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def run(self, x_hosts, y_hosts, weights) -> None:
        if len(x_hosts) != len(y_hosts):
            raise ValueError("one result buffer per request")
        for x, y in zip(x_hosts, y_hosts):
            if not (x.is_pinned() and y.is_pinned()):
                raise ValueError("requests and results must be in pinned host memory")
        main = torch.cuda.current_stream()
        depth = self.depth
        fork = torch.cuda.Event()
        fork.record(main)
        self.s_in.wait_event(fork)
        self.s_out.wait_event(fork)
        uploaded = [None] * depth          # x_dev[slot] holds its request
        consumed = [None] * depth          # the kernels have read x_dev[slot]
        produced = [None] * depth          # y of the slot is complete
        drained = [None] * depth           # y of the slot has been copied out
        y_dev = [None] * depth             # the product's output, kept alive until its download was ordered
        for i, (x, y) in enumerate(zip(x_hosts, y_hosts)):
            slot = i % depth
            if consumed[slot] is not None:
                self.s_in.wait_event(consumed[slot])
            with torch.cuda.stream(self.s_in):
                self.x_dev[slot].copy_(x, non_blocking=True)
                uploaded[slot] = torch.cuda.Event()
                uploaded[slot].record(self.s_in)
            main.wait_event(uploaded[slot])
            if drained[slot] is not None:
                main.wait_event(drained[slot])       # the output block of this slot may be reused by the allocator
            wq, ws = weights[i % len(weights)]
            xq, xs = quantise_activations(self.x_dev[slot], self.t)
            consumed[slot] = torch.cuda.Event()
            consumed[slot].record(main)              # x_dev[slot] is free once the transform kernel is done
            y_dev[slot] = w4a4_product(xq, xs, wq, ws)
            produced[slot] = torch.cuda.Event()
            produced[slot].record(main)
            self.s_out.wait_event(produced[slot])
            with torch.cuda.stream(self.s_out):
                y.copy_(y_dev[slot].view_as(y), non_blocking=True)
                drained[slot] = torch.cuda.Event()
                drained[slot].record(self.s_out)
        # join: everything this call started is ordered before whatever follows on the caller's stream
        join_in, join_out = torch.cuda.Event(), torch.cuda.Event()
        join_in.record(self.s_in)
        join_out.record(self.s_out)
        main.wait_event(join_in)
        main.wait_event(join_out)
