"""Measurement helpers shared by the benchmark and the profiling targets: CUDA-event timing on
the launching stream, CUDA-Graph capture of a step (the reference times graph replays,
``bench/exp_p13_official.py:15-29``) and an nvidia-smi clock sampler."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time

import torch

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def capture(step, warmups: int = 3):
    """Runs ``step`` a few times on a side stream, then captures it into a CUDA Graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmups):
            out = step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    return graph, out


def time_events(fn, reps: int) -> float:
    """Milliseconds for ``reps`` calls of ``fn`` on the current stream (sync on both sides)."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop)


def median_of(fn, reps: int, batches: int = 5, warmup: int = 20) -> float:
    """Median over ``batches`` of the mean time per call in microseconds."""
    for _ in range(warmup):
        fn()
    return statistics.median(time_events(fn, reps) / reps for _ in range(batches)) * 1e3


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.rows: list[list[str]] = []
        self._proc = None
        self._thread = None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        return self

    def _read(self):
        for line in self._proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 10:
                continue
            try:
                clock, cmax, util = float(r[1]), float(r[2]), float(r[4])
            except ValueError:
                continue
            if util <= 0:
                continue                                   # keep samples taken under load only
            sm.append(clock)
            sm_max.append(cmax)
            for name, val in zip(names, r[6:10]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm)}
