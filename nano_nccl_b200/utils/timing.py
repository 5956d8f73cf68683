"""Device-side timing helpers: CUDA-event loops with L2 flushes, percentiles, max over ranks, and
a background sampler of SM clocks and throttle reasons."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable, Optional

import torch

L2_BYTES = 126 * 1024 * 1024


class L2Flusher:
    """Writes a buffer larger than L2 so the next timed iteration starts cold."""

    def __init__(self, device=None, nbytes: int = 2 * L2_BYTES):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")

    def __call__(self):
        self.buf.zero_()


def time_iterations(fn: Callable[[], None], iters: int, warmup: int, flush: Optional[Callable[[], None]] = None,
                    pre: Optional[Callable[[], None]] = None, head_start_ms: float = 3.0) -> list[float]:
    """Times each of `iters` calls of fn() with CUDA events on the current stream; returns µs."""
    for _ in range(warmup):
        if flush:
            flush()
        if pre:
            pre()
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    # Keep the GPU busy for a few milliseconds first, so that the host enqueues the whole timed loop ahead of the
    # device: otherwise a short kernel is timed from its start event to whenever the host gets round to launching
    # it, and the figure measures the host (a bounded spin, not a wait on anything).
    torch.cuda._sleep(int(head_start_ms * 1.9e6))
    for i in range(iters):
        if flush:
            flush()
        if pre:
            pre()
        starts[i].record()
        fn()
        stops[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) * 1e3 for s, e in zip(starts, stops)]


def p50(values: list[float]) -> float:
    return statistics.median(values)


def max_over_ranks(value: float) -> float:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.lines: list[str] = []
        self._thread: Optional[threading.Thread] = None

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self

        def pump():
            assert self.proc is not None and self.proc.stdout is not None
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        if self.proc is not None:
            time.sleep(self.period_ms / 1000.0)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}
