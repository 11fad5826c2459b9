"""Measurement helpers: CUDA-event timing, L2 flush, clock/throttle sampling with nvidia-smi."""
from __future__ import annotations

import statistics
import subprocess
import threading

import torch

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU every 200 ms while a region runs (read only)."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.rows: list[list[str]] = []
        self._proc = None
        self._thread = None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            for line in self._proc.stdout:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 9:
                    self.rows.append(parts)

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # keep the samples taken under load (upper half) so idle ticks at the edges do not skew the median
        sm_sorted = sorted(sm)
        return {"sm_mhz": statistics.median(sm_sorted), "sm_min_mhz": sm_sorted[0], "sm_max_mhz": max(mx),
                "reasons": sorted(reasons), "samples": len(sm)}


_flush_buf = None


def flush_l2() -> None:
    """Overwrite a 256 MiB buffer (larger than the 126 MB L2) so the next kernel starts cold."""
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    _flush_buf.zero_()


def time_cuda(fn, iters: int = 20, warmup: int = 5, flush: bool = True) -> float:
    """Median milliseconds of fn() measured with CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)
