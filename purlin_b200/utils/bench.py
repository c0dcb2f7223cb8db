"""Benchmark harness: device-timed sweeps, max over ranks, NCCL baseline, CSV rows.

Method kept from the reference's harness (csrc/support/purlin/benchmark/benchmark.cuh:156-214 and
purlin_report.cuh:21-41): barrier, warm-up launches, CUDA events around ``runs`` back-to-back launches (or
replays of a captured CUDA graph), result = max over ranks, one untimed exact-correctness run per size with
seeded inputs.  The reference prints algorithm bandwidth (logical bytes / time); bus bandwidth is added here
with the usual factors (all-reduce 2(n-1)/n on per-rank bytes; the others (n-1)/n on total bytes).
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist

CSV_HEADER = "collective,impl,world,totalBytes,datatype,lat(us),algbw(GB/s),busbw(GB/s),error(%),GPUName,warmup,runs,graph_launches"


@dataclass
class Timing:
    us: float          # per launch, max over ranks
    runs: int
    graph: int


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next timed launch starts cold."""

    def __init__(self, device, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.fill_(1)


def measure(fn: Callable[[], None], warmup: int = 5, runs: int = 20, graph_launches: int = 0, group=None,
            flush: Optional[L2Flusher] = None) -> Timing:
    """Device time of one call of ``fn`` in microseconds, as the max over the ranks of ``group``."""
    dev = torch.cuda.current_device()
    if graph_launches:
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()   # lazy initialisation outside capture
            s.synchronize()
            with torch.cuda.graph(g, stream=s):
                for _ in range(runs):
                    fn()
        launch = g.replay
        reps, per = graph_launches, runs
    else:
        launch = fn
        reps, per = runs, 1
    for _ in range(warmup if not graph_launches else 1):
        launch()
    torch.cuda.synchronize(dev)
    if dist.is_initialized():
        dist.barrier(group)
    torch.cuda.synchronize(dev)
    if flush is not None and not graph_launches:
        # per-iteration events so the flush itself is not timed
        total = 0.0
        for _ in range(reps):
            flush()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            launch()
            b.record()
            b.synchronize()
            total += a.elapsed_time(b)
        ms = total
    else:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            launch()
        b.record()
        b.synchronize()
        ms = a.elapsed_time(b)
    t = torch.tensor([ms * 1000.0 / (reps * per)], dtype=torch.float64, device=f"cuda:{dev}")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return Timing(float(t.item()), reps * per, graph_launches)


def bus_factor(collective: str, world: int) -> float:
    if world <= 1:
        return 1.0
    return 2.0 * (world - 1) / world if collective in ("ar", "all_reduce") else (world - 1) / world


def logical_bytes(collective: str, per_rank_bytes: int, world: int) -> int:
    """Bytes the reference's benches report: all-reduce = per-rank payload, the others = per-rank x world."""
    return per_rank_bytes if collective in ("ar", "all_reduce") else per_rank_bytes * world


def csv_row(collective, impl, world, total_bytes, dtype, t: Timing, err_pct=0.0):
    alg = total_bytes / 1e9 / (t.us * 1e-6) if t.us > 0 else 0.0
    bus = alg * bus_factor(collective, world)
    name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    return f"{collective},{impl},{world},{total_bytes},{dtype},{t.us:.2f},{alg:.2f},{bus:.2f},{err_pct:.3f},{name},-,{t.runs},{t.graph}"


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mult = 1
    for suf, m in (("KB", 1 << 10), ("MB", 1 << 20), ("GB", 1 << 30), ("K", 1 << 10), ("M", 1 << 20), ("G", 1 << 30)):
        if s.endswith(suf):
            mult, s = m, s[: -len(suf)]
            break
    return int(float(s) * mult)


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while a timed region runs (read-only).

    NVML is initialised in the constructor, outside the timed region, so the sampling thread spends the region
    sampling. One sampler can bracket several regions (``with sampler: ...`` more than once); samples accumulate.
    """

    def __init__(self, index: int = 0, period_s: float = 0.001):
        import threading
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = 0
        self._threading = threading
        self._stop = threading.Event()
        self._thread = None
        self._nvml = self._handle = None
        self._names = {}
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = self._handle_for(pynvml, self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            self._names = {
                pynvml.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
                pynvml.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                pynvml.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                pynvml.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            }
            self._sample()   # the calls are warm before the region starts; this sample is dropped
            self.samples.clear()
            self.reasons.clear()
        except Exception as e:   # NVML missing: report that instead of clocks
            self._nvml = None
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    @staticmethod
    def _handle_for(pynvml, cuda_index):
        """NVML handle of a CUDA device: by UUID (CUDA_VISIBLE_DEVICES may renumber devices), else by index."""
        try:
            uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:
            return pynvml.nvmlDeviceGetHandleByIndex(cuda_index)

    def _sample(self):
        self.samples.append(self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM))
        r = self._nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        for bit, n in self._names.items():
            if r & bit:
                self.reasons.add(n)

    def _run(self):
        try:
            while not self._stop.is_set():
                self._sample()
                self._stop.wait(self.period)
        except Exception as e:
            self.reasons.add(f"nvml_error:{type(e).__name__}")

    def __enter__(self):
        if self._nvml is not None:
            self._stop.clear()
            self._thread = self._threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(2.0)
            self._thread = None

    def summary(self) -> dict:
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else 0
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}
