"""Device-side timing helpers: CUDA events on the launching stream, max over ranks, an L2
flush, and a background sampler of SM clocks and throttle reasons.

Method of the reference for comparison: 10 warm-up launches, 3 timed ones, per-kernel device
time from the profiler, mean of the three, one process's numbers only
(examples/dynamic_tiling/include/info.h:22-23, examples/dynamic_tiling/utils/process_data.py:32-58).
Here the figure is the max over ranks.
"""
from __future__ import annotations

import csv
import io
import os
import shutil
import statistics
import subprocess
import tempfile
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

_L2_BYTES = 126 * 1024 * 1024
_flush_buf: Dict[int, torch.Tensor] = {}


def flush_l2(device: torch.device) -> None:
    """Overwrites a buffer twice the size of L2 so that the next kernel starts cold."""
    key = device.index or 0
    buf = _flush_buf.get(key)
    if buf is None:
        buf = torch.empty(2 * _L2_BYTES, dtype=torch.uint8, device=device)
        _flush_buf[key] = buf
    buf.zero_()


def max_over_ranks(value: float, device: torch.device, group=None) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.get_backend(group) == "gloo":
        t = t.cpu()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sync_all(device: torch.device, group=None) -> None:
    torch.cuda.synchronize(device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)
    torch.cuda.synchronize(device)


def time_steps(step: Callable[[], object], steps: int, warmup: int, device: torch.device, group=None,
               flush: bool = False) -> float:
    """Milliseconds per step, device-timed, max over ranks. With ``flush`` every step is timed
    on its own after an L2 flush (the flush itself is outside the timed interval)."""
    for _ in range(warmup):
        step()
    sync_all(device, group)
    if not flush:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step()
        stop.record()
        sync_all(device, group)
        ms = start.elapsed_time(stop) / steps
    else:
        total = 0.0
        for _ in range(steps):
            flush_l2(device)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            step()
            stop.record()
            torch.cuda.synchronize(device)
            total += start.elapsed_time(stop)
        sync_all(device, group)
        ms = total / steps
    return max_over_ranks(ms, device, group)


class ClockSampler:
    """Samples ``nvidia-smi`` every 200 ms while a timed region runs (start before, stop after).

    ``summary()`` gives the median SM clock under load, the maximum SM clock and the throttle
    reasons that were active in any sample."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: Optional[int] = None, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc: Optional[subprocess.Popen] = None
        self._file = None

    def start(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self._file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        cmd = [exe, "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", str(self.period_ms)]
        if self.gpu_index is not None:
            cmd += ["-i", str(self.gpu_index)]
        try:
            self._proc = subprocess.Popen(cmd, stdout=self._file, stderr=subprocess.DEVNULL)
        except OSError:
            self._proc = None
        return self

    def stop(self) -> None:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            self._proc = None

    def summary(self) -> Dict[str, object]:
        self.stop()
        out: Dict[str, object] = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self._file is None:
            return out
        self._file.flush()
        with open(self._file.name) as fh:
            rows = [r for r in csv.reader(fh) if len(r) >= 9]
        try:
            os.unlink(self._file.name)
        except OSError:
            pass
        clocks: List[float] = []
        loaded: List[float] = []
        reasons = set()
        max_mhz = None
        for r in rows:
            r = [x.strip() for x in r]
            try:
                sm, mx, power = float(r[1]), float(r[2]), float(r[3])
            except ValueError:
                continue
            clocks.append(sm)
            if power > 300.0:
                loaded.append(sm)
            max_mhz = mx if max_mhz is None else max(max_mhz, mx)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        use = loaded or clocks
        if use:
            out["sm_mhz"] = statistics.median(use)
        out["sm_max_mhz"] = max_mhz
        out["reasons"] = sorted(reasons)
        out["samples"] = len(clocks)
        return out
