"""Device-side timing helpers.

All numbers are taken with CUDA events on the launching stream after warm-up, with a
synchronise on both sides, and either an L2 flush between iterations or inputs larger than
the 126 MB L2. Multi-rank numbers are reduced with MAX over ranks.
"""

from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Callable

import torch

L2_BYTES = 126 * 1024 * 1024
_flush_buf: dict[int, torch.Tensor] = {}


def flush_l2(device: torch.device | None = None) -> None:
    """Overwrite a buffer larger than L2 so the next kernel starts from a cold cache."""
    dev = torch.device(device or "cuda").index or torch.cuda.current_device()
    if dev not in _flush_buf:
        _flush_buf[dev] = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=f"cuda:{dev}")
    _flush_buf[dev].zero_()


def time_cuda(fn: Callable[[], None], iters: int = 20, warmup: int = 3, flush: bool = True) -> dict:
    """Return per-iteration device milliseconds (median/min/mean) of ``fn``."""
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return {"median_ms": statistics.median(times), "min_ms": min(times), "mean_ms": statistics.fmean(times), "iters": iters}


def max_over_ranks(value: float) -> float:
    """MAX-reduce a device-timed number over the default process group (no-op single rank)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class ClockSampler:
    """Samples SM clocks and throttle reasons with ``nvidia-smi`` while a timed region runs.

    Read-only: never changes a GPU setting.
    """

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int = 0, period_ms: int = 200) -> None:
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.rows: list[list[str]] = []
        self._proc: subprocess.Popen | None = None
        self._thread: threading.Thread | None = None

    def start(self) -> "ClockSampler":
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except (FileNotFoundError, OSError):
            self._proc = None
            return self
        self._thread = threading.Thread(target=self._pump, daemon=True)
        self._thread.start()
        return self

    def _pump(self) -> None:
        assert self._proc is not None and self._proc.stdout is not None
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0)
            self._proc.terminate()  # the exact child we started, never a pattern kill
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


class PhaseTimer:
    """Per-phase timing of a training step (rollout / fwd-bwd / optim / sync): wall clock always, plus the device
    time between CUDA events when a GPU is in use, plus an NVTX range per phase so the phases show up in a
    timeline profile. ``with timer.phase("rollout"): ...``; ``timer.summary()`` -> ``{"rollout_s": .., "rollout_dev_ms": ..}``."""

    def __init__(self, device=None, nvtx: bool = True):
        import torch

        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.nvtx = nvtx and self.cuda
        self.wall: dict[str, float] = {}
        self._events: dict[str, list] = {}

    def phase(self, name: str):
        return _Phase(self, name)

    def summary(self) -> dict[str, float]:
        import torch

        out = {f"{k}_s": v for k, v in self.wall.items()}
        if self.cuda:
            torch.cuda.synchronize()
            for k, pairs in self._events.items():
                out[f"{k}_dev_ms"] = float(sum(a.elapsed_time(b) for a, b in pairs))
        return out

    def reset(self) -> None:
        self.wall.clear()
        self._events.clear()


class _Phase:
    def __init__(self, timer: PhaseTimer, name: str):
        self.t, self.name = timer, name

    def __enter__(self):
        import torch

        if self.t.nvtx:
            torch.cuda.nvtx.range_push(self.name)
        if self.t.cuda:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        self.w0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        import torch

        self.t.wall[self.name] = self.t.wall.get(self.name, 0.0) + time.perf_counter() - self.w0
        if self.t.cuda:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.t._events.setdefault(self.name, []).append((self.e0, e1))
        if self.t.nvtx:
            torch.cuda.nvtx.range_pop()
        return False
