"""Wall-clock function timers (sync and async) and CUDA-event device timers.

``TimerProfiler.profile(name)`` decorates a function and records call count / total / min / max /
mean of its duration (reference: src/tplr/profilers/timer_profiler.py:10-197).  ``CudaEventTimer``
times a region on the launching stream with CUDA events — the device-side number the benchmarks
report (max over ranks is taken by the caller).
"""

from __future__ import annotations

import asyncio
import functools
import time
from collections import defaultdict

import torch

from ..logging import logger


class TimerProfiler:
    def __init__(self, name: str = "TimerProfiler"):
        self.name = name
        self.timings: dict[str, list[float]] = defaultdict(list)
        self.errors: dict[str, int] = defaultdict(int)
        self.active: dict[str, float] = {}

    def _record_timing(self, name: str, elapsed: float, error: bool = False) -> None:
        """One finished call of ``name``; a call that raised is timed too and counted as an error."""
        self.timings[name].append(elapsed)
        if error:
            self.errors[name] += 1

    def start_timer(self, name: str) -> None:
        self.active[name] = time.perf_counter()

    def end_timer(self, name: str) -> float:
        t0 = self.active.pop(name, None)
        if t0 is None:
            return 0.0
        dt = time.perf_counter() - t0
        self.timings[name].append(dt)
        return dt

    def profile(self, func_name: str | None = None):
        def deco(fn):
            label = func_name or fn.__qualname__
            if asyncio.iscoroutinefunction(fn):
                @functools.wraps(fn)
                async def awrap(*a, **kw):
                    t0, failed = time.perf_counter(), True
                    try:
                        out = await fn(*a, **kw)
                        failed = False
                        return out
                    finally:
                        self._record_timing(label, time.perf_counter() - t0, error=failed)
                return awrap

            @functools.wraps(fn)
            def wrap(*a, **kw):
                t0, failed = time.perf_counter(), True
                try:
                    out = fn(*a, **kw)
                    failed = False
                    return out
                finally:
                    self._record_timing(label, time.perf_counter() - t0, error=failed)
            return wrap
        return deco

    def get_stats(self, func_name: str | None = None) -> dict:
        """Per function: count, errors, total / min / max / mean seconds (``avg`` is the same number under the
        reference's key) and the last ten durations."""
        def one(k, v):
            if not v:
                return {}
            mean = sum(v) / len(v)
            return {"function": k, "count": len(v), "errors": self.errors.get(k, 0), "total": sum(v), "min": min(v),
                    "max": max(v), "mean": mean, "avg": mean, "timings": v[-10:]}
        if func_name is not None:
            return one(func_name, self.timings.get(func_name, []))
        return {k: one(k, v) for k, v in self.timings.items()}

    def log_summary(self) -> None:
        for k, s in sorted(self.get_stats().items(), key=lambda kv: -kv[1].get("total", 0)):
            logger.info(f"[{self.name}] {k}: n={s['count']} errors={s['errors']} total={s['total']:.3f}s mean={s['mean'] * 1e3:.2f}ms "
                        f"min={s['min'] * 1e3:.2f}ms max={s['max'] * 1e3:.2f}ms")

    def reset(self, func_name: str | None = None) -> None:
        if func_name is None:
            self.timings.clear()
            self.errors.clear()
            self.active.clear()
        else:
            self.timings.pop(func_name, None)
            self.errors.pop(func_name, None)


class DummyTimerProfiler:
    """No-op with the same surface."""

    def __init__(self, *a, **k):
        self.timings = {}

    def start_timer(self, name): return None
    def end_timer(self, name): return 0.0
    def _record_timing(self, *a, **k): return None
    def get_stats(self, func_name=None): return {}
    def log_summary(self): return None
    def reset(self, func_name=None): return None

    def profile(self, func_name=None):
        return lambda fn: fn


class CudaEventTimer:
    """``with CudaEventTimer() as t: ...`` then ``t.ms`` (synchronises on exit)."""

    def __init__(self, stream=None):
        self.stream, self.ms = stream, None

    def __enter__(self):
        self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._e0.record(self.stream)
        return self

    def __exit__(self, *exc):
        self._e1.record(self.stream)
        self._e1.synchronize()
        self.ms = self._e0.elapsed_time(self._e1)
        return False
