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
    """``timings[name]`` holds the durations of every call, ``counts[name]`` the number of calls and
    ``counts[name + "_errors"]`` how many of them raised; ``active_timers`` the regions opened with
    ``start_timer`` and not closed yet."""

    def __init__(self, name: str = "TimerProfiler"):
        self.name = name
        self.timings: dict[str, list[float]] = defaultdict(list)
        self.counts: dict[str, int] = defaultdict(int)
        self.active_timers: dict[str, float] = {}

    def _record_timing(self, name: str, elapsed: float, error: bool = False) -> None:
        """One finished call of ``name``; a call that raised is timed too and counted as an error."""
        self.timings[name].append(elapsed)
        self.counts[name] += 1
        if error:
            self.counts[f"{name}_errors"] += 1

    def start_timer(self, name: str) -> None:
        self.active_timers[name] = time.perf_counter()

    def end_timer(self, name: str) -> float:
        t0 = self.active_timers.pop(name, None)
        if t0 is None:
            return 0.0
        dt = time.perf_counter() - t0
        self._record_timing(name, dt)
        return dt

    def profile(self, func_name: str | None = None):
        """Decorator for plain and ``async`` functions; the label defaults to the function's name."""
        def deco(fn):
            label = func_name or fn.__name__
            if asyncio.iscoroutinefunction(fn):
                @functools.wraps(fn)
                async def awrap(*a, **kw):
                    t0, failed = time.perf_counter(), True
                    try:
                        out = await fn(*a, **kw)
                        failed = False
                        return out
                    finally:
                        dt = time.perf_counter() - t0
                        self._record_timing(label, dt, error=failed)
                        (logger.error if failed else logger.debug)(f"[TIMER] {self.name}.{label}: {dt:.4f}s"
                                                                   + (" (raised)" if failed else ""))
                return awrap

            @functools.wraps(fn)
            def wrap(*a, **kw):
                t0, failed = time.perf_counter(), True
                try:
                    out = fn(*a, **kw)
                    failed = False
                    return out
                finally:
                    dt = time.perf_counter() - t0
                    self._record_timing(label, dt, error=failed)
                    (logger.error if failed else logger.debug)(f"[TIMER] {self.name}.{label}: {dt:.4f}s"
                                                               + (" (raised)" if failed else ""))
            return wrap
        return deco

    def get_stats(self, func_name: str | None = None) -> dict:
        """One function: count, errors, total / min / max / mean seconds (``avg`` is the same number under the
        reference's key) and the last ten durations, or ``{"error": ...}`` when it was never timed.  Without a
        name: every timed function's statistics."""
        if func_name is None:
            return {k: self.get_stats(k) for k in self.timings}
        v = self.timings.get(func_name, [])
        if not v:
            return {"error": f"No timings found for {func_name}"}
        mean = sum(v) / len(v)
        return {"function": func_name, "count": self.counts[func_name], "errors": self.counts.get(f"{func_name}_errors", 0),
                "total": sum(v), "min": min(v), "max": max(v), "mean": mean, "avg": mean, "timings": v[-10:]}

    def log_summary(self) -> None:
        logger.info(f"[TIMER] {self.name} Summary:")
        for k, s in sorted(self.get_stats().items(), key=lambda kv: -kv[1].get("total", 0)):
            logger.info(f"  {k}: n={s['count']} errors={s['errors']} total={s['total']:.3f}s mean={s['mean'] * 1e3:.2f}ms "
                        f"min={s['min'] * 1e3:.2f}ms max={s['max'] * 1e3:.2f}ms")

    def reset(self, func_name: str | None = None) -> None:
        if func_name is None:
            self.timings.clear()
            self.counts.clear()
            self.active_timers.clear()
        else:
            self.timings.pop(func_name, None)
            self.counts.pop(func_name, None)
            self.counts.pop(f"{func_name}_errors", None)


class DummyTimerProfiler:
    """No-op with the same surface."""

    def __init__(self, name: str = "DummyTimerProfiler", *a, **k):
        self.name, self.timings, self.counts, self.active_timers = name, {}, {}, {}

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
