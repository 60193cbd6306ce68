"""Env-gated profilers: ``TPLR_ENABLE_PROFILERS`` switches both on, ``TPLR_ENABLE_TIMER_PROFILER`` /
``TPLR_ENABLE_SHARD_PROFILER`` one of them; disabled profilers are no-op stand-ins
(reference: src/tplr/profilers/__init__.py:13-20)."""

import os

from .shard_profiler import DummyShardProfiler, ShardProfiler
from .timer_profiler import CudaEventTimer, DummyTimerProfiler, TimerProfiler


def _on(name: str) -> bool:
    truthy = ("1", "true", "yes", "on")
    return os.environ.get("TPLR_ENABLE_PROFILERS", "0").lower() in truthy or os.environ.get(name, "0").lower() in truthy


ENABLE_PROFILERS = os.environ.get("TPLR_ENABLE_PROFILERS", "0").lower() in ("1", "true", "yes", "on")
ENABLE_TIMER_PROFILER = _on("TPLR_ENABLE_TIMER_PROFILER")
ENABLE_SHARD_PROFILER = _on("TPLR_ENABLE_SHARD_PROFILER")

_timer = TimerProfiler("global") if ENABLE_TIMER_PROFILER else DummyTimerProfiler()
_shard = ShardProfiler("global") if ENABLE_SHARD_PROFILER else DummyShardProfiler()


def get_timer_profiler(name: str | None = None):
    return _timer


def get_shard_profiler(name: str | None = None):
    return _shard


get_profiler = get_shard_profiler          # the reference's name for the shard profiler's accessor


__all__ = ["ENABLE_PROFILERS", "ENABLE_TIMER_PROFILER", "ENABLE_SHARD_PROFILER", "get_profiler", "TimerProfiler", "ShardProfiler", "DummyTimerProfiler", "DummyShardProfiler", "CudaEventTimer",
           "get_timer_profiler", "get_shard_profiler"]
