"""Env-gated profilers: ``TPLR_ENABLE_PROFILERS`` switches both on, ``TPLR_ENABLE_TIMER_PROFILER`` /
``TPLR_ENABLE_SHARD_PROFILER`` one of them; while a profiler is off its accessor hands out a no-op stand-in with the
same surface (reference: src/tplr/profilers/__init__.py:13-20).  The switches are module attributes read at every
call of an accessor, so a test or a long-running node can flip them."""

import os

from .shard_profiler import DummyShardProfiler, ShardProfiler
from .timer_profiler import CudaEventTimer, DummyTimerProfiler, TimerProfiler

_TRUTHY = ("1", "true", "yes", "on")
ENABLE_PROFILERS = os.environ.get("TPLR_ENABLE_PROFILERS", "0").lower() in _TRUTHY
ENABLE_TIMER_PROFILER = ENABLE_PROFILERS or os.environ.get("TPLR_ENABLE_TIMER_PROFILER", "0").lower() in _TRUTHY
ENABLE_SHARD_PROFILER = ENABLE_PROFILERS or os.environ.get("TPLR_ENABLE_SHARD_PROFILER", "0").lower() in _TRUTHY

_timer: TimerProfiler | None = None
_shard: ShardProfiler | None = None
_dummy_timer, _dummy_shard = DummyTimerProfiler(), DummyShardProfiler()


def get_timer_profiler(name: str | None = None):
    """The process-wide timer profiler, or the no-op stand-in while timing is switched off."""
    global _timer
    if not ENABLE_TIMER_PROFILER:
        return _dummy_timer
    if _timer is None:
        _timer = TimerProfiler(name or "global")
    return _timer


def get_shard_profiler(name: str | None = None):
    """The process-wide shard profiler, or the no-op stand-in while it is switched off."""
    global _shard
    if not ENABLE_SHARD_PROFILER:
        return _dummy_shard
    if _shard is None:
        _shard = ShardProfiler(name or "global")
    return _shard


get_profiler = get_shard_profiler          # the reference's name for the shard profiler's accessor


__all__ = ["ENABLE_PROFILERS", "ENABLE_TIMER_PROFILER", "ENABLE_SHARD_PROFILER", "get_profiler", "TimerProfiler",
           "ShardProfiler", "DummyTimerProfiler", "DummyShardProfiler", "CudaEventTimer", "get_timer_profiler",
           "get_shard_profiler"]
