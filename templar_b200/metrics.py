"""Metrics logger: batched, non-blocking time-series writes with standard tags.

Interface parity with the reference's ``MetricsLogger`` (src/tplr/metrics.py:63-368): ``log(measurement,
tags, fields, timestamp=None, with_system_metrics=False, with_gpu_metrics=False, sample_rate=1.0)``
queues a point (queue bound 600 000) that a private writer thread flushes in batches; lists of numbers
are expanded to mean/min/max/median statistics and lists of integers (uids) are written as text; system
(psutil) and GPU memory fields are added on request; tags carry uid / prefix / version / runtime id /
role / group / job type and one ``config_<name>`` per scalar option of the node.

Sinks: InfluxDB when ``influxdb_client`` is importable and a token is configured, otherwise (and in
addition when ``TPLR_METRICS_JSONL`` is set) a JSON-lines file — the offline sink.
"""

from __future__ import annotations

import json
import os
import queue
import random
import statistics
import threading
import time
from typing import Any

import torch

from . import __version__
from .logging import logger

DEFAULT_HOST = os.environ.get("INFLUXDB_HOST", "localhost")
DEFAULT_PORT = int(os.environ.get("INFLUXDB_PORT", 8086))
DEFAULT_ORG = os.environ.get("INFLUXDB_ORG", "templar")
DEFAULT_BUCKET = os.environ.get("INFLUXDB_BUCKET", "tplr")
DEFAULT_DATABASE = DEFAULT_BUCKET          # the same setting under the name the reference gives it


def get_system_metrics() -> dict[str, float]:
    try:
        import psutil

        vm = psutil.virtual_memory()
        return {"sys_cpu_usage": psutil.cpu_percent(interval=None), "sys_mem_used": vm.used / 1024 ** 2,
                "sys_mem_total": vm.total / 1024 ** 2}
    except Exception:  # noqa: BLE001
        return {}


def get_gpu_metrics() -> dict[str, Any]:
    """Allocator figures of the current device; ``gpu_id`` / ``gpu_name`` become tags of the point."""
    if not torch.cuda.is_available():
        return {}
    try:
        dev = torch.cuda.current_device()
        return {"gpu_mem_segments": float(torch.cuda.memory_stats(dev).get("segment.all.current", 0)),
                "gpu_mem_allocated_mb": torch.cuda.memory_allocated(dev) / 1024 ** 2,
                "gpu_mem_cached_mb": torch.cuda.memory_reserved(dev) / 1024 ** 2,
                "gpu_mem_total_mb": torch.cuda.max_memory_allocated(dev) / 1024 ** 2,
                "gpu_name": f"CUDA:{dev}", "gpu_id": dev}
    except Exception:  # noqa: BLE001
        return {}


RUNTIME_ID = os.environ.get("TPLR_RUNTIME_ID") or f"{int(time.time()):x}-{os.getpid():x}"      # one per process start


class _JsonlSink:
    def __init__(self, path: str):
        self.path = path
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def write(self, points: list[dict]) -> None:
        with open(self.path, "a") as f:
            for p in points:
                f.write(json.dumps(p) + "\n")


class _InfluxSink:
    def __init__(self, host, port, token, org, bucket):
        from influxdb_client import InfluxDBClient, Point  # optional dependency
        from influxdb_client.client.write_api import SYNCHRONOUS

        scheme = "https" if int(port) == 443 else "http"
        self.client = InfluxDBClient(url=f"{scheme}://{host}:{port}", token=token, org=org)
        self.write_api = self.client.write_api(write_options=SYNCHRONOUS)
        self.bucket, self.org, self.Point = bucket, org, Point

    def write(self, points: list[dict]) -> None:
        recs = []
        for p in points:
            pt = self.Point(p["measurement"])
            for k, v in p["tags"].items():
                pt = pt.tag(k, v)
            for k, v in p["fields"].items():
                pt = pt.field(k, v)
            recs.append(pt.time(int(p["time"] * 1e9)))
        self.write_api.write(bucket=self.bucket, org=self.org, record=recs)


class MetricsLogger:
    def __init__(self, prefix: str = "", uid: str | None = None, role: str = "", config: Any = None, group: str = "",
                 job_type: str = "", host: str = DEFAULT_HOST, port: int = DEFAULT_PORT, token: str | None = None,
                 org: str = DEFAULT_ORG, database: str = DEFAULT_BUCKET, max_queue_size: int = 600_000,
                 batch_size: int = 500, flush_interval: float = 5.0, jsonl_path: str | None = None,
                 version: str = __version__, runtime_id: str = RUNTIME_ID):
        self.prefix, self.uid, self.role, self.config = prefix, uid, role, config
        self.group, self.job_type, self.version, self.runtime_id = group, job_type, version, runtime_id
        self.batch_size, self.flush_interval = batch_size, flush_interval
        self._q: queue.Queue = queue.Queue(maxsize=max_queue_size)
        self._sinks = []
        token = token or os.environ.get("INFLUXDB_TOKEN")
        if token:
            try:
                self._sinks.append(_InfluxSink(host, port, token, org, database))
            except Exception as e:  # noqa: BLE001
                logger.debug(f"InfluxDB sink unavailable: {e}")
        path = jsonl_path or os.environ.get("TPLR_METRICS_JSONL")
        if path or not self._sinks:
            self._sinks.append(_JsonlSink(path or os.path.join("/tmp", f"tplr_metrics_{role or 'node'}_{uid}.jsonl")))
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._writer, name="metrics-writer", daemon=True)
        self._thread.start()

    # -- public ----------------------------------------------------------------------------
    def log(self, measurement: str, tags: dict, fields: dict, timestamp: float | None = None,
            with_system_metrics: bool = False, with_gpu_metrics: bool = False, sample_rate: float = 1.0) -> None:
        if sample_rate < 1.0 and random.random() > sample_rate:
            return
        try:
            f = self.process_fields(fields)
            tags = dict(tags or {})
            if with_system_metrics:
                f.update(get_system_metrics())
            if with_gpu_metrics:
                for k, v in get_gpu_metrics().items():
                    (tags if k in ("gpu_id", "gpu_name") else f)[k] = v
            point = {"measurement": f"{self.prefix}{measurement}", "tags": self._tags(tags), "fields": f,
                     "time": timestamp if timestamp is not None else time.time()}
            self._q.put_nowait(point)
        except queue.Full:
            logger.warning("metrics queue full – dropping point")
        except Exception as e:  # noqa: BLE001
            logger.debug(f"metrics log failed: {e}")

    def process_value(self, v):
        """One field value in the form the time-series store takes (reference src/tplr/metrics.py:155-181): numbers
        stay numbers (booleans as 0 / 1); a non-empty list of integers is a list of uids and is written as its text; any
        other list of numbers becomes mean / min / max / median (and count); an empty list and None are 0.0; tensors
        are read back (one element: the number, more: the list); everything else is its text."""
        if isinstance(v, torch.Tensor):
            v = v.detach().float().cpu().tolist() if v.numel() > 1 else float(v)
        if isinstance(v, bool):
            return int(v)
        if isinstance(v, (int, float)):
            return v
        if isinstance(v, (list, tuple)):
            if not v:
                return 0.0
            if all(isinstance(x, int) and not isinstance(x, bool) for x in v):
                return str(list(v))
            nums = [float(x) for x in v if isinstance(x, (int, float))]
            if not nums:
                return str(list(v))
            return {"mean": statistics.fmean(nums), "min": min(nums), "max": max(nums), "median": statistics.median(nums),
                    "count": len(nums)}
        if v is None:
            return 0.0
        return str(v)

    def process_fields(self, fields: dict) -> dict:
        out = {}
        for k, v in fields.items():
            pv = self.process_value(v)
            if isinstance(pv, dict):
                out.update({f"{k}_{stat}": x for stat, x in pv.items()})
            else:
                out[k] = pv
        return out

    def _tags(self, tags: dict) -> dict:
        """Standard tags (uid, prefix, version, runtime id, role, group, job type: those that are set), one
        ``config_<name>`` tag per scalar attribute of the node's config, then the caller's tags."""
        base = {k: str(v) for k, v in (("uid", self.uid), ("prefix", self.prefix), ("version", self.version),
                                       ("runtime_id", self.runtime_id), ("role", self.role or "unknown"),
                                       ("group", self.group), ("job_type", self.job_type)) if v not in (None, "")}
        cfg = self.config
        try:
            for key, value in (vars(cfg) if cfg is not None and hasattr(cfg, "__dict__") else {}).items():
                if not key.startswith("_") and value is not None and isinstance(value, (str, int, float, bool)):
                    base[f"config_{key}"] = str(value)
        except Exception as e:  # noqa: BLE001
            logger.debug(f"config tags skipped: {e}")
        base.update({k: str(v) for k, v in (tags or {}).items()})
        return base

    # -- writer ------------------------------------------------------------------------------
    def _writer(self) -> None:
        batch, last = [], time.time()
        while not self._stop.is_set() or not self._q.empty():
            try:
                batch.append(self._q.get(timeout=0.2))
            except queue.Empty:
                pass
            if batch and (len(batch) >= self.batch_size or time.time() - last >= self.flush_interval or self._stop.is_set()):
                self._flush(batch)
                batch, last = [], time.time()
        if batch:
            self._flush(batch)

    def _flush(self, batch: list[dict]) -> None:
        for sink in self._sinks:
            try:
                sink.write(batch)
            except Exception as e:  # noqa: BLE001
                logger.debug(f"metrics sink {type(sink).__name__} failed: {e}")

    def close(self, timeout: float = 5.0) -> None:
        self._stop.set()
        self._thread.join(timeout=timeout)


class NullMetricsLogger:
    """Stand-in with the logger's surface that drops everything: what the ranks other than rank 0 hold."""

    def log(self, *_a, **_k) -> None:
        return None

    def close(self, *_a, **_k) -> None:
        return None

