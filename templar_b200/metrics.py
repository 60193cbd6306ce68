"""Metrics logger: batched, non-blocking time-series writes with standard tags.

Interface parity with the reference's ``MetricsLogger`` (src/tplr/metrics.py:63-368): ``log(measurement,
tags, fields, timestamp=None, with_system_metrics=False, with_gpu_metrics=False, sample_rate=1.0)``
queues a point (queue bound 600 000) that a private writer thread flushes in batches; list-valued
fields are expanded to mean/min/max/median statistics; system (psutil) and GPU memory fields are
added on request; tags carry role / uid / version / host config.

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


def get_system_metrics() -> dict[str, float]:
    try:
        import psutil

        vm = psutil.virtual_memory()
        return {"sys_cpu_usage": psutil.cpu_percent(interval=None), "sys_mem_used": vm.used / 1024 ** 2,
                "sys_mem_total": vm.total / 1024 ** 2}
    except Exception:  # noqa: BLE001
        return {}


def get_gpu_metrics() -> dict[str, float]:
    if not torch.cuda.is_available():
        return {}
    try:
        return {"gpu_mem_segments": float(torch.cuda.memory_stats().get("segment.all.current", 0)),
                "gpu_mem_allocated_mb": torch.cuda.memory_allocated() / 1024 ** 2,
                "gpu_mem_cached_mb": torch.cuda.memory_reserved() / 1024 ** 2,
                "gpu_mem_total_mb": torch.cuda.max_memory_allocated() / 1024 ** 2}
    except Exception:  # noqa: BLE001
        return {}


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
                 batch_size: int = 500, flush_interval: float = 5.0, jsonl_path: str | None = None):
        self.prefix, self.uid, self.role, self.config = prefix, uid, role, config
        self.group, self.job_type = group, job_type
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
            if with_system_metrics:
                f.update(get_system_metrics())
            if with_gpu_metrics:
                f.update(get_gpu_metrics())
            point = {"measurement": f"{self.prefix}{measurement}", "tags": self._tags(tags), "fields": f,
                     "time": timestamp if timestamp is not None else time.time()}
            self._q.put_nowait(point)
        except queue.Full:
            logger.warning("metrics queue full – dropping point")
        except Exception as e:  # noqa: BLE001
            logger.debug(f"metrics log failed: {e}")

    def process_fields(self, fields: dict) -> dict:
        out = {}
        for k, v in fields.items():
            if v is None:
                continue
            if isinstance(v, torch.Tensor):
                v = v.detach().float().cpu().tolist() if v.numel() > 1 else float(v)
            if isinstance(v, (list, tuple)):
                nums = [float(x) for x in v if isinstance(x, (int, float))]
                if nums:
                    out[f"{k}_mean"], out[f"{k}_min"], out[f"{k}_max"] = statistics.fmean(nums), min(nums), max(nums)
                    out[f"{k}_median"] = statistics.median(nums)
                    out[f"{k}_count"] = len(nums)
                else:
                    out[k] = str(list(v))
            elif isinstance(v, bool):
                out[k] = int(v)
            elif isinstance(v, (int, float)):
                out[k] = v
            else:
                out[k] = str(v)
        return out

    def _tags(self, tags: dict) -> dict:
        base = {"version": __version__, "role": self.role or "unknown", "uid": str(self.uid)}
        if self.group:
            base["group"] = self.group
        if self.job_type:
            base["job_type"] = self.job_type
        cfg = self.config
        for attr in ("netuid", "device"):
            if cfg is not None and getattr(cfg, attr, None) is not None:
                base[f"config_{attr}"] = str(getattr(cfg, attr))
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
