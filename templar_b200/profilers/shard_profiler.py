"""Dataset shard read profiler: per-shard read timings, slow-read warnings, JSON export
(reference: src/tplr/profilers/shard_profiler.py:12-331)."""

from __future__ import annotations

import json
import time
from collections import defaultdict

from ..logging import logger


class ShardProfiler:
    def __init__(self, name: str = "ShardProfiler", slow_read_s: float = 1.0):
        self.name, self.slow_read_s = name, slow_read_s
        self.reads: dict[str, list[dict]] = defaultdict(list)
        self.metadata: dict[str, dict] = {}
        self._active: dict[int, tuple[str, float, dict]] = {}
        self._next = 0

    def start_read(self, shard_path: str, chosen_shard: dict | None = None) -> int:
        self._next += 1
        self._active[self._next] = (shard_path, time.perf_counter(), dict(chosen_shard or {}))
        return self._next

    def end_read(self, timer_id: int, shard_path: str | None = None) -> float:
        item = self._active.pop(timer_id, None)
        if item is None:
            return 0.0
        path, t0, meta = item
        dt = time.perf_counter() - t0
        self.reads[path].append({"seconds": dt, **meta})
        if dt > self.slow_read_s:
            logger.warning(f"[{self.name}] slow shard read: {path} took {dt:.2f}s")
        return dt

    def log_read_details(self, shard_path: str, group_index: int, num_groups: int, offset: int, rows_per_group: int) -> None:
        """One line per partial read of a shard (a row group of a columnar file, a slice of a token file)."""
        logger.info(f"[{self.name}] reading part {group_index}/{num_groups} of {shard_path}: offset {offset}, "
                    f"{rows_per_group} rows")

    def log_shard_metadata(self, shard_path: str, file_size, num_groups: int, total_rows: int) -> None:
        """Remember size and layout of a shard; they travel with its timings into the analysis and the export."""
        logger.debug(f"[{self.name}] opening {shard_path}: size {file_size}, {num_groups} parts, {total_rows} rows")
        m = self.metadata.setdefault(shard_path, {})
        if file_size != "unknown":
            m["file_size"] = file_size
        m.setdefault("row_groups", num_groups)
        m["total_rows"] = total_rows

    log_parquet_metadata = log_shard_metadata            # the name this hook has in src/tplr/profilers/shard_profiler.py:120

    def log_read_complete(self, shard_path: str, elapsed: float) -> None:
        s = self.get_stats(shard_path)
        if s:
            logger.info(f"[{self.name}] read of {shard_path} done in {elapsed:.4f}s (mean {s['mean']:.4f}s, min {s['min']:.4f}s, "
                        f"max {s['max']:.4f}s over {s['reads']} reads)")

    def get_stats(self, shard_path: str | None = None) -> dict:
        def one(v):
            ts = [r["seconds"] for r in v]
            return {"reads": len(ts), "total": sum(ts), "min": min(ts), "max": max(ts), "mean": sum(ts) / len(ts)} if ts else {}
        if shard_path is not None:
            return one(self.reads.get(shard_path, []))
        return {k: one(v) for k, v in self.reads.items()}

    def log_analysis(self) -> None:
        for k, s in sorted(self.get_stats().items(), key=lambda kv: -kv[1].get("mean", 0)):
            logger.info(f"[{self.name}] {k}: reads={s['reads']} mean={s['mean']:.3f}s max={s['max']:.3f}s")

    def export_data(self, output_file: str = "shard_performance_report.json") -> None:
        with open(output_file, "w") as f:
            json.dump({"stats": self.get_stats(), "reads": self.reads, "metadata": self.metadata}, f, indent=2)

    def reset(self, shard_path: str | None = None) -> None:
        """Forget one shard's records, or everything (reads in flight included)."""
        if shard_path is not None:
            self.reads.pop(shard_path, None)
            self.metadata.pop(shard_path, None)
            return
        self.reads.clear()
        self.metadata.clear()
        self._active.clear()


class DummyShardProfiler:
    def __init__(self, *a, **k): pass
    def start_read(self, shard_path, chosen_shard=None): return 0
    def end_read(self, timer_id, shard_path=None): return 0.0
    def get_stats(self, shard_path=None): return {}
    def log_analysis(self): return None
    def export_data(self, output_file="shard_performance_report.json"): return None
    def reset(self, shard_path=None): return None
    def log_read_details(self, *a, **k): return None
    def log_shard_metadata(self, *a, **k): return None
    log_parquet_metadata = log_shard_metadata
    def log_read_complete(self, *a, **k): return None
