"""Dataset shard read profiler: per-shard read timings, slow-read warnings, analysis and JSON export.

One record per shard path in ``shard_performance``: the shard's own facts (``num_rows``, ``file_size``,
``row_groups``, ``rows_per_group``) and its reads (``reads``, ``total_time``, ``min_time``, ``max_time``, the
individual ``timings`` with whatever the caller attached to each).  ``start_read`` / ``end_read`` bracket a read and
are matched by a timer id, so reads of one shard may overlap (reference: src/tplr/profilers/shard_profiler.py:12-331).
"""

from __future__ import annotations

import json
import time

from ..logging import logger


class ShardProfiler:
    def __init__(self, name: str = "ShardProfiler", slow_read_s: float = 1.0):
        self.name, self.slow_read_s = name, slow_read_s
        self.shard_performance: dict[str, dict] = {}
        self._active_timers: dict[str, tuple[str, float, dict]] = {}
        self._next = 0

    def _record(self, shard_path: str) -> dict:
        rec = self.shard_performance.get(shard_path)
        if rec is None:
            rec = self.shard_performance[shard_path] = {
                "reads": 0, "total_time": 0.0, "min_time": float("inf"), "max_time": 0.0, "timings": [],
                "num_rows": None, "file_size": None, "row_groups": None, "rows_per_group": None}
        return rec

    def start_read(self, shard_path: str, chosen_shard: dict | None = None) -> str:
        """Open a timer for a read of ``shard_path``; ``chosen_shard`` may carry ``num_rows`` / ``file_size`` (kept as
        the shard's facts) and anything else the caller wants noted with this read."""
        info = dict(chosen_shard or {})
        rec = self._record(shard_path)
        for k in ("num_rows", "file_size"):
            if info.get(k) is not None:
                rec[k] = info[k]
        self._next += 1
        timer_id = f"{shard_path}#{self._next}"
        self._active_timers[timer_id] = (shard_path, time.perf_counter(), info)
        return timer_id

    def end_read(self, timer_id: str, shard_path: str | None = None, num_row_groups: int | None = None,
                 rows_per_group: int | None = None) -> float:
        item = self._active_timers.pop(timer_id, None)
        if item is None:
            return 0.0
        path, t0, info = item
        dt = time.perf_counter() - t0
        rec = self._record(path)
        rec["reads"] += 1
        rec["total_time"] += dt
        rec["min_time"], rec["max_time"] = min(rec["min_time"], dt), max(rec["max_time"], dt)
        rec["timings"].append({"seconds": dt, **{k: v for k, v in info.items() if k not in ("num_rows", "file_size")}})
        if num_row_groups is not None:
            rec["row_groups"] = num_row_groups
        if rows_per_group is not None:
            rec["rows_per_group"] = rows_per_group
        if dt > self.slow_read_s:
            logger.warning(f"[{self.name}] slow shard read: {path} took {dt:.2f}s")
        return dt

    def log_read_details(self, shard_path: str, group_index: int, num_row_groups: int, offset: int, rows_per_group: int) -> None:
        """One line per partial read of a shard (a row group of a columnar file, a slice of a token file)."""
        logger.info(f"Reading row group {group_index}/{num_row_groups} from shard: {shard_path}, offset: {offset}, "
                    f"rows_per_group: {rows_per_group}")

    def log_shard_metadata(self, shard_path: str, file_size, num_row_groups: int, total_rows: int) -> None:
        """Size and layout of a shard as its file says; stored with the shard's record when it has one."""
        logger.debug(f"Opening shard file: {shard_path} - size: {file_size}, row groups: {num_row_groups}, "
                     f"total rows: {total_rows}")
        rec = self.shard_performance.get(shard_path)
        if rec is not None:
            if file_size != "unknown":
                rec["file_size"] = file_size
            if rec["row_groups"] is None:
                rec["row_groups"] = num_row_groups
            if rec["num_rows"] is None:
                rec["num_rows"] = total_rows

    log_parquet_metadata = log_shard_metadata            # the name this hook has in src/tplr/profilers/shard_profiler.py:120

    def log_read_complete(self, shard_path: str, elapsed: float) -> None:
        rec = self.shard_performance.get(shard_path)
        if rec and rec["reads"]:
            logger.info(f"Read of {shard_path} done in {elapsed:.4f}s (avg: {rec['total_time'] / rec['reads']:.4f}s, "
                        f"min: {rec['min_time']:.4f}s, max: {rec['max_time']:.4f}s, reads: {rec['reads']})")

    def get_stats(self, shard_path: str | None = None) -> dict:
        """All records (path -> record), or one shard's record ({} when it was never read)."""
        if shard_path is not None:
            return self.shard_performance.get(shard_path, {})
        return self.shard_performance

    def _summary(self) -> dict:
        read = {p: r for p, r in self.shard_performance.items() if r["reads"]}
        n = sum(r["reads"] for r in read.values())
        total = sum(r["total_time"] for r in read.values())
        slowest = max(read.items(), key=lambda kv: kv[1]["total_time"] / kv[1]["reads"], default=(None, None))[0]
        return {"shards": len(read), "reads": n, "total_time": total, "avg_read_time": total / n if n else 0.0,
                "slowest_shard": slowest}

    def log_analysis(self) -> None:
        if not any(r["reads"] for r in self.shard_performance.values()):
            logger.info("No shard performance data collected yet")
            return
        s = self._summary()
        logger.info(f"=== SHARD PERFORMANCE ANALYSIS ({self.name}) ===")
        logger.info(f"{s['shards']} shards, {s['reads']} reads, {s['total_time']:.3f}s in total, "
                    f"{s['avg_read_time']:.4f}s per read; slowest on average: {s['slowest_shard']}")
        ranked = sorted(((p, r) for p, r in self.shard_performance.items() if r["reads"]),
                        key=lambda kv: -kv[1]["total_time"] / kv[1]["reads"])
        for path, r in ranked:
            logger.info(f"  {path}: reads={r['reads']} avg={r['total_time'] / r['reads']:.4f}s min={r['min_time']:.4f}s "
                        f"max={r['max_time']:.4f}s rows={r['num_rows']} size={r['file_size']} row_groups={r['row_groups']}")

    def export_data(self, output_file: str = "shard_performance_report.json") -> None:
        stats = {p: {**r, "min_time": r["min_time"] if r["reads"] else None} for p, r in self.shard_performance.items()}
        with open(output_file, "w") as f:
            json.dump({"shard_statistics": stats, "summary": self._summary()}, f, indent=2, default=str)

    def reset(self, shard_path: str | None = None) -> None:
        """Forget one shard's record, or everything (reads in flight included)."""
        if shard_path is not None:
            self.shard_performance.pop(shard_path, None)
            return
        self.shard_performance.clear()
        self._active_timers.clear()


class DummyShardProfiler:
    """No-op with the same surface: what ``get_shard_profiler`` hands out while the profiler is switched off."""

    def __init__(self, name: str = "DummyShardProfiler", *a, **k): self.name = name
    def start_read(self, *a, **k) -> str: return "dummy_timer"
    def end_read(self, *a, **k) -> float: return 0.0
    def get_stats(self, *a, **k) -> dict: return {}
    def log_analysis(self) -> None: return None
    def export_data(self, *a, **k) -> None: return None
    def reset(self, *a, **k) -> None: return None
    def log_read_details(self, *a, **k) -> None: return None
    def log_shard_metadata(self, *a, **k) -> None: return None
    log_parquet_metadata = log_shard_metadata
    def log_read_complete(self, *a, **k) -> None: return None
