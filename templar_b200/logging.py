"""Logging: the ``"templar"`` logger, phase timers ``T()`` / ``P()``, contextual and JSON logs.

Parity: src/tplr/logging.py:41-320 — Rich console handler when ``rich`` is importable, a TRACE
level, ``log_with_context`` (extra fields carried on the record), a JSON formatter and an
optional Loki push handler behind a ``QueueHandler`` so that logging never blocks the loop.
The Loki transport is optional (``logging_loki`` may be absent); without it
``setup_loki_logger`` attaches a JSON-lines file handler instead when ``TPLR_LOG_JSONL`` is set.
"""

from __future__ import annotations

import json
import logging as _logging
import os
import queue
import time
from logging.handlers import QueueHandler, QueueListener

TRACE = 5
_logging.addLevelName(TRACE, "TRACE")


def T() -> float:
    """Monotonic timestamp for phase timing."""
    return time.perf_counter()


def P(window: int, duration: float) -> str:
    """Prefix ``[window] (duration)`` used in phase log lines."""
    return f"[{window}] ({duration:.2f}s)"


class JsonFormatter(_logging.Formatter):
    STANDARD = set(vars(_logging.LogRecord("", 0, "", 0, "", (), None))) | {"message", "asctime"}

    def format(self, record: _logging.LogRecord) -> str:
        out = {"ts": round(record.created, 3), "level": record.levelname, "logger": record.name,
               "message": record.getMessage()}
        for k, v in vars(record).items():
            if k not in self.STANDARD and not k.startswith("_"):
                try:
                    json.dumps(v)
                    out[k] = v
                except TypeError:
                    out[k] = repr(v)
        if record.exc_info:
            out["exc"] = self.formatException(record.exc_info)
        return json.dumps(out)


def _console_handler() -> _logging.Handler:
    try:
        from rich.logging import RichHandler

        return RichHandler(markup=False, rich_tracebacks=True, show_path=False, show_time=True)
    except Exception:  # pragma: no cover
        h = _logging.StreamHandler()
        h.setFormatter(_logging.Formatter("%(asctime)s %(levelname)s %(message)s"))
        return h


logger = _logging.getLogger("templar")
if not logger.handlers:
    logger.addHandler(_console_handler())
    logger.setLevel(os.environ.get("TPLR_LOG_LEVEL", "INFO").upper())
    logger.propagate = False


def _trace_message(msg, *a, **kw):
    if logger.isEnabledFor(TRACE):
        logger._log(TRACE, msg, a, **kw)


logger.trace = _trace_message  # type: ignore[attr-defined]


def trace(msg=None, *a, **kw) -> None:
    """``trace()`` switches the logger to the TRACE level, as ``debug()`` switches it to DEBUG (the call the
    reference's neurons make for ``--trace``, src/tplr/logging.py:113-146); ``trace("text")`` logs at that level."""
    if msg is None:
        logger.setLevel(TRACE)
    else:
        _trace_message(msg, *a, **kw)


class NoSubtensorWarning(_logging.Filter):
    """Drops the chain client's repeated "not connected / reconnecting" warnings from a handler."""

    NEEDLES = ("Verify your local subtensor", "subtensor is running", "reconnecting to subtensor")

    def filter(self, record: _logging.LogRecord) -> bool:
        text = record.getMessage()
        return not any(n in text for n in self.NEEDLES)


def debug() -> None:
    logger.setLevel(_logging.DEBUG)


def trace_on() -> None:
    logger.setLevel(TRACE)


def log_with_context(level: str, message: str, **context) -> None:
    """Log ``message`` with structured fields (window, uid, step, ...) attached to the record."""
    lvl = TRACE if level.lower() == "trace" else getattr(_logging, level.upper(), _logging.INFO)
    logger.log(lvl, message, extra={k: v for k, v in context.items() if k not in JsonFormatter.STANDARD})


_listener: QueueListener | None = None


def setup_loki_logger(service: str, uid: str, version: str, environment: str = "finney",
                      url: str | None = None) -> bool:
    """Attach a non-blocking structured sink. Returns True when a sink was attached."""
    global _listener
    url = url or os.environ.get("LOKI_URL")
    tags = {"service": service, "uid": str(uid), "version": version, "environment": environment,
            "host": os.uname().nodename, "pid": str(os.getpid())}
    target: _logging.Handler | None = None
    if url:
        try:
            import logging_loki  # optional

            target = logging_loki.LokiHandler(url=url, tags=tags, version="1")
        except Exception:
            target = None
    if target is None and os.environ.get("TPLR_LOG_JSONL"):
        target = _logging.FileHandler(os.environ["TPLR_LOG_JSONL"])
    if target is None:
        return False
    target.setFormatter(JsonFormatter())
    q: queue.Queue = queue.Queue(-1)
    logger.addHandler(QueueHandler(q))
    _listener = QueueListener(q, target, respect_handler_level=True)
    _listener.start()
    return True


def shutdown_logging() -> None:
    global _listener
    if _listener is not None:
        _listener.stop()
        _listener = None


__all__ = ["logger", "T", "P", "debug", "trace", "trace_on", "log_with_context", "setup_loki_logger", "JsonFormatter",
           "NoSubtensorWarning"]
