"""Small control-flow decorators.

Parity: src/tplr/decos.py:36-208 — ``retry_on_failure`` (async, fixed delay, optional total
timeout, returns None when exhausted), ``async_exception_catcher`` / ``sync_exception_catcher``
(log through a handler and return ``on_error_return(e)``), the S3 / general / evaluator partials
and ``master_only`` (run only where ``self.is_master``).
"""

from __future__ import annotations

import asyncio
import functools
import time
from typing import Any, Callable

from . import exceptions as _ex


def retry_on_failure(retries: int = 3, delay: float = 1.0, timeout: float | None = None):
    def deco(fn):
        @functools.wraps(fn)
        async def wrapper(*a, **kw):
            start = time.monotonic()
            for attempt in range(retries):
                if timeout is not None and time.monotonic() - start > timeout:
                    return None
                result = await fn(*a, **kw)
                if result is not None:
                    return result
                if attempt < retries - 1:
                    await asyncio.sleep(delay)
            return None
        return wrapper
    return deco


def async_exception_catcher(on_error_return: Callable[[Exception], Any] = lambda e: None,
                            handler: Callable[[Exception, str], None] = _ex.handle_general_exceptions):
    def deco(fn):
        @functools.wraps(fn)
        async def wrapper(*a, **kw):
            try:
                return await fn(*a, **kw)
            except Exception as e:  # noqa: BLE001
                handler(e, fn.__name__)
                return on_error_return(e)
        return wrapper
    return deco


def sync_exception_catcher(on_error_return: Callable[[Exception], Any] = lambda e: None,
                           handler: Callable[[Exception, str], None] = _ex.handle_general_exceptions):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            try:
                return fn(*a, **kw)
            except Exception as e:  # noqa: BLE001
                handler(e, fn.__name__)
                return on_error_return(e)
        return wrapper
    return deco


async_s3_exception_catcher = functools.partial(async_exception_catcher, handler=_ex.handle_s3_exceptions)
s3_exception_catcher = functools.partial(sync_exception_catcher, handler=_ex.handle_s3_exceptions)
general_exception_catcher = functools.partial(sync_exception_catcher, handler=_ex.handle_general_exceptions)
async_general_exception_catcher = functools.partial(async_exception_catcher, handler=_ex.handle_general_exceptions)
evaluator_exception_catcher = functools.partial(sync_exception_catcher, handler=_ex.handle_evaluator_exceptions)
async_evaluator_exception_catcher = functools.partial(async_exception_catcher, handler=_ex.handle_evaluator_exceptions)


def master_only(fn):
    """Run the method only on the master rank (``self.is_master``); others get None."""
    if asyncio.iscoroutinefunction(fn):
        @functools.wraps(fn)
        async def awrapper(self, *a, **kw):
            if not getattr(self, "is_master", True):
                return None
            return await fn(self, *a, **kw)
        return awrapper

    @functools.wraps(fn)
    def wrapper(self, *a, **kw):
        if not getattr(self, "is_master", True):
            return None
        return fn(self, *a, **kw)
    return wrapper
