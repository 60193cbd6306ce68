"""Exception handlers used by the retry / catcher decorators.

Parity: src/tplr/exceptions.py:8-100 (log-and-swallow handlers for object-store, generic and
evaluator failures).  The object-store handler recognises botocore's error classes by name so
that botocore stays optional.
"""

from __future__ import annotations

import asyncio

from .logging import logger

_S3_NAMES = {"ClientError", "ConnectionClosedError", "EndpointConnectionError", "NoCredentialsError",
             "ParamValidationError", "ReadTimeoutError", "ConnectTimeoutError"}


def is_s3_error(e: BaseException) -> bool:
    return any(c.__name__ in _S3_NAMES for c in type(e).__mro__)


def handle_s3_exceptions(e: Exception, func_name: str) -> None:
    if is_s3_error(e):
        code = getattr(e, "response", {}).get("Error", {}).get("Code", type(e).__name__) if hasattr(e, "response") else type(e).__name__
        logger.error(f"[{func_name}] object-store error {code}: {e}")
    elif isinstance(e, (asyncio.TimeoutError, TimeoutError)):
        logger.error(f"[{func_name}] object-store timeout: {e}")
    else:
        logger.error(f"[{func_name}] unexpected storage failure: {e}")


def handle_general_exceptions(e: Exception, func_name: str) -> None:
    if isinstance(e, (asyncio.TimeoutError, TimeoutError)):
        logger.error(f"[{func_name}] timed out: {e}")
    elif isinstance(e, (ValueError, KeyError, TypeError)):
        logger.error(f"[{func_name}] bad value: {type(e).__name__}: {e}")
    elif isinstance(e, (OSError, IOError)):
        logger.error(f"[{func_name}] I/O error: {e}")
    else:
        logger.error(f"[{func_name}] {type(e).__name__}: {e}")


def handle_evaluator_exceptions(e: Exception, func_name: str) -> None:
    logger.error(f"[evaluator:{func_name}] {type(e).__name__}: {e}")
