"""Apply a function to every tensor inside nested lists / tuples / dicts / namespaces."""

from __future__ import annotations

from types import SimpleNamespace
from typing import Callable

import torch


def map_tensors(obj, fn: Callable[[torch.Tensor], torch.Tensor]):
    """A copy of ``obj`` with ``fn`` applied to its tensors; namespaces and dicts are updated in place
    (their identity is kept because callers hold references to them), other leaves pass through."""
    if torch.is_tensor(obj):
        return fn(obj)
    if isinstance(obj, list):
        return [map_tensors(x, fn) for x in obj]
    if isinstance(obj, tuple):
        return tuple(map_tensors(x, fn) for x in obj)
    if isinstance(obj, dict):
        for k in list(obj):
            obj[k] = map_tensors(obj[k], fn)
        return obj
    if isinstance(obj, SimpleNamespace):
        for k, v in list(vars(obj).items()):
            setattr(obj, k, map_tensors(v, fn))
        return obj
    return obj


def to_pinned_cpu(t: torch.Tensor) -> torch.Tensor:
    """A device tensor copied (asynchronously) into page-locked host memory, or plain host memory where there
    is no CUDA runtime; a tensor that already lives on the host is returned as it is."""
    pin = torch.cuda.is_available()
    if t.device.type == "cpu":
        return t
    dst = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
    dst.copy_(t, non_blocking=True)
    return dst


def tensor_bytes(obj) -> int:
    total = 0

    def count(t):
        nonlocal total
        total += t.element_size() * t.numel()
        return t

    map_tensors(obj, count)
    return total
