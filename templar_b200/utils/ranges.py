"""Named phases for traces: ``with phase("Optimizer Step"): ...``.

Every phase is a ``torch.profiler.record_function`` scope (it shows up in the traces that
``--profile-iters`` writes; a few microseconds when no profiler is active) and, when ``TPLR_NVTX=1``, an
NVTX range as well, so that an external timeline tool groups the kernels of a phase.  The reference labels
the same phases in its training loop (neurons/trainer.py:811-922: "Data Loading", "Prepare Inputs",
"Forward Pass", "Backward Pass", "Optimizer Step").
"""

from __future__ import annotations

import os
from contextlib import contextmanager

import torch

_NVTX = os.environ.get("TPLR_NVTX", "0") == "1"


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


@contextmanager
def phase(name: str):
    nv = nvtx_enabled()
    if nv:
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if nv:
            torch.cuda.nvtx.range_pop()


def labelled(iterable, name: str = "Data Loading"):
    """Iterate ``iterable`` with every ``next()`` inside a phase called ``name``."""
    it = iter(iterable)
    while True:
        with phase(name):
            try:
                item = next(it)
            except StopIteration:
                return
        yield item
