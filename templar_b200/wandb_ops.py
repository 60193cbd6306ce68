"""Weights & Biases helper: resumable run ids and versioned metric names.

Parity: src/tplr/wandb_ops.py:22-127 — the run id is kept in ``wandb/wandb_run_id_<prefix><uid>.txt`` so a
restart resumes the same run, and every logged metric is duplicated under ``v<version>/…`` and
``latest/…``.  When ``wandb`` is unusable (offline, no API key) a :class:`NullRun` with the same
``log`` / ``finish`` surface is returned.
"""

from __future__ import annotations

import os

from . import __version__
from .logging import logger


class NullRun:
    """Run stand-in that remembers the last logged payload (useful for tests and offline runs)."""

    def __init__(self):
        self.history: list[tuple[dict, int | None]] = []
        self.id = "offline"

    def log(self, metrics: dict, step: int | None = None, **_):
        self.history.append((metrics, step))

    def finish(self):
        return None


def versioned(metrics: dict, version: str = __version__) -> dict:
    out = {}
    for k, v in metrics.items():
        out[f"v{version}/{k}"] = v
        out[f"latest/{k}"] = v
    return out


def initialize_wandb(run_prefix: str, uid, config, group: str, job_type: str):
    enabled = getattr(config, "use_wandb", None)
    if enabled is False or os.environ.get("WANDB_MODE", "").lower() == "disabled" or not os.environ.get("WANDB_API_KEY"):
        return NullRun()
    try:
        import wandb

        wandb_dir = os.path.join(os.getcwd(), "wandb")
        os.makedirs(wandb_dir, exist_ok=True)
        id_file = os.path.join(wandb_dir, f"wandb_run_id_{run_prefix}{uid}.txt")
        run_id = open(id_file).read().strip() if os.path.exists(id_file) else None
        run = wandb.init(project=getattr(config, "project", "templar"), entity=getattr(config, "wandb_entity", None),
                         id=run_id, resume="allow" if run_id else None, name=f"{run_prefix}{uid}", config=vars(config)
                         if hasattr(config, "__dict__") else None, group=group, job_type=job_type, dir=wandb_dir,
                         tags=[f"v{__version__}"], settings=wandb.Settings(init_timeout=300))
        with open(id_file, "w") as f:
            f.write(run.id)
        raw_log = run.log

        def log(metrics, **kw):
            raw_log(versioned(metrics), **kw)

        run.log = log
        return run
    except Exception as e:  # noqa: BLE001
        logger.warning(f"wandb unavailable ({e}); metrics will not be mirrored there")
        return NullRun()
