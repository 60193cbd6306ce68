"""Environment-driven storage configuration.

``BUCKET_SECRETS`` has the reference's shape (src/tplr/config.py:32-60):
``{"gradients"|"aggregator"|"dataset": {"account_id", "name", "credentials": {"read": {...}, "write": {...}}}}``
read from ``R2_<ROLE>_*`` variables, with ``R2_DATASET_BUCKET_LIST`` (JSON list) selecting several
dataset endpoints.  Unlike the reference, a missing variable does not make the package
un-importable: offline runs use the local-filesystem store.  Set ``TPLR_STRICT_ENV=1`` to get the
reference's ``ImportError`` (src/tplr/config.py:107-112).
"""

from __future__ import annotations

import json
import os
import sys
from pathlib import Path

REQUIRED_VARS = [
    "R2_GRADIENTS_ACCOUNT_ID", "R2_GRADIENTS_BUCKET_NAME", "R2_GRADIENTS_READ_ACCESS_KEY_ID",
    "R2_GRADIENTS_READ_SECRET_ACCESS_KEY", "R2_GRADIENTS_WRITE_ACCESS_KEY_ID",
    "R2_GRADIENTS_WRITE_SECRET_ACCESS_KEY", "R2_AGGREGATOR_ACCOUNT_ID", "R2_AGGREGATOR_BUCKET_NAME",
    "R2_AGGREGATOR_READ_ACCESS_KEY_ID", "R2_AGGREGATOR_READ_SECRET_ACCESS_KEY", "DATASET_BINS_PATH",
]


def load_dotenv(path: str | os.PathLike = ".env") -> int:
    """Minimal ``KEY=VALUE`` loader (existing variables win). Returns the number of keys set."""
    p = Path(path)
    if not p.is_file():
        return 0
    n = 0
    for line in p.read_text().splitlines():
        line = line.strip()
        if not line or line.startswith("#") or "=" not in line:
            continue
        k, v = line.split("=", 1)
        k, v = k.replace("export ", "").strip(), v.strip().strip("'\"")
        if k and k not in os.environ:
            os.environ[k] = v
            n += 1
    return n


def format_bucket_secrets(base: str) -> dict:
    g = os.getenv
    return {
        "account_id": g(f"{base}_ACCOUNT_ID"),
        "name": g(f"{base}_BUCKET_NAME"),
        "credentials": {
            "read": {"access_key_id": g(f"{base}_READ_ACCESS_KEY_ID"),
                     "secret_access_key": g(f"{base}_READ_SECRET_ACCESS_KEY")},
            "write": {"access_key_id": g(f"{base}_WRITE_ACCESS_KEY_ID"),
                      "secret_access_key": g(f"{base}_WRITE_SECRET_ACCESS_KEY")},
        },
    }


def missing_env() -> list[str]:
    return [v for v in REQUIRED_VARS if not os.environ.get(v)]


def load_bucket_secrets(strict: bool | None = None) -> dict:
    secrets = {role: format_bucket_secrets(f"R2_{role.upper()}") for role in ("gradients", "aggregator", "dataset")}
    raw = os.environ.get("R2_DATASET_BUCKET_LIST")
    if raw:
        try:
            cfgs = json.loads(raw.strip())
            if isinstance(cfgs, list) and cfgs:
                secrets["dataset"] = {"multiple": cfgs}
        except Exception as e:  # noqa: BLE001
            print(f"R2_DATASET_BUCKET_LIST is not valid JSON ({e}); using the single dataset bucket", file=sys.stderr)
    if strict is None:
        strict = os.environ.get("TPLR_STRICT_ENV", "0") == "1"
    miss = missing_env()
    if miss and strict:
        raise ImportError(f"Required environment variables missing: {miss}")
    secrets["_missing"] = miss
    return secrets


class ClientConfig(dict):
    """Connection settings handed to the S3 client (pool 256, adaptive retries x10, keep-alive)."""

    def __init__(self):
        super().__init__(max_pool_connections=256, tcp_keepalive=True, retries={"max_attempts": 10, "mode": "adaptive"})

    def to_botocore(self):
        import botocore.config  # optional dependency

        return botocore.config.Config(**self)


load_dotenv()
client_config = ClientConfig()
BUCKET_SECRETS = load_bucket_secrets()
