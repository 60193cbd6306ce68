"""Operator tools for the buckets of a node: check access, list, fetch a gradient, prune old objects and versions.

    python -m templar_b200.bucket_tools validate                       write / read / delete a probe in the node's bucket
    python -m templar_b200.bucket_tools list [--prefix gradient-]      objects with size and age
    python -m templar_b200.bucket_tools summary                        objects and bytes per kind and per version
    python -m templar_b200.bucket_tools get-gradient --uid U --window W [--out file.pt]
    python -m templar_b200.bucket_tools cleanup --keep-windows N [--dry-run]        drop all but the newest N windows
    python -m templar_b200.bucket_tools clean-versions [--keep 2.1.28] [--dry-run]  drop objects of other versions
    python -m templar_b200.bucket_tools delete-version --version 2.1.20 [--dry-run]   drop every object of one version
    python -m templar_b200.bucket_tools delete-gather --version 2.1.28 [--dry-run]    drop the stored gather results
    python -m templar_b200.bucket_tools delete [--prefix P] [--suffix S] [--older-than-hours H] [--all] [--dry-run]
                                               [--bucket gradients|aggregator|dataset]
                                               objects that match every given selector (``--all``: the whole bucket)

They work on whatever store the environment selects (a local directory offline, S3 / R2 with credentials; see
:func:`templar_b200.comms.default_store`), on the bucket that the ``R2_GRADIENTS_*`` variables name (offline: the
per-uid bucket of ``--uid``).  Counterparts in the reference: scripts/validate_r2_access.py, scripts/s3_manager.py,
scripts/cleanup_bucket.py, scripts/clean_versions.py, scripts/delete_version.py, scripts/delete_gather.py,
scripts/get_gradients.py.
"""

from __future__ import annotations

import argparse
import asyncio
import io
import re
from collections import defaultdict
from datetime import datetime, timezone

import torch

from . import __version__
from .backends.store import ObjectStore

_OBJ = re.compile(r"^(?P<kind>gradient|debug|aggregator|peers|start_window)[-_](?P<window>\d+)?.*?v(?P<version>\d+\.\d+\.\d+)")


def classify(key: str) -> tuple[str, int | None, str | None]:
    """(kind, window, version) parsed from an object name; kind "other" when the name follows no known pattern."""
    if key.startswith("checkpoints/"):
        parts = key.split("/")
        win = int(parts[2]) if len(parts) > 2 and parts[2].isdigit() else None
        return "checkpoint", win, parts[1] if len(parts) > 1 else None
    m = _OBJ.match(key)
    if not m:
        return "other", None, None
    return m.group("kind"), int(m.group("window")) if m.group("window") else None, m.group("version")


async def validate(store: ObjectStore, bucket) -> dict:
    """Round trip of a small probe object: put, head, get, delete.  Returns what worked."""
    key, body = f"access-probe-{int(datetime.now(timezone.utc).timestamp())}.bin", b"templar-b200 access probe"
    out = {"put": False, "head": False, "get": False, "delete": False}
    await store.put_bytes(bucket, key, body)
    out["put"] = True
    info = await store.head(bucket, key)
    out["head"] = info is not None and info.size == len(body)
    out["get"] = (await store.get_bytes(bucket, key)) == body
    await store.delete(bucket, [key])
    out["delete"] = (await store.head(bucket, key)) is None
    return out


async def summary(store: ObjectStore, bucket) -> dict:
    per = defaultdict(lambda: [0, 0])
    for o in await store.list(bucket, ""):
        kind, _, version = classify(o.key)
        per[(kind, version or "-")][0] += 1
        per[(kind, version or "-")][1] += o.size
    return {f"{k}@{v}": {"objects": n, "bytes": b} for (k, v), (n, b) in sorted(per.items())}


async def cleanup(store: ObjectStore, bucket, keep_windows: int, dry_run: bool = False) -> list[str]:
    """Delete gradient / debug / aggregator objects of all but the newest ``keep_windows`` windows."""
    objs = [(o.key, classify(o.key)) for o in await store.list(bucket, "")]
    windows = sorted({w for _, (k, w, _) in objs if k in ("gradient", "debug", "aggregator") and w is not None})
    keep = set(windows[-keep_windows:]) if keep_windows > 0 else set()
    doomed = [key for key, (k, w, _) in objs if k in ("gradient", "debug", "aggregator") and w is not None and w not in keep]
    if doomed and not dry_run:
        await store.delete(bucket, doomed)
    return doomed


async def clean_versions(store: ObjectStore, bucket, keep: str = __version__, dry_run: bool = False) -> list[str]:
    """Delete every versioned object whose version is not ``keep``."""
    doomed = [o.key for o in await store.list(bucket, "") if (classify(o.key)[2] or keep) != keep]
    if doomed and not dry_run:
        await store.delete(bucket, doomed)
    return doomed


async def delete_selected(store: ObjectStore, bucket, *, prefix: str = "", suffix: str = "", older_than_hours: float | None = None,
                          everything: bool = False, dry_run: bool = False, now: datetime | None = None) -> list[str]:
    """Delete the objects that match every selector given (name prefix, name suffix, age).  Without a selector
    nothing is deleted unless ``everything`` says that the whole bucket is meant."""
    if not (prefix or suffix or older_than_hours is not None or everything):
        raise ValueError("no selector given: pass a prefix, a suffix, an age, or everything=True for the whole bucket")
    now = now or datetime.now(timezone.utc)
    doomed = []
    for o in await store.list(bucket, prefix):
        if suffix and not o.key.endswith(suffix):
            continue
        if older_than_hours is not None and (now - o.last_modified).total_seconds() < older_than_hours * 3600.0:
            continue
        doomed.append(o.key)
    if doomed and not dry_run:
        await store.delete(bucket, doomed)
    return doomed


async def delete_version(store: ObjectStore, bucket, version: str, dry_run: bool = False) -> list[str]:
    """Delete every object that carries ``version`` in its name or path (gradients, debug dictionaries, peer lists,
    start window, aggregated gradients, checkpoints, gather results)."""
    doomed = [o.key for o in await store.list(bucket, "")
              if classify(o.key)[2] == version or o.key.startswith(f"gathers/{version}/")]
    if doomed and not dry_run:
        await store.delete(bucket, doomed)
    return doomed


async def delete_gather(store: ObjectStore, bucket, version: str = __version__, dry_run: bool = False) -> list[str]:
    """Delete the gather results stored under ``gathers/<version>/``."""
    return await delete_selected(store, bucket, prefix=f"gathers/{version}/", dry_run=dry_run)


async def get_gradient(store: ObjectStore, bucket, uid: int, window: int, version: str = __version__) -> dict | None:
    data = await store.get_bytes(bucket, f"gradient-{window}-{uid}-v{version}.pt")
    if data is None:
        return None
    return torch.load(io.BytesIO(data), weights_only=True, map_location="cpu")


def describe_gradient(obj: dict) -> dict:
    sd = obj.get("state_dict", obj)
    vals = [v for k, v in sd.items() if k.endswith("vals") and torch.is_tensor(v)]
    idxs = [v for k, v in sd.items() if k.endswith("idxs") and torch.is_tensor(v)]
    return {"global_step": obj.get("global_step"), "metadata": sd.get("metadata"), "tensors": len(vals),
            "value_dtype": str(vals[0].dtype) if vals else None, "values": sum(v.numel() for v in vals),
            "index_bytes": sum(i.numel() for i in idxs),
            "quantised": any(sd.get(k[:-4] + "quant_params") is not None for k in sd if k.endswith("vals"))}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("command", choices=["validate", "list", "summary", "get-gradient", "cleanup", "clean-versions",
                                        "delete-version", "delete-gather", "delete"])
    ap.add_argument("--bucket", choices=["gradients", "aggregator", "dataset"], default="gradients")
    ap.add_argument("--version", default=__version__)
    ap.add_argument("--suffix", default="")
    ap.add_argument("--older-than-hours", type=float, default=None)
    ap.add_argument("--all", action="store_true", help="delete: the whole bucket")
    ap.add_argument("--uid", type=int, default=0)
    ap.add_argument("--window", type=int, default=None)
    ap.add_argument("--prefix", default="")
    ap.add_argument("--keep-windows", type=int, default=10)
    ap.add_argument("--keep", default=__version__)
    ap.add_argument("--out", default=None)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    from .backends.chain import StaticWallet
    from .comms import Comms

    comms = Comms(wallet=StaticWallet(f"hotkey-{a.uid}"), uid=a.uid)
    store = comms.store
    bucket = comms.bucket if a.bucket == "gradients" else comms.get_own_bucket(a.bucket, "write")
    now = datetime.now(timezone.utc)

    async def run():
        if a.command == "validate":
            print(await validate(store, bucket))
        elif a.command == "list":
            for o in await store.list(bucket, a.prefix):
                print(f"{o.size:>14}  {(now - o.last_modified).total_seconds():>10.0f}s  {o.key}")
        elif a.command == "summary":
            for k, v in (await summary(store, bucket)).items():
                print(f"{k:<32} {v['objects']:>8} objects {v['bytes']:>16} bytes")
        elif a.command == "get-gradient":
            obj = await get_gradient(store, bucket, a.uid, a.window)
            if obj is None:
                raise SystemExit(f"no gradient of uid {a.uid} for window {a.window}")
            print(describe_gradient(obj))
            if a.out:
                torch.save(obj, a.out)
        elif a.command == "cleanup":
            gone = await cleanup(store, bucket, a.keep_windows, a.dry_run)
            print(f"{'would delete' if a.dry_run else 'deleted'} {len(gone)} objects")
        else:
            if a.command == "clean-versions":
                gone = await clean_versions(store, bucket, a.keep, a.dry_run)
            elif a.command == "delete-version":
                gone = await delete_version(store, bucket, a.version, a.dry_run)
            elif a.command == "delete-gather":
                gone = await delete_gather(store, bucket, a.version, a.dry_run)
            else:
                gone = await delete_selected(store, bucket, prefix=a.prefix, suffix=a.suffix, older_than_hours=a.older_than_hours,
                                             everything=a.all, dry_run=a.dry_run)
            print(f"{'would delete' if a.dry_run else 'deleted'} {len(gone)} objects")
    asyncio.run(run())


if __name__ == "__main__":
    main()
