"""Model checkpoints in ``torch.distributed.checkpoint`` (DCP) format, with upload/download.

On-disk and in-bucket layout is the reference's (src/tplr/dcp_checkpoint.py:56-1011), so either
framework can read the other's checkpoints:

    checkpoints/<version>/<window>/__{rank}_{i}.distcp, .metadata, extra_metadata.json
    checkpoints/<version>/_LATEST.json            {"latest_window": w}

The state is ``{"app": AppState(model)}`` — model tensors only, keyed by the torchtitan FQNs
(``app.tok_embeddings.weight`` …).  ``extra_metadata.json`` carries ``version, window, sync_window,
global_step, world_size_at_save, topology, uid``.  Each rank uploads the shard files it wrote,
rank 0 uploads the metadata, waits until every writer's shards are listed remotely (mopping up
missing ones from a shared file system), and only then publishes the ``_LATEST.json`` pointer.

Models attached to a :class:`~templar_b200.parallel.window_engine.WindowEngine` are saved from
their fp32 master weights (gathered per tensor from the shard owners), not from the bf16 compute
copy; loading scatters back into the shards and refreshes the compute copy.
"""

from __future__ import annotations

import asyncio
import hashlib
import json
import re
import shutil
import time
from concurrent.futures import Future
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.stateful import Stateful

from .logging import logger

_OWNER_RE = re.compile(r"__([0-9]+)_[0-9]+\.distcp$")


def _owner_rank_from_name(name: str) -> int | None:
    m = _OWNER_RE.search(name)
    return int(m.group(1)) if m else None


def _is_meta(p) -> bool:
    n = Path(p).name.lower()
    return n == ".metadata" or n.endswith(".metadata") or n.endswith(".json")


def _rank(group=None) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    return dist.get_rank(group) if group is not None else dist.get_rank()


def _world(group=None) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group) if group is not None else dist.get_world_size()


def _barrier(group=None) -> None:
    if dist.is_available() and dist.is_initialized():
        if torch.cuda.is_available() and group is None and dist.get_backend() == "nccl":
            dist.barrier(device_ids=[torch.cuda.current_device()])
        else:
            dist.barrier(group=group)


async def _retry_n(op, *, desc: str = "", attempts: int = 3, delay_s: float = 1.0):
    last = None
    for i in range(1, attempts + 1):
        try:
            return await op()
        except Exception as e:  # noqa: BLE001
            last = e
            logger.warning(f"[DCP][retry] {desc} failed (attempt {i}/{attempts}): {e}")
            if i < attempts:
                await asyncio.sleep(delay_s)
    raise last


def model_state_dict(model) -> dict:
    engine = getattr(model, "_window_engine", None)
    if engine is not None:
        return engine.full_state_dict()
    from torch.distributed.checkpoint.state_dict import get_model_state_dict

    return get_model_state_dict(model)


def load_model_state_dict(model, state: dict) -> None:
    engine = getattr(model, "_window_engine", None)
    if engine is not None:
        engine.load_full_state_dict(state)
        return
    from torch.distributed.checkpoint.state_dict import set_model_state_dict

    set_model_state_dict(model, state)


class AppState(Stateful):
    def __init__(self, model):
        self.model = model

    def state_dict(self):
        return model_state_dict(self.model)

    def load_state_dict(self, state) -> None:
        load_model_state_dict(self.model, state)


class SnapshotState(Stateful):
    """Host-memory copy of the model state taken at construction, so an asynchronous save is not
    affected by training steps that follow."""

    def __init__(self, model):
        engine = getattr(model, "_window_engine", None)
        if engine is not None:
            self._snap = {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v)
                          for k, v in engine.full_state_dict().items()}
        else:
            from torch.distributed.checkpoint.state_dict import StateDictOptions, get_model_state_dict

            self._snap = get_model_state_dict(model, options=StateDictOptions(full_state_dict=False, cpu_offload=True))

    def state_dict(self):
        return self._snap

    def load_state_dict(self, state) -> None:
        return


@dataclass(slots=True)
class Layout:
    version: str
    window: int | None = None

    @property
    def prefix(self) -> str:
        base = f"checkpoints/{self.version}"
        return f"{base}/{self.window}" if self.window is not None else base


class DCPCheckpointer:
    def __init__(self, comms, *, uid: int, version: str, repo_root: str | Path = "."):
        self.comms, self.uid, self.version = comms, int(uid), version
        self.repo_root = Path(repo_root).resolve()
        self._bg: set[asyncio.Task] = set()
        self._cpu_pg = None
        if dist.is_available() and dist.is_initialized() and dist.get_backend() != "gloo":
            try:
                self._cpu_pg = dist.new_group(ranks=list(range(_world())), backend=dist.Backend.GLOO)
            except Exception as e:  # noqa: BLE001
                logger.warning(f"[DCP] failed to create CPU(Gloo) PG: {e}")

    def _local_dir(self, layout: Layout) -> Path:
        d = self.repo_root / layout.prefix
        d.mkdir(parents=True, exist_ok=True)
        return d

    def _sidecar(self, window, sync_window, global_step, world, topology) -> dict:
        d = {"version": self.version, "window": int(window), "sync_window": int(sync_window),
             "world_size_at_save": int(world), "topology": topology, "uid": self.uid}
        if global_step is not None:
            d["global_step"] = int(global_step)
        return d

    # -- save -----------------------------------------------------------------------------------
    async def save_local(self, *, model, window: int, sync_window: int, topology: str = "FSDP", process_group=None,
                         global_step: int | None = None) -> Path:
        """Call on ALL ranks of the saving group."""
        out_dir = self._local_dir(Layout(self.version, window))
        t0 = time.perf_counter()
        dcp.save(state_dict={"app": AppState(model)}, checkpoint_id=str(out_dir), process_group=process_group)
        if _rank(process_group) == 0:
            (out_dir / "extra_metadata.json").write_text(json.dumps(
                self._sidecar(window, sync_window, global_step, _world(process_group), topology), indent=2))
        _barrier(process_group)
        logger.info(f"[DCP][save] rank {_rank(process_group)}/{_world(process_group)} done in {time.perf_counter() - t0:.2f}s → {out_dir}")
        return out_dir

    @dataclass(slots=True)
    class SaveHandle:
        future: Future
        out_dir: Path
        window: int
        t0: float

        async def wait(self) -> None:
            await asyncio.to_thread(self.future.result)

    async def save_local_async(self, *, model, window: int, sync_window: int, global_step: int,
                               topology: str = "FSDP") -> "DCPCheckpointer.SaveHandle":
        from torch.distributed.checkpoint.state_dict_saver import AsyncCheckpointerType, async_save

        out_dir = self._local_dir(Layout(self.version, window))
        snap = SnapshotState(model)
        if _rank() == 0:
            (out_dir / "extra_metadata.json").write_text(json.dumps(
                self._sidecar(window, sync_window, global_step, _world(), topology), indent=2))
        t0 = time.perf_counter()
        fut = async_save(state_dict={"app": snap}, checkpoint_id=str(out_dir), process_group=self._cpu_pg,
                         async_checkpointer_type=AsyncCheckpointerType.THREAD)
        return DCPCheckpointer.SaveHandle(future=fut, out_dir=out_dir, window=window, t0=t0)

    # -- upload ---------------------------------------------------------------------------------
    async def _remote_names(self, layout: Layout) -> set[str]:
        objs = await _retry_n(lambda: self.comms.store.list(self.comms.bucket, f"{layout.prefix}/"),
                              desc=f"LIST {layout.prefix}/")
        return {Path(o.key).name for o in objs}

    async def upload(self, *, window: int, background: bool = False, delete_local_on_success: bool = True,
                     wait_for: "DCPCheckpointer.SaveHandle | None" = None, process_group=None,
                     pointer_poll_timeout_s: float = 800.0, pointer_poll_interval_s: float = 20.0,
                     fs_rescan_timeout_s: float = 20.0, fs_rescan_interval_s: float = 0.5, shared_fs: bool = True,
                     mop_up_missing: bool = True, pointer_require_all_ranks: bool = True,
                     initial_sleep_s: float = 10.0) -> None:
        layout = Layout(self.version, window)
        local_dir = self._local_dir(layout)

        async def _do() -> None:
            if wait_for is not None:
                await wait_for.wait()
            world, r = _world(process_group), _rank(process_group)
            await asyncio.sleep(initial_sleep_s)

            def scan():
                files = [p for p in local_dir.iterdir() if p.is_file()]
                return [q for q in files if not _is_meta(q)], [q for q in files if _is_meta(q)]

            data_files, meta_files = scan()
            owned = [p for p in data_files if _owner_rank_from_name(p.name) == r]
            if shared_fs and not owned:
                deadline = time.perf_counter() + fs_rescan_timeout_s
                while time.perf_counter() < deadline and not owned:
                    await asyncio.sleep(fs_rescan_interval_s)
                    data_files, meta_files = scan()
                    owned = [p for p in data_files if _owner_rank_from_name(p.name) == r]

            async def put(p: Path):
                await _retry_n(lambda: self.comms.s3_put_object(key=f"{layout.prefix}/{p.name}", file_path=str(p)),
                               desc=f"PUT {layout.prefix}/{p.name}")

            todo = list(owned) + (list(meta_files) if r == 0 else [])
            if todo:
                await asyncio.gather(*(put(p) for p in todo))
            if r == 0:
                try:
                    saved_world = int(json.loads((local_dir / "extra_metadata.json").read_text()).get("world_size_at_save", world))
                except Exception:  # noqa: BLE001
                    saved_world = world
                local_owners = {o for p in data_files if (o := _owner_rank_from_name(p.name)) is not None}
                expected = set(range(saved_world)) if pointer_require_all_ranks else (local_owners or set(range(saved_world)))
                # DCP may legitimately give a rank no shard file (all tensors deduplicated elsewhere)
                expected = expected & local_owners if shared_fs and local_owners else expected

                def owners(names):
                    return {o for n in names if (o := _owner_rank_from_name(n)) is not None}

                deadline = time.perf_counter() + float(pointer_poll_timeout_s)
                ok = False
                while True:
                    if expected.issubset(owners(await self._remote_names(layout))):
                        ok = True
                        break
                    if time.perf_counter() >= deadline:
                        break
                    await asyncio.sleep(min(pointer_poll_interval_s, max(deadline - time.perf_counter(), 0.01)))
                if not ok and mop_up_missing and shared_fs:
                    remote = await self._remote_names(layout)
                    fix = [p for p in local_dir.iterdir() if p.is_file() and not _is_meta(p)
                           and _owner_rank_from_name(p.name) in expected and p.name not in remote]
                    if fix:
                        await asyncio.gather(*(put(p) for p in fix))
                    ok = expected.issubset(owners(await self._remote_names(layout)))
                    if not ok:
                        logger.warning(f"[DCP][upload] after mop-up shards of some ranks are still missing (expected {sorted(expected)})")
                ptr = local_dir / "_LATEST.json"
                ptr.write_text(json.dumps({"latest_window": int(window)}, indent=2))
                await _retry_n(lambda: self.comms.s3_put_object(key=f"checkpoints/{self.version}/_LATEST.json",
                                                                file_path=str(ptr)), desc="PUT _LATEST.json")
                logger.info(f"[DCP][upload] published pointer for version {self.version} → window {window}")
            if delete_local_on_success:
                for p in owned + (meta_files if r == 0 else []):
                    p.unlink(missing_ok=True)
                if r == 0:
                    (local_dir / "_LATEST.json").unlink(missing_ok=True)
                    try:
                        next(local_dir.iterdir())
                    except StopIteration:
                        local_dir.rmdir()
                    except OSError as e:
                        logger.debug(f"[DCP] could not inspect {local_dir}: {e}")

        if background:
            t = asyncio.create_task(_do())
            self._bg.add(t)
            t.add_done_callback(self._bg.discard)
        else:
            await _do()

    async def flush_background_uploads(self) -> None:
        if self._bg:
            await asyncio.gather(*list(self._bg), return_exceptions=True)
            self._bg.clear()

    # -- discovery / download ------------------------------------------------------------------
    async def _choose_read_bucket(self, prefer_highest_staked: bool = True):
        if prefer_highest_staked:
            try:
                bucket, _ = await self.comms._get_highest_stake_validator_bucket()
                if bucket is not None:
                    return bucket
            except Exception as e:  # noqa: BLE001
                logger.debug(f"[DCP] highest-stake validator bucket not available ({e}); reading from the own bucket")
        return self.comms.bucket

    async def _discover_latest(self, *, prefer_highest_staked: bool = True) -> int | None:
        bucket = await self._choose_read_bucket(prefer_highest_staked)
        try:
            obj = await self.comms.s3_get_object(key=f"checkpoints/{self.version}/_LATEST.json", bucket=bucket)
            if isinstance(obj, dict) and "latest_window" in obj:
                return int(obj["latest_window"])
        except Exception as e:  # noqa: BLE001
            logger.debug(f"[DCP] no readable _LATEST.json ({e}); listing the checkpoint prefix instead")
        prefix = Layout(self.version).prefix + "/"
        windows = set()
        for o in await self.comms.store.list(bucket, prefix):
            m = re.match(rf"^{re.escape(prefix)}(\d+)/", o.key)
            if m:
                windows.add(int(m.group(1)))
        return max(windows) if windows else None

    async def _fetch(self, bucket, key: str, local_dir: Path) -> bool:
        return bool(await _retry_n(lambda: self.comms.store.get_to_file(bucket, key, str(local_dir / Path(key).name)),
                                   desc=f"GET {key}"))

    async def download_all(self, *, window: int | None = None, prefer_highest_staked: bool = True) -> Path | None:
        if window is None:
            window = await self._discover_latest(prefer_highest_staked=prefer_highest_staked)
            if window is None:
                return None
        layout = Layout(self.version, window)
        bucket = await self._choose_read_bucket(prefer_highest_staked)
        objs = await _retry_n(lambda: self.comms.store.list(bucket, f"{layout.prefix}/"), desc=f"LIST {layout.prefix}/")
        if not objs:
            return None                 # no local directory is made for a window that does not exist remotely
        local_dir = self._local_dir(layout)
        await asyncio.gather(*(self._fetch(bucket, o.key, local_dir) for o in objs))
        return local_dir

    async def download_distributed(self, *, window: int | None = None, prefer_highest_staked: bool = True,
                                   process_group=None) -> Path | None:
        """Shared file system: rank 0 fetches metadata, shard files are split over the ranks by a
        hash of their name, rank 0 then fetches anything still missing; two barriers bracket it."""
        if window is None:
            window = await self._discover_latest(prefer_highest_staked=prefer_highest_staked)
            if window is None:
                return None
        layout = Layout(self.version, window)
        bucket = await self._choose_read_bucket(prefer_highest_staked)
        world, r = _world(process_group), _rank(process_group)
        objs = await _retry_n(lambda: self.comms.store.list(bucket, f"{layout.prefix}/"), desc=f"LIST {layout.prefix}/")
        if not objs:
            return None
        local_dir = self._local_dir(layout)
        mine = []
        for o in objs:
            if _is_meta(o.key):
                if r == 0:
                    mine.append(o.key)
            elif int.from_bytes(hashlib.blake2b(Path(o.key).name.encode(), digest_size=8).digest(), "big") % world == r:
                mine.append(o.key)
        if mine:
            await asyncio.gather(*(self._fetch(bucket, k, local_dir) for k in mine))
        _barrier(process_group)
        if r == 0:
            missing = [o.key for o in objs if not (local_dir / Path(o.key).name).exists()]
            if missing:
                await asyncio.gather(*(self._fetch(bucket, k, local_dir) for k in missing))
        _barrier(process_group)
        return local_dir

    def load_local(self, *, model, window: int, process_group=None) -> None:
        d = self._local_dir(Layout(self.version, window))
        dcp.load(state_dict={"app": AppState(model)}, checkpoint_id=str(d), process_group=process_group)

    async def download_and_load(self, *, model, window: int | None = None, shared_fs: bool = True, process_group=None,
                                prefer_highest_staked: bool = True) -> tuple[int, int] | None:
        """Returns ``(sync_window, global_step)`` (global_step −1 when the sidecar has none)."""
        if shared_fs:
            local_dir = await self.download_distributed(window=window, prefer_highest_staked=prefer_highest_staked,
                                                        process_group=process_group)
        else:
            local_dir = await self.download_all(window=window, prefer_highest_staked=prefer_highest_staked)
        if local_dir is None:
            return None
        w = int(Path(local_dir).name)
        try:
            self.load_local(model=model, window=w, process_group=process_group)
        except Exception as e:  # noqa: BLE001
            logger.error(f"[DCP] load of window {w} failed: {e}")
            return None
        try:
            side = json.loads((Path(local_dir) / "extra_metadata.json").read_text())
            return int(side.get("sync_window", w)), int(side.get("global_step", -1))
        except Exception:  # noqa: BLE001
            return w, -1

    async def check_checkpoint_exists(self, *, window: int, prefer_highest_staked: bool = True) -> bool:
        """True when the window's metadata, sidecar and the shards of every writer rank are listed."""
        layout = Layout(self.version, window)
        bucket = await self._choose_read_bucket(prefer_highest_staked)
        try:
            objs = await self.comms.store.list(bucket, f"{layout.prefix}/")
        except Exception as e:  # noqa: BLE001
            logger.warning(f"[DCP] listing {layout.prefix}/ failed: {e}")
            return False
        names = {Path(o.key).name for o in objs}
        if ".metadata" not in names or "extra_metadata.json" not in names:
            return False
        owners = {o for n in names if (o := _owner_rank_from_name(n)) is not None}
        if not owners:
            return False
        side = await self.comms.s3_get_object(key=f"{layout.prefix}/extra_metadata.json", bucket=bucket)
        if isinstance(side, dict) and "shard_owners" in side:
            return set(side["shard_owners"]).issubset(owners)
        return True

    def cleanup_local_checkpoints(self, keep_latest: int = 1) -> None:
        base = self.repo_root / Layout(self.version).prefix
        if not base.is_dir():
            return
        dirs = [p for p in base.iterdir() if p.is_dir() and p.name.isdigit()]
        # only directories that hold a finished checkpoint count as "latest".  Empty directories go; a partial
        # one goes when a newer finished checkpoint exists, otherwise it may be a save in progress and stays
        whole = sorted((int(p.name) for p in dirs if (p / ".metadata").exists()), reverse=True)
        keep = set(whole[:keep_latest])
        for p in dirs:
            n = int(p.name)
            if n in keep:
                continue
            finished = (p / ".metadata").exists()
            empty = not any(p.iterdir())
            if finished or empty or (whole and n < whole[0]):
                shutil.rmtree(p, ignore_errors=True)
