"""Storage-backed exchange of gradients, peer lists, start windows and debug slices.

Public surface and object naming follow the reference's ``Comms`` (src/tplr/comms.py:62-2822):

* objects: ``gradient-{window}-{uid}-v{version}.pt`` / ``debug-…`` in the sender's bucket,
  ``aggregator-{window}-v{version}.pt`` in the aggregator bucket, ``peers_{window}_v{version}.json``
  and ``start_window_v{version}.json`` in the lead validator's bucket; a ``.pt`` holds
  ``{"state_dict": …, "global_step": n}`` and is read back with ``weights_only=True``;
* ``get`` honours an upload-time window (``time_min`` / ``time_max`` against the object's
  last-modified stamp → ``TOO_EARLY`` / ``TOO_LATE``); ``get_with_retry`` polls every 0.5 s and
  makes exactly one more attempt once ``time_max`` + 3 s has passed;
* ``gather`` fetches all peers concurrently (600 s cap), validates every payload (quantisation
  parameters finite and bounded, 12-bit indices in range with the expected k, values finite,
  shape prefix equal to the full-tensor chunk grid, every expected key present) and returns
  per-key *lists* over the accepted peers; ``gather_with_reserve`` tops up from a reserve tier.

The transport is a pluggable :class:`~templar_b200.backends.store.ObjectStore` (S3/R2, local
directory, in-memory with fault injection), so the whole protocol runs offline.
"""

from __future__ import annotations

import asyncio
import json
import math
import os
import random
import re
import shutil
import time
from datetime import datetime, timezone
from functools import partial
from types import SimpleNamespace
from typing import Any, Literal

import torch

from . import __version__
from .backends.store import LocalFSStore, MemoryStore, ObjectStore, S3Store, download_params
from .chain import ChainManager
from .compress import TopKCompressor, unpack_12bit_indices
from .config import BUCKET_SECRETS
from .logging import P, T, log_with_context, logger
from .schemas import Bucket, CommsGetResult

CF_REGION_NAME = "enam"
LOCAL_TMP_DIR = os.environ.get("TPLR_LOCAL_STORE", "/tmp/local_store")
PEERS_FILE_PREFIX = "peers_"
CPU_COUNT = os.cpu_count() or 4
CPU_MAX_CONNECTIONS = min(100, max(30, CPU_COUNT * 4))       # connection-pool bound of the object-store clients
SAFE_BUCKET_RE = re.compile(r"^[a-zA-Z0-9._-]+$")           # bucket names and object keys a node will talk about
SAFE_KEY_RE = re.compile(r"^[a-zA-Z0-9._/-]+$")
_WINDOW_RE = re.compile(r"^(?:gradient|debug|aggregator|checkpoint)-(\d+)-")


def default_store() -> ObjectStore:
    kind = os.environ.get("TPLR_STORE", "").lower()
    if kind == "memory":
        return MemoryStore()
    if kind != "local" and not BUCKET_SECRETS.get("_missing"):
        try:
            import aiobotocore  # noqa: F401

            return S3Store(region=CF_REGION_NAME)
        except ImportError as e:
            # credentials say "object store": falling back to a private directory would cut the node off from
            # its peers without anybody noticing
            raise RuntimeError("bucket credentials are set but the aiobotocore package is not installed; "
                               "set TPLR_STORE=local for a local-directory store") from e
    return LocalFSStore(os.environ.get("TPLR_STORE_ROOT", "/tmp/tplr_store"))


def _placeholder(s: str | None, n: int, fill: str) -> str:
    return s if s else fill * n


class Comms(ChainManager):
    def __init__(self, wallet=None, save_location: str = "/tmp", key_prefix: str = "model", config=None,
                 hparams=None, uid: int | None = None, store: ObjectStore | None = None, subtensor=None, **kwargs):
        self.uid = uid
        self.wallet = wallet
        self.store = store or default_store()
        self.bucket = self.get_own_bucket("gradients", "write")
        super().__init__(config=config or SimpleNamespace(netuid=3), hparams=hparams, wallet=wallet, bucket=self.bucket,
                         subtensor=subtensor)
        hotkey = getattr(getattr(wallet, "hotkey", None), "ss58_address", "default")
        self.temp_dir = os.path.join("/tmp", f"templar_{hotkey}")
        os.makedirs(self.temp_dir, exist_ok=True)
        self.save_location = os.path.join(save_location, f"hotkey_{hotkey}")
        os.makedirs(self.save_location, exist_ok=True)
        self.key_prefix = key_prefix
        self.current_window = 0
        self.recent_windows = getattr(self.hparams, "recent_windows", 3)
        self.active_check_interval = getattr(self.hparams, "active_check_interval", 60)
        # how often the chain's bucket commitments are read again; an offline run with windows of seconds sets it low
        self.fetch_interval = getattr(self.hparams, "commitment_fetch_interval", self.fetch_interval)
        self.client_semaphore = asyncio.Semaphore(30)
        self.gather_semaphore = asyncio.Semaphore(20)
        self.gather_timeout = 600

    # ------------------------------------------------------------------------------------ #
    # buckets
    # ------------------------------------------------------------------------------------ #
    def get_own_bucket(self, bucket_type: Literal["gradients", "dataset", "aggregator"],
                       access_type: Literal["read", "write"] | None = None) -> Bucket:
        if bucket_type not in ("gradients", "dataset", "aggregator"):
            raise ValueError("bucket_type must be 'gradients', 'dataset' or 'aggregator'")
        if bucket_type in ("gradients", "aggregator") and access_type not in ("read", "write"):
            raise ValueError(f"For {bucket_type} bucket, access_type must be either 'read' or 'write'.")
        cfg = BUCKET_SECRETS.get(bucket_type) or {}
        if "multiple" in cfg:
            cfg = random.choice(cfg["multiple"])
        cred = (cfg.get("credentials") or {}).get(access_type or "read") or {}
        account = cfg.get("account_id")
        if not account:
            # offline: a per-uid account id that survives the 128-character chain commitment, where the
            # bucket name is by construction the account id (the aggregator / dataset buckets are shared)
            owner = self.uid if bucket_type == "gradients" and self.uid is not None else "shared"
            account = f"{bucket_type}-{owner}-".ljust(32, "0")[:32]
            cfg = {**cfg, "name": account}
        return Bucket(name=cfg.get("name") or account,
                      account_id=_placeholder(account, 32, "a"),
                      access_key_id=_placeholder(cred.get("access_key_id"), 32, "k"),
                      secret_access_key=_placeholder(cred.get("secret_access_key"), 64, "s"))

    def get_base_url(self, account_id: str) -> str:
        return f"https://{account_id}.r2.cloudflarestorage.com"

    def peer_bucket(self, uid) -> Bucket | None:
        return self.commitments.get(int(uid))

    # ------------------------------------------------------------------------------------ #
    # raw objects
    # ------------------------------------------------------------------------------------ #
    async def s3_put_object(self, key: str, file_path: str | None = None, bucket: Bucket | None = None) -> None:
        bucket = bucket or self.bucket
        async with self.client_semaphore:
            if file_path is None:
                raise ValueError("file_path is required")
            await self.store.put_file(bucket, key, file_path)

    async def s3_get_object(self, key: str, bucket: Bucket | None = None, timeout: int = 30,
                            time_min: datetime | None = None, time_max: datetime | None = None,
                            load_data: bool = True, show_progress: bool = True, map_location: str | None = None):
        """Returns the decoded object (dict for ``.pt``/``.json``), ``{"__status": …}`` when the upload
        time is outside ``[time_min, time_max]``, or None when it is missing / on error."""
        bucket = bucket or self.bucket
        tmp = os.path.join(self.temp_dir, f"temp_{os.getpid()}_{random.getrandbits(32):08x}_{os.path.basename(key)}")
        try:
            async with self.client_semaphore:
                info = await asyncio.wait_for(self.store.head(bucket, key), timeout=timeout)
                if info is None:
                    return None
                lm = info.last_modified
                norm = lambda t: t if t is None or t.tzinfo is not None else t.replace(tzinfo=timezone.utc)  # noqa: E731
                tmin, tmax = norm(time_min), norm(time_max)
                if tmin is not None and lm < tmin:
                    return {"__status": "TOO_EARLY"}
                if tmax is not None and lm > tmax:
                    return {"__status": "TOO_LATE"}
                if not load_data:
                    # the object becomes a local file at the path that the key spells (dataset shards are kept under
                    # the same relative or absolute path in the bucket and on disk; reference: src/tplr/comms.py:
                    # 608-617); written beside it first, so that a reader never sees half a file
                    part = f"{key}.part{os.getpid()}"
                    os.makedirs(os.path.dirname(key) or ".", exist_ok=True)
                    try:
                        if not await self.store.get_to_file(bucket, key, part):
                            return None
                        os.replace(part, key)
                    finally:
                        if os.path.exists(part):
                            os.remove(part)
                    return key
                ok = await asyncio.wait_for(self.store.get_to_file(bucket, key, tmp), timeout=max(timeout, 1) * 10)
                if not ok:
                    return None
            if key.endswith(".json"):
                with open(tmp) as f:
                    return json.load(f)
            dev = map_location if map_location is not None else getattr(self.config, "device", "cpu")
            return await asyncio.to_thread(torch.load, tmp, map_location=dev, weights_only=True)
        except asyncio.TimeoutError:
            logger.debug(f"Timeout fetching {key}")
            return None
        except Exception as e:  # noqa: BLE001
            logger.debug(f"s3_get_object({key}) failed: {e}")
            return None
        finally:
            if os.path.exists(tmp):
                os.remove(tmp)

    async def s3_head_object(self, key: str, bucket: Bucket | None = None):
        return await self.store.head(bucket or self.bucket, key)

    async def s3_get_object_size(self, bucket: Bucket, key: str) -> int | None:
        info = await self.store.head(bucket, key)
        return None if info is None else info.size

    async def upload_large_file(self, file_path: str, key: str, bucket: Bucket | None = None) -> None:
        """Multipart upload of a file, whatever its size (parallel parts, per-part retries, restart when the store
        forgets the upload; reference src/tplr/comms.py:634-891).  Stores without multipart take it as one object."""
        bucket = bucket or self.bucket
        up = getattr(self.store, "upload_large_file", None)
        if up is None:
            return await self.store.put_file(bucket, key, file_path)
        await up(bucket, key, file_path)

    _calc_download_params = staticmethod(download_params)      # the plan of a ranged download, under the reference's name

    async def download_large_file(self, bucket: Bucket, key: str, file_size: int, temp_file_path: str) -> bool:
        """Ranged, parallel, resumable download of ``key`` into ``temp_file_path`` (reference src/tplr/comms.py:
        936-1187); stores without ranged reads fetch the object whole."""
        down = getattr(self.store, "download_large_file", None)
        if down is None:
            return bool(await self.store.get_to_file(bucket, key, temp_file_path))
        return bool(await down(bucket, key, file_size, temp_file_path))

    async def s3_get_object_range(self, bucket: Bucket, key: str, start: int, end: int, timeout: int = 30) -> bytes | None:
        """Bytes ``start..end`` (inclusive) of an object, or None on a miss, a short read or a timeout
        (reference: src/tplr/comms.py:2648-2703)."""
        try:
            return await asyncio.wait_for(self.store.get_range(bucket, key, start, end), timeout=timeout)
        except asyncio.TimeoutError:
            logger.error(f"timeout reading bytes {start}-{end} of {key}")
        except Exception as e:  # noqa: BLE001
            logger.error(f"reading bytes {start}-{end} of {key} failed: {e}")
        return None

    # ------------------------------------------------------------------------------------ #
    # cleanup
    # ------------------------------------------------------------------------------------ #
    async def cleanup_local_data(self, uid, current_window: int, stale_retention: int) -> None:
        root = os.path.join(LOCAL_TMP_DIR, str(uid))
        if not os.path.isdir(root):
            return
        floor = current_window - stale_retention
        for name in os.listdir(root):
            if name.isdigit() and int(name) < floor:
                shutil.rmtree(os.path.join(root, name), ignore_errors=True)

    async def cleanup_s3_data(self, uid, current_window: int, stale_retention: int) -> None:
        try:
            floor = current_window - stale_retention
            stale = []
            for obj in await self.store.list(self.bucket, ""):
                m = _WINDOW_RE.match(obj.key)
                if m and f"-{uid}-" in obj.key and int(m.group(1)) < floor:
                    stale.append(obj.key)
            if stale:
                await self.store.delete(self.bucket, stale)
                logger.debug(f"Removed {len(stale)} stale objects")
        except Exception as e:  # noqa: BLE001
            logger.debug(f"cleanup_s3_data failed: {e}")

    # ------------------------------------------------------------------------------------ #
    # put / get
    # ------------------------------------------------------------------------------------ #
    def _filename(self, key: str, window: int, uid) -> str:
        if key == "aggregator":
            return f"{key}-{window}-v{__version__}.pt"
        return f"{key}-{window}-{uid}-v{__version__}.pt"

    def _aggregator_bucket(self, access: str) -> Bucket:
        return self.get_own_bucket("aggregator", access)

    async def put(self, state_dict: dict[str, Any], window: int, key: Literal["debug", "gradient", "aggregator"],
                  uid: str | None = None, global_step: int = 0, local: bool = True, stale_retention: int = 10) -> float:
        filename = self._filename(key, window, uid)
        bucket = self._aggregator_bucket("write") if key == "aggregator" else None
        t0 = T()
        tmp_dir = os.path.join("/tmp", str(self.uid))
        os.makedirs(tmp_dir, exist_ok=True)
        tmp = os.path.join(tmp_dir, f"temp_{filename}")
        try:
            await asyncio.to_thread(torch.save, {"state_dict": state_dict, "global_step": global_step}, tmp)
            if local:
                await self.cleanup_local_data(uid, window, stale_retention)
                dst_dir = os.path.join(LOCAL_TMP_DIR, str(uid), str(window))
                os.makedirs(dst_dir, exist_ok=True)
                os.replace(tmp, os.path.join(dst_dir, filename))
            else:
                await self.s3_put_object(filename, tmp, bucket)
                asyncio.create_task(self.cleanup_s3_data(uid, window, stale_retention))
        finally:
            if os.path.exists(tmp):
                os.remove(tmp)
        dt = T() - t0
        logger.info(f"{P(window, dt)} PUT {filename} <--")
        return dt

    async def gradient_timestamp(self, uid: int, window: int, version: str = __version__) -> float:
        bucket = self.commitments.get(int(uid))
        if not bucket:
            return 0.0
        try:
            info = await self.store.head(bucket, f"gradient-{window}-{uid}-v{version}.pt")
            return info.last_modified.timestamp() if info else 0.0
        except Exception:  # noqa: BLE001
            return 0.0

    async def get(self, uid: str, window: int, key: Literal["debug", "gradient", "aggregator"], local: bool = True,
                  stale_retention: int = 10, timeout: int = 30, time_min: datetime | None = None,
                  time_max: datetime | None = None, show_progress: bool = True,
                  map_location: str | None = None) -> CommsGetResult:
        filename = self._filename(key, window, uid)
        try:
            if local:
                await self.cleanup_local_data(uid, window, stale_retention)
                path = os.path.join(LOCAL_TMP_DIR, str(uid), str(window), filename)
                if not os.path.exists(path):
                    return CommsGetResult(status="NOT_FOUND")
                loaded = torch.load(path, weights_only=True, map_location=map_location)
                return CommsGetResult(data=loaded.get("state_dict"), global_step=loaded.get("global_step", 0))
            bucket = self._aggregator_bucket("read") if key == "aggregator" else self.commitments.get(int(uid))
            if not bucket:
                return CommsGetResult(status="NOT_FOUND")
            loaded = await self.s3_get_object(key=filename, bucket=bucket, timeout=timeout, time_min=time_min,
                                              time_max=time_max, show_progress=show_progress, map_location=map_location)
            if loaded is None:
                return CommsGetResult(status="NOT_FOUND")
            if isinstance(loaded, dict) and loaded.get("__status") in ("TOO_LATE", "TOO_EARLY"):
                return CommsGetResult(status=loaded["__status"])
            return CommsGetResult(data=loaded.get("state_dict"), global_step=loaded.get("global_step", 0))
        except Exception as e:  # noqa: BLE001
            logger.debug(f"GET error {filename}: {e}")
            return CommsGetResult(status="ERROR")

    async def get_with_retry(self, uid: str, window: int, key: str, timeout: int, local: bool = True,
                             stale_retention: int = 10, time_min: datetime | None = None,
                             time_max: datetime | None = None, show_progress: bool = False,
                             map_location: str | None = None) -> CommsGetResult | None:
        end = time.time() + timeout
        grace, tried_after_max = 3.0, False
        while True:
            if time.time() >= end:
                return None
            past_max = time_max is not None and (datetime.now(timezone.utc) - _aware(time_max)).total_seconds() > grace
            if past_max and tried_after_max:
                return None
            if past_max:
                tried_after_max = True
            result = await self.get(uid=uid, window=window, key=key, local=local, stale_retention=stale_retention,
                                    time_min=time_min, time_max=time_max, show_progress=show_progress,
                                    map_location=map_location)
            if result.success:
                return result
            if result.status in ("TOO_LATE", "TOO_EARLY"):
                logger.info(f"Gradient for UID {uid}, window {window} exists but was uploaded "
                            f"{result.status.lower().replace('_', ' ')}. Skipping.")
                return None
            await asyncio.sleep(0.5)

    # ------------------------------------------------------------------------------------ #
    # gather
    # ------------------------------------------------------------------------------------ #
    def validate_payload(self, uid, state_dict: dict, totalks: dict, xshapes: dict | None, device,
                         expected: set[str]) -> bool:
        """The per-peer acceptance test of ``gather`` (see module docstring)."""
        received = set()
        for name, tensor in state_dict.items():
            received.add(name)
            if name.endswith("quant_params"):
                if tensor is None:
                    continue
                if not isinstance(tensor, (tuple, list)) or len(tensor) != 5:
                    logger.warning(f"Malformed quant-params in {name} from UID {uid}")
                    return False
                shift, scale, _offset, lookup, _dtype = tensor
                try:
                    bad_shift = not bool(torch.isfinite(torch.as_tensor(shift, dtype=torch.float32)).all())
                except (TypeError, ValueError, RuntimeError):
                    bad_shift = True
                bad_scale = isinstance(scale, float) and (not math.isfinite(scale) or abs(scale) < 1e-12 or abs(scale) > 1e4)
                if bad_shift or bad_scale:
                    logger.warning(f"Bad quant-params in {name} from UID {uid}; shift={shift}, scale={scale}")
                    return False
                # The codes index this table on the device: its shape is checked here, on the host, so that a
                # short or oddly shaped table from a peer can never become an out-of-range gather on the GPU.
                # Peers may quantise with fewer bins than this node: any table that a byte can address is accepted,
                # as long as no code of the payload points past its end (checked below).
                if (not torch.is_tensor(lookup) or lookup.dim() != 1 or not lookup.is_floating_point()
                        or lookup.numel() < 1 or lookup.numel() > 256):
                    logger.warning(f"Lookup table of {name} from UID {uid} is not a 1-D float table of 1..256 entries")
                    return False
                if not torch.isfinite(lookup).all():
                    logger.warning(f"Lookup table contains non-finite values in {name} from UID {uid}")
                    return False
                codes = state_dict.get(name[: -len("quant_params")] + "vals")
                if (torch.is_tensor(codes) and codes.dtype == torch.uint8 and codes.numel()
                        and int(codes.max()) >= lookup.numel()):
                    logger.warning(f"Value codes of {name} from UID {uid} exceed the lookup table")
                    return False
            elif name.endswith("idxs"):
                base = name[:-4]
                tk = totalks.get(base)
                if tk is None:
                    logger.warning(f"Missing totalk for parameter {base} from UID {uid}, skipping UID.")
                    return False
                tk = tk if isinstance(tk, int) else tk.numel()
                try:
                    self.check_compressed_indices(name, tensor, tk, allowed_topk=getattr(self.hparams, "topk_compression", None),
                                                  vals=state_dict.get(base + "vals"))
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"Compressed indices check failed for parameter {name} from UID {uid}: {e}")
                    return False
            elif name.endswith("vals"):
                base = name[:-4]
                if tensor.dtype == torch.uint8:
                    if tensor.nelement() == 0:
                        logger.warning(f"Empty tensor in {name} from UID {uid}, skipping")
                        return False
                    if state_dict.get(base + "quant_params") is None:
                        logger.warning(f"Missing quant_params for quantized {name} from UID {uid}")
                        return False
                elif not torch.isfinite(tensor.to(device)).all():
                    logger.warning(f"NaN/Inf in {name} from UID {uid}, skipping")
                    return False
                if xshapes is not None and xshapes.get(base) is not None:
                    exp = tuple(xshapes[base])
                    prefix = exp[:2] if len(exp) == 4 else exp[:1]
                    if tuple(tensor.shape[:-1]) != tuple(prefix):
                        logger.warning(f"Shape mismatch for {name} from UID {uid}: expected shape prefix {prefix}, "
                                       f"got {tuple(tensor.shape[:-1])} (likely sharded gradient)")
                        return False
        missing = expected - received
        if missing:
            logger.warning(f"UID {uid} missing compressed parameters: {sorted(missing)[:4]}…, skipping UID.")
            return False
        return True

    async def gather(self, my_uid: int | None, uids: list[int], window: int, key: str, timeout: int, device: str,
                     totalks: dict, compressor: TopKCompressor | None = None,
                     expected_compressed_params: set[str] | None = None, local: bool = True, stale_retention: int = 10,
                     time_min: datetime | None = None, time_max: datetime | None = None,
                     xshapes: dict | None = None) -> SimpleNamespace | None:
        if not expected_compressed_params:
            expected_compressed_params = set()
        t_start = time.time()
        uids = sorted(uids)
        agg: dict[str, list] = {}
        valid, skipped, steps = [], [], []
        nbytes = 0
        # uids that run on this box and have posted this window's payload in peer memory are not fetched: the engine
        # reads them where they are (backends/store.py PeerMemoryStore)
        local_ranks: dict[int, int] = {}
        locate = getattr(self.store, "local_rank", None)
        if locate is not None and not local:
            for u in uids:
                r = locate(u, window)
                if r is not None:
                    local_ranks[int(u)] = int(r)
            uids = [u for u in uids if int(u) not in local_ranks]
        n_asked = len(uids) + len(local_ranks)
        async with self.gather_semaphore:
            tasks = [self.get_with_retry(uid=str(u), window=window, key=key, timeout=timeout, local=local,
                                         stale_retention=stale_retention, time_min=time_min, time_max=time_max,
                                         map_location=device) for u in uids]
            t0 = T()
            try:
                responses = await asyncio.wait_for(asyncio.gather(*tasks, return_exceptions=True),
                                                   timeout=self.gather_timeout)
            except asyncio.TimeoutError:
                logger.error(f"Gather download phase timed out after {self.gather_timeout}s. Aborting gather.")
                return None
            logger.info(f"{P(window, T() - t0)} Downloaded peer gradients <--")
            for uid, resp in zip(uids, responses):
                if isinstance(resp, Exception) or resp is None or getattr(resp, "data", None) is None:
                    if isinstance(resp, Exception):
                        log_with_context(level="debug", message=f"Error from UID {uid}: {resp}", current_window=window)
                    skipped.append(uid)
                    continue
                sd = resp.data
                try:
                    ok = self.validate_payload(uid, sd, totalks, xshapes, device, set(expected_compressed_params))
                except Exception as e:  # noqa: BLE001
                    logger.warning(f"Validation of UID {uid} raised {e}")
                    ok = False
                if not ok:
                    logger.info(f"Skipping UID {uid} due to validation failures")
                    skipped.append(uid)
                    continue
                for name, tensor in sd.items():
                    if name.endswith(("idxs", "vals", "quant_params")):
                        agg.setdefault(name, []).append(tensor)
                        if torch.is_tensor(tensor):
                            nbytes += tensor.element_size() * tensor.nelement()
                valid.append(uid)
                steps.append(resp.global_step)
        if not valid and not local_ranks:
            logger.info("No valid gradients received from any UID")
            return None
        dt = time.time() - t_start
        n_ok = len(valid) + len(local_ranks)
        logger.info(f"Gather done in {dt:.2f}s. Success rate: {n_ok}/{n_asked}, Download: {nbytes} bytes"
                    + (f", {len(local_ranks)} from peer memory" if local_ranks else ""))
        # fetched peers come first (their list entries fill the engine's slots in this order), then the co-located ones
        return SimpleNamespace(time=dt, upload_bytes=0, download_bytes=nbytes, success_rate=n_ok / max(n_asked, 1),
                               state_dict=SimpleNamespace(**agg), uids=valid + sorted(local_ranks), global_steps=steps,
                               skipped_uids=skipped, local_ranks=local_ranks)

    async def gather_with_reserve(self, *, my_uid: int | None, gather_uids: list[int], reserve_uids: list[int],
                                  expected_compressed_params: set[str] | None = None, **kwargs) -> SimpleNamespace | None:
        if not gather_uids:
            return None
        expected_compressed_params = expected_compressed_params or set()
        ctx = partial(log_with_context, level="info", window=kwargs.get("window"))
        ctx(message=f"[gather_with_reserve] start | gather={gather_uids} reserve={reserve_uids}")
        primary = await self.gather(my_uid=my_uid, uids=gather_uids,
                                    expected_compressed_params=expected_compressed_params, **kwargs)
        if primary is None:
            primary = SimpleNamespace(time=0.0, upload_bytes=0, download_bytes=0, success_rate=0.0,
                                      state_dict=SimpleNamespace(), uids=[], global_steps=[],
                                      skipped_uids=list(gather_uids))
        missing = set(gather_uids) - set(primary.uids)
        if missing and reserve_uids:
            repl = [u for u in reserve_uids if u not in primary.uids][: len(missing)]
            if repl:
                ctx(message=f"[gather_with_reserve] retrying with reserve uids={repl}")
                fb = await self.gather(my_uid=my_uid, uids=repl,
                                       expected_compressed_params=expected_compressed_params, **kwargs)
                if fb:
                    for k, v in vars(fb.state_dict).items():
                        setattr(primary.state_dict, k, getattr(primary.state_dict, k, []) + v)
                    n_fetched = len(primary.uids) - len(getattr(primary, "local_ranks", {}) or {})
                    fb_local = getattr(fb, "local_ranks", {}) or {}
                    fb_fetched = [u for u in fb.uids if u not in fb_local]
                    primary.uids[n_fetched:n_fetched] = fb_fetched          # fetched peers stay in front, in list order
                    primary.uids.extend(sorted(fb_local))
                    primary.local_ranks = {**(getattr(primary, "local_ranks", {}) or {}), **fb_local}
                    primary.global_steps.extend(fb.global_steps)
                    primary.skipped_uids.extend(fb.skipped_uids)
                    primary.upload_bytes += fb.upload_bytes
                    primary.download_bytes += fb.download_bytes
        target = len(gather_uids)
        primary.success_rate = len(primary.uids) / target if target else 0.0
        ctx(message=f"[gather_with_reserve] done | {len(primary.uids)}/{target} skipped={primary.skipped_uids}")
        return primary if primary.uids else None

    def check_compressed_indices(self, param_name: str, idxs: torch.Tensor, totalk: int,
                                 allowed_topk: int | None = None, vals: torch.Tensor | None = None) -> None:
        """Raises ``ValueError`` unless ``idxs`` is a well-formed 12-bit packed index tensor for ``vals``."""
        default_k = getattr(self.hparams, "topk_compression", totalk)
        allowed_topk = min(default_k if allowed_topk is None else allowed_topk, totalk)
        if not isinstance(idxs, torch.Tensor):
            raise ValueError(f"[{param_name}] Expected tensor but got {type(idxs)}")
        if idxs.dtype != torch.uint8:
            raise ValueError(f"[{param_name}] Expected uint8 for 12-bit packed indices, got {idxs.dtype}")
        if vals is None:
            raise ValueError(f"[{param_name}] Values tensor required to validate 12-bit packed indices")
        if idxs.numel() == 0:
            raise ValueError(f"[{param_name}] Empty packed indices tensor")
        try:
            if idxs.numel() * 2 != vals.numel() * 3:
                raise ValueError(f"packed length {idxs.numel()} does not match {vals.numel()} values")
            unpacked = unpack_12bit_indices(idxs, vals.shape)
            if unpacked.shape[-1] != allowed_topk:
                raise ValueError(f"Invalid topk dimension: shape[-1]={unpacked.shape[-1]} but expected {allowed_topk}")
            lo, hi = int(unpacked.min()), int(unpacked.max())
            if lo < 0 or hi >= totalk:
                raise ValueError(f"Index {hi if hi >= totalk else lo} out of bounds (totalk = {totalk})")
        except Exception as e:  # noqa: BLE001
            raise ValueError(f"[{param_name}] Failed to unpack 12-bit indices: {e}") from e

    # ------------------------------------------------------------------------------------ #
    # liveness
    # ------------------------------------------------------------------------------------ #
    async def is_miner_active(self, uid: int, recent_windows: int = 3) -> bool:
        bucket = self.commitments.get(uid)
        if not bucket or self.current_window is None:
            return False
        try:
            for w in range(self.current_window - recent_windows, self.current_window + 1):
                if await self.store.head(bucket, f"gradient-{w}-{uid}-v{__version__}.pt") is not None:
                    return True
        except Exception as e:  # noqa: BLE001
            logger.error(f"Error accessing bucket for UID {uid}: {e}")
        return False

    async def refresh_active_peers(self) -> set[int]:
        sem = asyncio.Semaphore(min(30, len(self.commitments) or 10))
        active: set[int] = set()

        async def check(uid):
            async with sem:
                if await self.is_miner_active(uid, self.recent_windows):
                    active.add(uid)

        uids = list(self.commitments.keys())
        for i in range(0, len(uids), 50):
            await asyncio.gather(*(check(u) for u in uids[i:i + 50]))
        self.active_peers = active
        return active

    async def track_active_peers(self) -> None:
        while True:
            await self.refresh_active_peers()
            logger.info(f"Updated active peers: {sorted(int(u) for u in self.active_peers)}")
            await asyncio.sleep(self.active_check_interval)

    # ------------------------------------------------------------------------------------ #
    # validator-published control files
    # ------------------------------------------------------------------------------------ #
    async def _get_highest_stake_validator_bucket(self):
        if self.metagraph is None:
            return None, None
        uid = int(self.metagraph.S.argmax().item())
        bucket = self.commitments.get(uid)
        return (bucket, uid) if bucket else (None, None)

    async def _put_json(self, key: str, obj: dict, bucket: Bucket | None = None) -> None:
        tmp = os.path.join(self.temp_dir, f"temp_{key}")
        try:
            with open(tmp, "w") as f:
                json.dump(obj, f)
            await self.s3_put_object(key=key, file_path=tmp, bucket=bucket)
        finally:
            if os.path.exists(tmp):
                os.remove(tmp)

    async def post_peer_list(self, *, peers: list[int], reserve_peers: list[int] | None = None,
                             first_effective_window: int, sync_window: int, initial_selection: bool) -> None:
        key = f"{PEERS_FILE_PREFIX}{first_effective_window}_v{__version__}.json"
        try:
            await self._put_json(key, {"peers": peers, "reserve_peers": reserve_peers or [],
                                       "initial_selection": initial_selection, "sync_window": sync_window,
                                       "first_effective_window": first_effective_window})
            logger.info(f"PUT {key} <--")
        except Exception as e:  # noqa: BLE001
            logger.info(f"Failed to upload peer list: {e}")

    async def post_start_window(self, start_window: int) -> None:
        await self._put_json(f"start_window_v{__version__}.json", {"start_window": start_window})

    async def get_peer_list(self, fetch_previous: bool = False, retries: int = -1,
                            retry_delay: float = 10.0) -> tuple[list[int], list[int], int] | None:
        pattern = re.compile(rf"^{PEERS_FILE_PREFIX}(?P<window>\d+)_v{re.escape(__version__)}\.json$")
        attempt = 0
        while retries == -1 or attempt < max(retries, 1):
            attempt += 1
            try:
                bucket, vuid = await self._get_highest_stake_validator_bucket()
                if bucket is None:
                    logger.warning("No highest staked validator bucket found. Retrying.")
                    await asyncio.sleep(retry_delay)
                    continue
                by_window = {}
                for obj in await self.store.list(bucket, PEERS_FILE_PREFIX):
                    m = pattern.match(obj.key)
                    if m:
                        by_window[int(m.group("window"))] = obj.key
                if not by_window:
                    logger.info("No peer list files found")
                    return None
                windows = sorted(by_window, reverse=True)
                if fetch_previous:
                    if len(windows) < 2:
                        return None
                    chosen = windows[1]
                else:
                    chosen = windows[0]
                data = await self.s3_get_object(key=by_window[chosen], bucket=bucket)
                if data is None:
                    return None
                if not isinstance(data, dict):
                    data = json.loads(bytes(data).decode("utf-8"))
                return data["peers"], data.get("reserve_peers", []), data["first_effective_window"]
            except Exception as e:  # noqa: BLE001
                logger.error(f"Error fetching peer list: {e}")
                await asyncio.sleep(retry_delay)
        return None

    async def get_start_window(self, retries: int = -1, version: str | None = None,
                               retry_delay: float = 10.0) -> int | None:
        attempt = 0
        while retries == -1 or attempt < retries:
            attempt += 1
            try:
                bucket, vuid = await self._get_highest_stake_validator_bucket()
                if bucket is None:
                    logger.warning("No highest staked validator bucket found. Retrying.")
                    await asyncio.sleep(retry_delay)
                    continue
                data = await self.s3_get_object(key=f"start_window_v{version or __version__}.json", bucket=bucket)
                if data is not None:
                    if not isinstance(data, dict):
                        data = json.loads(bytes(data).decode("utf-8"))
                    return int(data["start_window"])
                logger.warning("start_window.json not found or empty. Retrying.")
            except Exception as e:  # noqa: BLE001
                logger.error(f"Error fetching start_window: {e}")
            await asyncio.sleep(retry_delay)
        return None

    async def get_debug_dict(self, window: int):
        """The lead validator's debug slice for ``window`` (None when unavailable)."""
        bucket, vuid = await self._get_highest_stake_validator_bucket()
        if bucket is None or vuid is None:
            return None
        loaded = await self.s3_get_object(key=f"debug-{window}-{vuid}-v{__version__}.pt", bucket=bucket, timeout=20)
        if isinstance(loaded, dict) and "state_dict" in loaded:
            return loaded["state_dict"]
        return loaded

    # ------------------------------------------------------------------------------------ #
    def weighted_random_sample_no_replacement(self, candidates: list[int], weights: list[int | float], k: int) -> list[int]:
        """Draw up to ``k`` distinct candidates with probability proportional to their weight."""
        if not candidates or not weights or k <= 0:
            return []
        pool = [(c, float(w)) for c, w in zip(candidates, weights) if w > 0]
        total = sum(w for _, w in pool)
        if total <= 0:
            return []
        k = min(k, len(pool))
        chosen = []
        for _ in range(k):
            total = sum(w for _, w in pool)
            if total <= 0:
                break
            r = random.uniform(0.0, total)
            acc = 0.0
            for i, (c, w) in enumerate(pool):
                acc += w
                if r <= acc:
                    chosen.append(c)
                    pool.pop(i)
                    break
        return chosen

    async def close(self) -> None:
        task = getattr(self, "_active_task", None)
        if task is not None:
            task.cancel()
            self._active_task = None
        await self.store.close()

    close_all_s3_clients = close          # the reference's name (src/tplr/comms.py:181-189)

    def start_background_tasks(self) -> None:
        """Start the peer-activity tracker on the running loop (reference src/tplr/comms.py:205-218).  Neurons that
        refresh the active set themselves once per window do not need it."""
        if getattr(self, "_active_task", None) is None:
            self.loop = asyncio.get_running_loop()
            self._active_task = self.loop.create_task(self.track_active_peers())

    @staticmethod
    def delete_local_directory(path: str) -> None:
        """Remove a directory tree of the local store; a missing path is not an error."""
        import shutil

        shutil.rmtree(path, ignore_errors=True)


def _aware(t: datetime) -> datetime:
    return t if t.tzinfo is not None else t.replace(tzinfo=timezone.utc)
