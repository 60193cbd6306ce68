"""Object-store backends behind :class:`templar_b200.comms.Comms`.

``ObjectStore`` is the small async interface Comms needs (put/get/head/list/delete by
``(bucket, key)``).  Implementations:

* :class:`LocalFSStore` — a directory per bucket; what offline runs, tests and single-box
  deployments use.  ``last_modified`` is the file mtime, so the upload-time window checks work.
* :class:`MemoryStore` — in-process dict with fault injection (drop, delay, corrupt, stale
  timestamps) for failure-handling tests; nothing touches a GPU.
* :class:`S3Store` — S3/R2 through aiobotocore when it is installed: persistent clients per
  credential, multipart upload for large files with per-part retries and restart on a vanished
  upload id, parallel ranged download with resume for very large objects.  Mirrors the transport
  behaviour of the reference (src/tplr/comms.py:140-203, :634-891, :936-1187) behind the same
  interface; the client factory is injectable so the logic is testable with a fake client.
* :class:`PeerMemoryStore` — wraps one of the above for nodes that share a box: gradients of co-located uids are
  not fetched at all but read by the aggregation kernel from the owner's GPU memory.
"""

from __future__ import annotations

import asyncio
import hashlib
import os
import shutil
from dataclasses import dataclass
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Callable

from ..logging import logger
from ..schemas import Bucket


@dataclass
class ObjectInfo:
    key: str
    size: int
    last_modified: datetime


class ObjectStore:
    async def put_file(self, bucket: Bucket, key: str, path: str) -> None: raise NotImplementedError
    async def put_bytes(self, bucket: Bucket, key: str, data: bytes) -> None: raise NotImplementedError
    async def get_bytes(self, bucket: Bucket, key: str) -> bytes | None: raise NotImplementedError
    async def get_to_file(self, bucket: Bucket, key: str, path: str) -> bool: raise NotImplementedError
    async def head(self, bucket: Bucket, key: str) -> ObjectInfo | None: raise NotImplementedError
    async def list(self, bucket: Bucket, prefix: str = "") -> list[ObjectInfo]: raise NotImplementedError
    async def delete(self, bucket: Bucket, keys: list[str]) -> None: raise NotImplementedError
    async def close(self) -> None: return None

    async def get_range(self, bucket: Bucket, key: str, start: int, end: int) -> bytes | None:
        """Bytes ``start..end`` (inclusive, as in an HTTP Range header) of an object; None when the object is
        missing or shorter than ``end + 1``.  Transports without a ranged read slice the whole object."""
        data = await self.get_bytes(bucket, key)
        if data is None or start < 0 or end < start or len(data) <= end:
            return None
        return data[start:end + 1]


# --------------------------------------------------------------------------------------- #
class LocalFSStore(ObjectStore):
    def __init__(self, root: str | os.PathLike):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)

    def _path(self, bucket: Bucket, key: str) -> Path:
        return self.root / bucket.name / key

    async def put_file(self, bucket, key, path):
        dst = self._path(bucket, key)
        dst.parent.mkdir(parents=True, exist_ok=True)
        tmp = dst.with_name(dst.name + f".part{os.getpid()}")
        await asyncio.to_thread(shutil.copyfile, path, tmp)
        os.replace(tmp, dst)

    async def put_bytes(self, bucket, key, data):
        dst = self._path(bucket, key)
        dst.parent.mkdir(parents=True, exist_ok=True)
        tmp = dst.with_name(dst.name + f".part{os.getpid()}")
        tmp.write_bytes(data)
        os.replace(tmp, dst)

    async def get_bytes(self, bucket, key):
        p = self._path(bucket, key)
        return await asyncio.to_thread(p.read_bytes) if p.is_file() else None

    async def get_to_file(self, bucket, key, path):
        p = self._path(bucket, key)
        if not p.is_file():
            return False
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        await asyncio.to_thread(shutil.copyfile, p, path)
        return True

    async def head(self, bucket, key):
        p = self._path(bucket, key)
        if not p.is_file():
            return None
        st = p.stat()
        return ObjectInfo(key, st.st_size, datetime.fromtimestamp(st.st_mtime, tz=timezone.utc))

    async def list(self, bucket, prefix=""):
        base = self.root / bucket.name
        if not base.is_dir():
            return []
        out = []
        for p in base.rglob("*"):
            if p.is_file() and ".part" not in p.name:
                key = str(p.relative_to(base))
                if key.startswith(prefix):
                    st = p.stat()
                    out.append(ObjectInfo(key, st.st_size, datetime.fromtimestamp(st.st_mtime, tz=timezone.utc)))
        return sorted(out, key=lambda o: o.key)

    async def delete(self, bucket, keys):
        for k in keys:
            try:
                self._path(bucket, k).unlink()
            except FileNotFoundError:
                pass


# --------------------------------------------------------------------------------------- #
class MemoryStore(ObjectStore):
    """Dict-backed store. ``faults`` maps a key substring to ``"drop" | "corrupt" | ("delay", s) |
    ("mtime", datetime)`` and is consulted on reads — the host-side fault injector of the test tier."""

    def __init__(self):
        self.objects: dict[tuple[str, str], tuple[bytes, datetime]] = {}
        self.faults: dict[str, Any] = {}
        self.reads = 0

    def _fault(self, key):
        for pat, f in self.faults.items():
            if pat in key:
                return f
        return None

    async def put_file(self, bucket, key, path):
        await self.put_bytes(bucket, key, Path(path).read_bytes())

    async def put_bytes(self, bucket, key, data):
        self.objects[(bucket.name, key)] = (bytes(data), datetime.now(timezone.utc))

    async def get_bytes(self, bucket, key):
        self.reads += 1
        f = self._fault(key)
        if f == "drop":
            return None
        if isinstance(f, tuple) and f[0] == "delay":
            await asyncio.sleep(f[1])
        item = self.objects.get((bucket.name, key))
        if item is None:
            return None
        data = item[0]
        if f == "corrupt":
            data = data[: len(data) // 2]
        return data

    async def get_to_file(self, bucket, key, path):
        data = await self.get_bytes(bucket, key)
        if data is None:
            return False
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_bytes(data)
        return True

    async def head(self, bucket, key):
        f = self._fault(key)
        if f == "drop":
            return None
        item = self.objects.get((bucket.name, key))
        if item is None:
            return None
        mtime = f[1] if isinstance(f, tuple) and f[0] == "mtime" else item[1]
        return ObjectInfo(key, len(item[0]), mtime)

    async def list(self, bucket, prefix=""):
        return sorted((ObjectInfo(k, len(v[0]), v[1]) for (b, k), v in self.objects.items()
                       if b == bucket.name and k.startswith(prefix)), key=lambda o: o.key)

    async def delete(self, bucket, keys):
        for k in keys:
            self.objects.pop((bucket.name, k), None)


# --------------------------------------------------------------------------------------- #
class PeerMemoryStore(ObjectStore):
    """The transport of nodes that share a box: gradients of co-located uids are read from peer memory, everything
    else goes through ``inner`` (a directory, S3 / R2, ...).

    Uploads are passed on unchanged, since peers and validators on other machines read them from the bucket.  What
    changes is the read side: :meth:`local_rank` tells :meth:`templar_b200.comms.Comms.gather` that a uid's payload of
    the current window sits in the symmetric heap of the rank it runs on, so the gather neither downloads nor
    deserialises it and the aggregation kernel pulls the packed payload over NVLink from the owner's buffers
    (see parallel/peer_group.py).  ``head`` answers for such gradients too, so liveness checks of co-located peers
    do not touch the bucket."""

    def __init__(self, inner: ObjectStore, peer_group):
        self.inner, self.peer_group = inner, peer_group

    def local_rank(self, uid: int, window: int) -> int | None:
        """Rank whose buffers hold ``uid``'s payload of ``window``, or None when that uid is not on this box (or has
        not posted this window)."""
        return self.peer_group.fresh(window).get(int(uid))

    def _local_gradient(self, key: str) -> bool:
        parts = key.split("-")
        if len(parts) < 3 or parts[0] != "gradient":
            return False
        try:
            window, uid = int(parts[1]), int(parts[2])
        except ValueError:
            return False
        return self.local_rank(uid, window) is not None

    async def put_file(self, bucket, key, path): return await self.inner.put_file(bucket, key, path)
    async def put_bytes(self, bucket, key, data): return await self.inner.put_bytes(bucket, key, data)
    async def get_bytes(self, bucket, key): return await self.inner.get_bytes(bucket, key)
    async def get_to_file(self, bucket, key, path): return await self.inner.get_to_file(bucket, key, path)
    async def list(self, bucket, prefix=""): return await self.inner.list(bucket, prefix)
    async def delete(self, bucket, keys): return await self.inner.delete(bucket, keys)
    async def close(self): return await self.inner.close()

    async def head(self, bucket, key):
        if self._local_gradient(key):
            return ObjectInfo(key, 0, datetime.now(timezone.utc))
        return await self.inner.head(bucket, key)

    def __getattr__(self, name):              # transport-specific extras (multipart plans, fault tables, ...)
        return getattr(self.inner, name)


# --------------------------------------------------------------------------------------- #
def download_params(file_size: int, custom_workers: str | None = None) -> dict:
    """Chunk size and worker count of a ranged download by object size (reference src/tplr/comms.py:1251-1285):
    above 100 GB 512 MB chunks and 8-32 workers, above 10 GB 256 MB and 8-16, below that 64 MB and 6-8; a valid
    ``custom_workers`` replaces the worker count; never more workers than chunks."""
    cpus = os.cpu_count() or 4
    gb = file_size / 1024 ** 3
    if gb > 100:
        chunk, workers = 512 * 1024 ** 2, min(32, max(8, cpus))
    elif gb > 10:
        chunk, workers = 256 * 1024 ** 2, min(16, max(8, cpus))
    else:
        chunk, workers = 64 * 1024 ** 2, min(8, max(6, 2 * cpus))
    if custom_workers:
        try:
            workers = max(1, int(custom_workers))
        except ValueError:
            pass
    chunks = max(1, -(-file_size // chunk))
    return {"chunk_size": chunk, "max_workers": min(workers, chunks), "total_chunks": chunks, "file_size_gb": gb}


def _is_named(e: BaseException, *names: str) -> bool:
    return any(c.__name__ in names for c in type(e).__mro__)


class S3Store(ObjectStore):
    """S3-compatible transport (Cloudflare R2 endpoint ``https://<account>.r2.cloudflarestorage.com``)."""

    MULTIPART_THRESHOLD = 100 * 1024 * 1024
    RANGED_GET_THRESHOLD = 1024 * 1024 * 1024

    def __init__(self, client_factory: Callable[[Bucket], Any] | None = None, *, part_size: int | None = None,
                 concurrency: int | None = None, max_retries: int = 5, region: str = "enam"):
        self._factory = client_factory or self._aiobotocore_client
        self._clients: dict[tuple, Any] = {}
        self._ctx: dict[tuple, Any] = {}
        self._lock = asyncio.Lock()
        self.part_size = part_size or int(os.getenv("TPLR_S3_PART_SIZE", 64 * 1024 * 1024))
        self.concurrency = concurrency or int(os.getenv("TPLR_S3_CONCURRENCY", 16))
        self.max_retries, self.region = max_retries, region

    def _aiobotocore_client(self, bucket: Bucket):
        from aiobotocore.session import get_session  # optional dependency

        from ..config import client_config

        return get_session().create_client(
            "s3", endpoint_url=f"https://{bucket.account_id}.r2.cloudflarestorage.com", region_name=self.region,
            config=client_config.to_botocore(), aws_access_key_id=bucket.access_key_id,
            aws_secret_access_key=bucket.secret_access_key)

    async def _client(self, bucket: Bucket):
        key = (bucket.access_key_id, bucket.secret_access_key, bucket.account_id)
        async with self._lock:
            c = self._clients.get(key)
            if c is None:
                made = self._factory(bucket)
                if hasattr(made, "__aenter__"):
                    self._ctx[key] = made
                    made = await made.__aenter__()
                self._clients[key] = c = made
            return c

    async def purge(self, bucket: Bucket) -> None:
        """Drop a client after a connection-level failure so the next call reconnects."""
        key = (bucket.access_key_id, bucket.secret_access_key, bucket.account_id)
        async with self._lock:
            self._clients.pop(key, None)
            ctx = self._ctx.pop(key, None)
        if ctx is not None:
            try:
                await ctx.__aexit__(None, None, None)
            except Exception:  # noqa: BLE001
                pass

    async def close(self):
        for ctx in list(self._ctx.values()):
            try:
                await ctx.__aexit__(None, None, None)
            except Exception:  # noqa: BLE001
                pass
        self._clients.clear()
        self._ctx.clear()

    async def _guard(self, bucket, coro_fn):
        try:
            return await coro_fn(await self._client(bucket))
        except Exception as e:  # noqa: BLE001
            # a connection-level failure (or a server-side error) drops the cached client so that the next call
            # reconnects; "no such object" / "not allowed" answers come over a healthy connection and keep it
            # (the reference purges on those too, src/tplr/comms.py:549-552, and reconnects on every miss)
            code = getattr(e, "response", {}).get("Error", {}).get("Code") if hasattr(e, "response") else None
            benign = code in ("404", "403", "401", "NoSuchKey", "NotFound", "NoSuchUpload")
            if _is_named(e, "ConnectionClosedError", "EndpointConnectionError") or (_is_named(e, "ClientError") and not benign):
                await self.purge(bucket)
            raise

    # -- uploads ----------------------------------------------------------------------------
    async def put_bytes(self, bucket, key, data):
        await self._guard(bucket, lambda c: c.put_object(Bucket=bucket.name, Key=key, Body=data))

    async def put_file(self, bucket, key, path):
        size = os.path.getsize(path)
        if size < self.MULTIPART_THRESHOLD:
            data = await asyncio.to_thread(Path(path).read_bytes)
            return await self.put_bytes(bucket, key, data)
        await self.upload_large_file(bucket, key, path)

    async def upload_large_file(self, bucket, key, path) -> None:
        """Multipart upload: parts in parallel, per-part retries with exponential back-off, and a
        full restart (new upload id) if the store forgets the upload."""
        size = os.path.getsize(path)
        n_parts = max(1, -(-size // self.part_size))
        for attempt in range(self.max_retries):
            client = await self._client(bucket)
            up = await client.create_multipart_upload(Bucket=bucket.name, Key=key)
            upload_id = up["UploadId"]
            sem = asyncio.Semaphore(self.concurrency)
            restart = False

            async def send(part_no: int):
                nonlocal restart
                off = (part_no - 1) * self.part_size
                ln = min(self.part_size, size - off)

                def _read():
                    with open(path, "rb") as f:
                        f.seek(off)
                        return f.read(ln)

                async with sem:
                    body = await asyncio.to_thread(_read)
                    md5 = hashlib.md5(body).digest()
                    import base64

                    for t in range(self.max_retries):
                        try:
                            r = await client.upload_part(Bucket=bucket.name, Key=key, PartNumber=part_no,
                                                         UploadId=upload_id, Body=body,
                                                         ContentMD5=base64.b64encode(md5).decode())
                            return {"ETag": r["ETag"], "PartNumber": part_no}
                        except Exception as e:  # noqa: BLE001
                            if "NoSuchUpload" in str(e):
                                restart = True
                                raise
                            if t == self.max_retries - 1:
                                raise
                            await asyncio.sleep(min(2 ** t, 30))

            try:
                parts = await asyncio.gather(*(send(i) for i in range(1, n_parts + 1)))
                await client.complete_multipart_upload(
                    Bucket=bucket.name, Key=key, UploadId=upload_id,
                    MultipartUpload={"Parts": sorted(parts, key=lambda p: p["PartNumber"])})
                return
            except Exception as e:  # noqa: BLE001
                try:
                    await client.abort_multipart_upload(Bucket=bucket.name, Key=key, UploadId=upload_id)
                except Exception as abort_err:  # noqa: BLE001
                    logger.debug(f"abort of multipart upload {upload_id} failed: {abort_err}")
                if attempt == self.max_retries - 1 or not (restart or _is_named(e, "ClientError", "ConnectionClosedError")):
                    raise
                logger.warning(f"multipart upload of {key} restarting ({e})")
                await self.purge(bucket)
                await asyncio.sleep(min(2 ** attempt, 30))

    # -- downloads --------------------------------------------------------------------------
    async def head(self, bucket, key):
        try:
            h = await self._guard(bucket, lambda c: c.head_object(Bucket=bucket.name, Key=key))
        except Exception as e:  # noqa: BLE001
            code = getattr(e, "response", {}).get("Error", {}).get("Code") if hasattr(e, "response") else None
            if code in ("404", "403", "401", "NoSuchKey", "NotFound"):
                return None
            raise
        lm = h["LastModified"]
        if lm.tzinfo is None:
            lm = lm.replace(tzinfo=timezone.utc)
        return ObjectInfo(key, int(h.get("ContentLength", 0)), lm)

    async def get_bytes(self, bucket, key):
        async def _get(c):
            r = await c.get_object(Bucket=bucket.name, Key=key)
            async with r["Body"] as stream:
                return await stream.read()
        try:
            return await self._guard(bucket, _get)
        except Exception as e:  # noqa: BLE001
            code = getattr(e, "response", {}).get("Error", {}).get("Code") if hasattr(e, "response") else None
            if code in ("404", "NoSuchKey", "NotFound"):
                return None
            raise

    async def get_range(self, bucket, key, start, end):
        async def _get(c):
            r = await c.get_object(Bucket=bucket.name, Key=key, Range=f"bytes={start}-{end}")
            async with r["Body"] as stream:
                return await stream.read()
        if start < 0 or end < start:
            return None
        try:
            data = await self._guard(bucket, _get)
        except Exception as e:  # noqa: BLE001
            code = getattr(e, "response", {}).get("Error", {}).get("Code") if hasattr(e, "response") else None
            if code in ("404", "416", "NoSuchKey", "NotFound", "InvalidRange"):
                return None
            raise
        return data if len(data) == end - start + 1 else None

    async def get_to_file(self, bucket, key, path):
        info = await self.head(bucket, key)
        if info is None:
            return False
        if info.size >= self.RANGED_GET_THRESHOLD:
            return await self.download_large_file(bucket, key, info.size, path)
        data = await self.get_bytes(bucket, key)
        if data is None:
            return False
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        await asyncio.to_thread(Path(path).write_bytes, data)
        return True

    def download_plan(self, size: int, workers: int | None = None) -> tuple[int, int]:
        """(chunk_size, n_workers) for a ranged download (see :func:`download_params`); the worker count can be
        fixed with ``workers`` or the ``DOWNLOAD_MAX_WORKERS`` variable."""
        p = download_params(size, str(workers) if workers else os.getenv("DOWNLOAD_MAX_WORKERS"))
        return p["chunk_size"], p["max_workers"]

    async def download_large_file(self, bucket, key, size: int, path: str) -> bool:
        """Parallel ranged GETs written at their offsets; chunks finished by an earlier, interrupted
        attempt (recorded in ``<path>.progress``) are not fetched again."""
        chunk, workers = self.download_plan(size)
        n_chunks = -(-size // chunk)
        prog_path = Path(str(path) + ".progress")
        done: set[int] = set()
        if prog_path.exists() and Path(path).exists() and os.path.getsize(path) == size:
            done = {int(x) for x in prog_path.read_text().split() if x.strip().isdigit()}
        else:
            Path(path).parent.mkdir(parents=True, exist_ok=True)
            with open(path, "wb") as f:
                f.truncate(size)
            prog_path.write_text("")
        sem = asyncio.Semaphore(workers)
        client = await self._client(bucket)
        lock = asyncio.Lock()

        async def fetch(i: int):
            lo, hi = i * chunk, min(size, (i + 1) * chunk) - 1
            async with sem:
                for t in range(self.max_retries):
                    try:
                        r = await client.get_object(Bucket=bucket.name, Key=key, Range=f"bytes={lo}-{hi}")
                        async with r["Body"] as stream:
                            data = await stream.read()
                        if len(data) != hi - lo + 1:
                            raise IOError(f"chunk {i}: got {len(data)} bytes, wanted {hi - lo + 1}")

                        def _write():
                            with open(path, "r+b") as f:
                                f.seek(lo)
                                f.write(data)
                        await asyncio.to_thread(_write)
                        async with lock:
                            with open(prog_path, "a") as pf:
                                pf.write(f"{i}\n")
                        return True
                    except Exception as e:  # noqa: BLE001
                        if t == self.max_retries - 1:
                            logger.error(f"ranged GET {key} chunk {i} failed: {e}")
                            return False
                        await asyncio.sleep(min(2 ** t, 30))

        results = await asyncio.gather(*(fetch(i) for i in range(n_chunks) if i not in done))
        if all(results):
            prog_path.unlink(missing_ok=True)
            return True
        return False

    async def list(self, bucket, prefix=""):
        out, token = [], None
        while True:
            kw = {"Bucket": bucket.name, "Prefix": prefix}
            if token:
                kw["ContinuationToken"] = token
            r = await self._guard(bucket, lambda c: c.list_objects_v2(**kw))
            for o in r.get("Contents", []):
                lm = o.get("LastModified", datetime.now(timezone.utc))
                out.append(ObjectInfo(o["Key"], int(o.get("Size", 0)), lm))
            if r.get("IsTruncated"):
                token = r.get("NextContinuationToken")
            else:
                return out

    async def delete(self, bucket, keys):
        for i in range(0, len(keys), 1000):
            batch = [{"Key": k} for k in keys[i:i + 1000]]
            await self._guard(bucket, lambda c: c.delete_objects(Bucket=bucket.name, Delete={"Objects": batch}))
