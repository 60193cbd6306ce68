"""Build the on-disk shards that :class:`templar_b200.sharded_dataset.SharedShardedDataset` reads.

Three steps, each a function and a sub-command of ``python -m templar_b200.dataset_prep``:

* ``pretokenize``  documents (``.jsonl`` with a ``text`` field, or plain ``.txt`` with one document per
  line) -> ``<prefix>_{i:06d}.npy`` shards of exactly ``shard_size`` uint32 tokens, every document
  followed by the tokenizer's EOS, documents split across shard ends (the layout written by the
  reference's scripts/dataset_prep/01_pretokenize_data.py:65-92, :181-240);
* ``ids``          one uint64 per ``seq_len`` slice of a shard: the first 8 bytes (little endian) of the
  BLAKE2b digest of the slice's bytes, saved as ``sample_ids_{i:06d}.npy``
  (scripts/dataset_prep/02_consolidate_shards.py:18-31);
* ``synthetic``    a small shard of seeded random tokens with its ids, for smoke tests and air-gapped
  boxes (the role of scripts/dataset_prep/single_testing_shard.py).

* ``upload`` / ``download``  shards and their ids between a directory and the dataset bucket, under the key that
  the nodes ask for (``$DATASET_BINS_PATH/<file name>``; scripts/download_dataset.py, and the upload half of
  scripts/dataset_prep/02_consolidate_shards.py);
* ``scan``         per shard: tokens, sequences, dtype, whether the ids file matches (scripts/shard_scanner.py
  counts rows of the raw dataset the same way, from metadata only: the token file is memory-mapped).
"""

from __future__ import annotations

import argparse
import glob
import hashlib
import json
import os
import struct
from concurrent.futures import ThreadPoolExecutor
from typing import Iterable, Iterator

import numpy as np


def sample_id(tokens: np.ndarray) -> int:
    """The 64-bit id of one sequence: BLAKE2b-8 of its bytes, little endian."""
    return struct.unpack("<Q", hashlib.blake2b(np.ascontiguousarray(tokens).tobytes(), digest_size=8).digest())[0]


def sample_ids(tokens: np.ndarray, seq_len: int, workers: int = 8) -> np.ndarray:
    """ids of all whole ``seq_len`` slices of ``tokens`` (a trailing partial slice is dropped).  hashlib
    releases the GIL on buffers above 2 KiB, so a thread pool scales on multi-core hosts."""
    n = tokens.shape[0] // seq_len
    body = np.ascontiguousarray(tokens[: n * seq_len]).reshape(n, seq_len)
    out = np.empty(n, dtype=np.uint64)

    def run(lo: int, hi: int) -> None:
        for i in range(lo, hi):
            out[i] = sample_id(body[i])

    step = max(1, -(-n // max(workers, 1)))
    with ThreadPoolExecutor(max_workers=max(workers, 1)) as ex:
        list(ex.map(lambda lo: run(lo, min(n, lo + step)), range(0, n, step)))
    return out


def shard_names(index: int, prefix: str = "train") -> tuple[str, str]:
    ids = f"sample_ids_{prefix}_{index:06d}.npy" if prefix == "anneal" else f"sample_ids_{index:06d}.npy"
    return f"{prefix}_{index:06d}.npy", ids


def write_sample_ids(directory: str, index: int, seq_len: int, prefix: str = "train", workers: int = 8) -> str:
    tok_name, ids_name = shard_names(index, prefix)
    tokens = np.load(os.path.join(directory, tok_name), mmap_mode="r", allow_pickle=False)
    path = os.path.join(directory, ids_name)
    np.save(path, sample_ids(tokens, seq_len, workers))
    return path


def iter_documents(paths: Iterable[str], text_field: str = "text") -> Iterator[str]:
    for path in paths:
        with open(path, encoding="utf-8") as f:
            if path.endswith(".jsonl"):
                for line in f:
                    if line.strip():
                        yield json.loads(line)[text_field]
            else:
                for line in f:
                    if line.strip():
                        yield line.rstrip("\n")


class ShardWriter:
    """Fills fixed-size uint32 shards from a stream of token arrays; documents may straddle two shards."""

    def __init__(self, directory: str, shard_size: int, start_shard: int = 0, end_shard: int | None = None,
                 prefix: str = "train"):
        os.makedirs(directory, exist_ok=True)
        self.directory, self.shard_size, self.prefix = directory, int(shard_size), prefix
        self.index, self.end = start_shard, end_shard
        self.buf = np.empty(self.shard_size, dtype=np.uint32)
        self.fill = 0
        self.written: list[str] = []

    @property
    def done(self) -> bool:
        return self.end is not None and self.index >= self.end

    def add(self, tokens) -> None:
        t = np.asarray(tokens, dtype=np.uint32).reshape(-1)
        while t.size and not self.done:
            n = min(t.size, self.shard_size - self.fill)
            self.buf[self.fill: self.fill + n] = t[:n]
            self.fill += n
            t = t[n:]
            if self.fill == self.shard_size:
                self._flush()

    def _flush(self) -> None:
        path = os.path.join(self.directory, shard_names(self.index, self.prefix)[0])
        tmp = path + ".tmp.npy"
        np.save(tmp, self.buf[: self.fill])
        os.replace(tmp, path)
        self.written.append(path)
        self.index += 1
        self.fill = 0

    def close(self, keep_partial: bool = False) -> list[str]:
        """A partly filled last shard is dropped (shards have one fixed size) unless ``keep_partial``."""
        if keep_partial and self.fill and not self.done:
            self._flush()
        return self.written


def pretokenize(documents: Iterable[str], tokenizer, directory: str, shard_size: int, start_shard: int = 0,
                end_shard: int | None = None, prefix: str = "train", keep_partial: bool = False,
                seq_len: int | None = None) -> list[str]:
    """Tokenise ``documents`` into shards; with ``seq_len`` the sample ids are written beside each shard."""
    w = ShardWriter(directory, shard_size, start_shard, end_shard, prefix)
    eos = tokenizer.eos_token_id
    for doc in documents:
        if w.done:
            break
        ids = list(tokenizer.encode(doc))
        ids.append(eos)
        w.add(ids)
    paths = w.close(keep_partial)
    if seq_len:
        for i in range(start_shard, start_shard + len(paths)):
            write_sample_ids(directory, i, seq_len, prefix)
    return paths


def synthetic_shard(directory: str, index: int, n_tokens: int, seq_len: int, vocab_size: int, seed: int = 0,
                    prefix: str = "train") -> tuple[str, str]:
    os.makedirs(directory, exist_ok=True)
    rng = np.random.default_rng(seed + index)
    tokens = rng.integers(0, vocab_size, size=n_tokens, dtype=np.uint32)
    tok_name, _ = shard_names(index, prefix)
    np.save(os.path.join(directory, tok_name), tokens)
    return os.path.join(directory, tok_name), write_sample_ids(directory, index, seq_len, prefix)


def shard_key(index: int, prefix: str, which: int, key_root: str | None = None) -> str:
    """Object key of a shard's token file (``which`` 0) or ids file (1): the path that the nodes build from
    ``DATASET_BINS_PATH``, which is also where they keep the file on disk."""
    root = key_root if key_root is not None else os.getenv("DATASET_BINS_PATH", "")
    return os.path.join(root, shard_names(index, prefix)[which])


async def upload_shards(comms, directory: str, indices: Iterable[int], prefix: str = "train", key_root: str | None = None,
                        seq_len: int | None = None) -> list[str]:
    """Put the token and ids files of ``indices`` into the dataset bucket (ids are computed first when ``seq_len``
    is given and the file is missing).  Returns the keys written."""
    bucket = comms.get_own_bucket("dataset", "write")
    out = []
    for i in indices:
        names = shard_names(i, prefix)
        if seq_len and not os.path.exists(os.path.join(directory, names[1])):
            write_sample_ids(directory, i, seq_len, prefix)
        for which in (0, 1):
            key = shard_key(i, prefix, which, key_root)
            await comms.s3_put_object(key, os.path.join(directory, names[which]), bucket)
            out.append(key)
    return out


async def download_shards(comms, directory: str, indices: Iterable[int], prefix: str = "train", key_root: str | None = None,
                          overwrite: bool = False) -> dict[int, bool]:
    """Fetch the token and ids files of ``indices`` from the dataset bucket into ``directory`` (files that are there
    already are kept).  Returns ``{index: complete}``."""
    bucket = comms.get_own_bucket("dataset", "read")
    os.makedirs(directory, exist_ok=True)
    done = {}
    for i in indices:
        ok = True
        for which, name in enumerate(shard_names(i, prefix)):
            dest = os.path.join(directory, name)
            if os.path.exists(dest) and not overwrite:
                continue
            part = dest + ".part"
            got = await comms.store.get_to_file(bucket, shard_key(i, prefix, which, key_root), part)
            if got:
                os.replace(part, dest)
            elif os.path.exists(part) and not os.path.exists(part + ".progress"):
                os.remove(part)                           # nothing worth resuming
            ok = ok and bool(got)
        done[i] = ok
    return done


def scan_shards(directory: str, prefix: str = "train", seq_len: int = 2048) -> list[dict]:
    """One record per ``<prefix>_*.npy`` shard in ``directory``: size, dtype, sequences, and whether the ids file
    exists with one id per complete sequence.  Reads headers only (memory map)."""
    out = []
    for f in sorted(glob.glob(os.path.join(directory, f"{prefix}_*.npy"))):
        stem = os.path.basename(f)[len(prefix) + 1: -4]
        if not stem.isdigit():
            continue
        tok = np.load(f, mmap_mode="r", allow_pickle=False)
        ids_path = os.path.join(directory, shard_names(int(stem), prefix)[1])
        n_ids = int(np.load(ids_path, mmap_mode="r", allow_pickle=False).shape[0]) if os.path.exists(ids_path) else None
        out.append({"shard": int(stem), "file": f, "tokens": int(tok.shape[0]), "dtype": str(tok.dtype),
                    "bytes": os.path.getsize(f), "sequences": int(tok.shape[0]) // seq_len,
                    "leftover_tokens": int(tok.shape[0]) % seq_len, "ids": n_ids,
                    "ids_ok": n_ids is not None and n_ids == int(tok.shape[0]) // seq_len})
    return out


def _dataset_comms(uid: int = 0):
    from .backends.chain import StaticWallet
    from .comms import Comms

    return Comms(wallet=StaticWallet(f"hotkey-{uid}"), uid=uid)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pretokenize")
    p.add_argument("--input", nargs="+", required=True, help="files or glob patterns (.jsonl / .txt)")
    p.add_argument("--tokenizer", required=True, help="name or local path for transformers.AutoTokenizer")
    p.add_argument("--output-dir", required=True)
    p.add_argument("--shard-size", type=int, default=1024 ** 3 // 4 * 4)
    p.add_argument("--start-shard", type=int, default=0)
    p.add_argument("--end-shard", type=int, default=None)
    p.add_argument("--prefix", default="train")
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--text-field", default="text")
    p.add_argument("--keep-partial", action="store_true")
    p = sub.add_parser("ids")
    p.add_argument("--dir", required=True)
    p.add_argument("--shards", type=int, nargs="*", default=None, help="indices (default: every shard found)")
    p.add_argument("--prefix", default="train")
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--workers", type=int, default=8)
    p = sub.add_parser("synthetic")
    p.add_argument("--dir", required=True)
    p.add_argument("--shards", type=int, default=1)
    p.add_argument("--tokens", type=int, default=2048 * 512)
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--vocab-size", type=int, default=128256)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--prefix", default="train")
    for name in ("upload", "download"):
        p = sub.add_parser(name)
        p.add_argument("shards", type=int, nargs="*", default=[0, 1], help="shard indices (default: 0 and 1)")
        p.add_argument("--path", "-p", default=os.getenv("DATASET_BINS_PATH", "."), help="local directory")
        p.add_argument("--prefix", default="train")
        p.add_argument("--key-root", default=None, help="directory part of the object keys (default: $DATASET_BINS_PATH)")
        if name == "upload":
            p.add_argument("--seq-len", type=int, default=None, help="compute missing ids files with this sequence length")
        else:
            p.add_argument("--overwrite", action="store_true")
    p = sub.add_parser("scan")
    p.add_argument("--dir", default=os.getenv("DATASET_BINS_PATH", "."))
    p.add_argument("--prefix", default="train")
    p.add_argument("--seq-len", type=int, default=2048)
    a = ap.parse_args(argv)
    if a.cmd in ("upload", "download"):
        import asyncio

        comms = _dataset_comms()
        if a.cmd == "upload":
            keys = asyncio.run(upload_shards(comms, a.path, a.shards, a.prefix, a.key_root, a.seq_len))
            print(f"uploaded {len(keys)} objects")
        else:
            done = asyncio.run(download_shards(comms, a.path, a.shards, a.prefix, a.key_root, a.overwrite))
            print(json.dumps({str(k): v for k, v in done.items()}))
            return 0 if all(done.values()) else 1
    elif a.cmd == "scan":
        for rec in scan_shards(a.dir, a.prefix, a.seq_len):
            print(json.dumps(rec))
    elif a.cmd == "pretokenize":
        from transformers import AutoTokenizer

        files = sorted(f for pat in a.input for f in (glob.glob(pat) or [pat]))
        tok = AutoTokenizer.from_pretrained(a.tokenizer)
        out = pretokenize(iter_documents(files, a.text_field), tok, a.output_dir, a.shard_size, a.start_shard,
                          a.end_shard, a.prefix, a.keep_partial, a.seq_len)
        print(f"wrote {len(out)} shard(s) to {a.output_dir}")
    elif a.cmd == "ids":
        idx = a.shards
        if idx is None:
            found = sorted(glob.glob(os.path.join(a.dir, f"{a.prefix}_*.npy")))
            idx = [int(os.path.basename(f)[len(a.prefix) + 1: -4]) for f in found]
        for i in idx:
            print(write_sample_ids(a.dir, i, a.seq_len, a.prefix, a.workers))
    else:
        for i in range(a.shards):
            print(*synthetic_shard(a.dir, i, a.tokens, a.seq_len, a.vocab_size, a.seed, a.prefix))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
