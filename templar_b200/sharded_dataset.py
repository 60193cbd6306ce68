"""Pre-tokenised shard datasets (memory-mapped) and the manager that rotates them.

File layout and behaviour follow the reference (src/tplr/sharded_dataset.py:32-446):
``<prefix>_{idx:06d}.npy`` holds uint32 tokens, ``sample_ids_{idx:06d}.npy`` (``sample_ids_anneal_…``
for the anneal prefix) holds one uint64 id per sequence; item ``i`` is
``tokens[i*seq:(i+1)*seq]``; the manager has rank 0 fetch the current shard, prefetches the next
in the background, swaps (cyclically over 14 shards, shard 7 remapped to 13) and deletes the old
files; anneal mode pins one shard.  :class:`SyntheticDataset` provides the uniform-random token
stream used by benchmarks when no shard files exist.
"""

from __future__ import annotations

import asyncio
import os
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import Dataset

from .logging import logger
from .profilers import get_shard_profiler


def compute_shard_state(global_step: int, outer_steps_per_shard: int, reset_outer_step: int | None = None) -> tuple[int, int]:
    """(epoch, shard_index) for ``global_step``; the epoch becomes 1 and counting restarts at ``reset_outer_step``."""
    if outer_steps_per_shard <= 0:
        return 0, 0
    if reset_outer_step is None or reset_outer_step < 0 or global_step < reset_outer_step:
        return 0, global_step // outer_steps_per_shard
    return 1, max(global_step - reset_outer_step, 0) // outer_steps_per_shard


class SharedShardedDataset(Dataset):
    def __init__(self, shard_index: int, sequence_length: int, rank: int, world_size: int, *,
                 token_dtype=np.uint32, file_prefix: str = "train", custom_path=None):
        super().__init__()
        t0 = time.perf_counter()
        self.seqlen, self.rank, self.world = sequence_length, rank, world_size
        if self.world > 1 and dist.is_available() and dist.is_initialized():
            if torch.cuda.is_available() and dist.get_backend() == "nccl":
                dist.barrier(device_ids=[torch.cuda.current_device()])
            else:
                dist.barrier()
        self.tokens_file, self.ids_file = self.locate_shards(shard_index, custom_path, file_prefix)
        self.check_paths([self.tokens_file, self.ids_file])
        prof = get_shard_profiler()                       # a no-op stand-in unless the profilers are switched on
        tid = prof.start_read(self.tokens_file, {"shard": shard_index, "rank": rank, "what": "open"})
        self.mmap_tokens_and_ids(token_dtype)
        prof.log_shard_metadata(self.tokens_file, os.path.getsize(self.tokens_file), 1, self.total_samples)
        prof.end_read(tid, self.tokens_file)
        logger.info(f"[Dataset] rank {rank}: shard {shard_index} ready in {time.perf_counter() - t0:.1f}s "
                    f"({self.total_samples} samples)")

    @staticmethod
    def locate_shards(shard_index: int, custom_path=None, file_prefix: str = "train"):
        root = custom_path or os.getenv("DATASET_BINS_PATH")
        if root is None:
            raise ValueError("Dataset path not configured. Set $DATASET_BINS_PATH or provide custom_path")
        tokens = os.path.join(root, f"{file_prefix}_{shard_index:06d}.npy")
        ids_name = (f"sample_ids_{file_prefix}_{shard_index:06d}.npy" if file_prefix == "anneal"
                    else f"sample_ids_{shard_index:06d}.npy")
        return tokens, os.path.join(root, ids_name)

    @staticmethod
    def check_paths(paths) -> None:
        for p in paths:
            if not os.path.exists(p):
                raise FileNotFoundError(f"Pre-processed file {os.path.basename(p)} not found in "
                                        f"{os.path.dirname(p)}. Run the preprocessing script first.")

    def mmap_tokens_and_ids(self, token_dtype) -> None:
        def _open(path, dtype):
            path = Path(path)
            if path.suffix == ".npy":
                arr = np.load(path, mmap_mode="r", allow_pickle=False)
                if arr.dtype != dtype:
                    arr = arr.astype(dtype, copy=False)
                return arr.reshape(-1)
            return np.memmap(path, dtype=np.dtype(dtype).newbyteorder("<"), mode="r")

        self._tokens_np = _open(self.tokens_file, np.uint32)
        self._ids_np = _open(self.ids_file, np.uint64)
        self.tokens = torch.from_numpy(self._tokens_np)
        self.sample_ids = self._ids_np
        total = int(self._tokens_np.shape[0])
        if total % self.seqlen != 0:
            raise ValueError(f"Token file length ({total}) not divisible by seqlen ({self.seqlen}). File: {self.tokens_file}")
        from_tokens = total // self.seqlen
        self.total_samples = min(from_tokens, int(self._ids_np.shape[0]))
        if from_tokens != int(self._ids_np.shape[0]):
            logger.warning(f"[Dataset] tokens hold {from_tokens} samples but {self._ids_np.shape[0]} sample ids "
                           f"({self.tokens_file}); using {self.total_samples}")

    def __len__(self):
        return self.total_samples

    def __getitem__(self, idx: int):
        if idx >= self.total_samples or idx < 0:
            raise IndexError(idx)
        return self.tokens[idx * self.seqlen: (idx + 1) * self.seqlen]

    def sample_id(self, idx: int) -> int:
        return int(self._ids_np[idx])


class SyntheticDataset(Dataset):
    """Uniform-random token ids, deterministic per index (no files): row ``i`` is drawn from a
    generator seeded with ``seed + i``.  Same interface as :class:`SharedShardedDataset`."""

    def __init__(self, n_samples: int, sequence_length: int, vocab_size: int, seed: int = 0):
        self.total_samples, self.seqlen, self.vocab, self.seed = n_samples, sequence_length, vocab_size, seed
        self.tokens_file = self.ids_file = None

    def __len__(self):
        return self.total_samples

    def __getitem__(self, idx: int):
        if idx >= self.total_samples or idx < 0:
            raise IndexError(idx)
        g = torch.Generator().manual_seed(self.seed + int(idx))
        return torch.randint(0, self.vocab, (self.seqlen,), generator=g, dtype=torch.int64)

    def sample_id(self, idx: int) -> int:
        return (self.seed * 0x9E3779B97F4A7C15 + int(idx)) & 0xFFFF_FFFF_FFFF_FFFF


class ShardedDatasetManager:
    def __init__(self, sequence_length: int, rank: int, world_size: int, comms, token_dtype=np.uint32,
                 file_prefix: str = "train", anneal_mode: bool = False):
        self.sequence_length, self.rank, self.world_size = sequence_length, rank, world_size
        self.token_dtype, self.file_prefix, self.anneal_mode = token_dtype, file_prefix, anneal_mode
        self.comms = comms
        self.shard_index = 0
        self.max_dataset_idx = 14
        self.active_dataset: SharedShardedDataset | None = None
        self.upcoming_dataset: asyncio.Task | None = None

    @staticmethod
    def remap_shard_index(shard_index: int) -> int:
        return 13 if shard_index == 7 else shard_index

    def prepare_shard(self, shard_index: int) -> asyncio.Task:
        tokens_file, ids_file = SharedShardedDataset.locate_shards(self.remap_shard_index(shard_index),
                                                                   file_prefix=self.file_prefix)
        if os.path.exists(tokens_file) and os.path.exists(ids_file):
            return asyncio.create_task(asyncio.sleep(0))
        bucket = self.comms.get_own_bucket("dataset", "read")
        return asyncio.create_task(self.download_files(bucket, tokens_file, ids_file))

    async def download_files(self, bucket, tokens_file, ids_file):
        prof = get_shard_profiler()
        tid = prof.start_read(tokens_file, {"what": "download"})
        try:
            return await self._download_files(bucket, tokens_file, ids_file)
        finally:
            prof.end_read(tid, tokens_file)

    async def _download_files(self, bucket, tokens_file, ids_file):
        return await asyncio.gather(self.comms.s3_get_object(tokens_file, bucket, load_data=False),
                                    self.comms.s3_get_object(ids_file, bucket, load_data=False))

    async def create_dataset(self, shard_index: int) -> SharedShardedDataset:
        if self.rank == 0:
            await self.prepare_shard(shard_index)
        return SharedShardedDataset(self.remap_shard_index(shard_index), self.sequence_length, self.rank,
                                    self.world_size, token_dtype=self.token_dtype, file_prefix=self.file_prefix)

    async def initialize_datasets(self, current_shard_index: int) -> None:
        self.shard_index = current_shard_index
        self.active_dataset = await self.create_dataset(current_shard_index)
        if self.anneal_mode or self.rank != 0:
            self.upcoming_dataset = asyncio.create_task(asyncio.sleep(0))
            return
        self.upcoming_dataset = self.prepare_shard((current_shard_index + 1) % self.max_dataset_idx)

    async def swap_datasets(self) -> int:
        if self.anneal_mode:
            return self.shard_index
        self.shard_index = (self.shard_index + 1) % self.max_dataset_idx
        if self.upcoming_dataset:
            await self.upcoming_dataset
        old = self.active_dataset
        await self.initialize_datasets(self.shard_index)
        if old is not None and self.rank == 0:
            for path in (old.tokens_file, old.ids_file):
                try:
                    os.remove(path)
                except (FileNotFoundError, TypeError):
                    logger.error(f"{path} not available for deletion")
        return self.shard_index
