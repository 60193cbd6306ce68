"""Window-seeded samplers: which dataset rows a (uid, window) trains or is evaluated on.

Bit-exact with the reference (src/tplr/sharded_sampler.py:30-221): the seed is
``(uid * 1_000_003 ^ window) & 0xFFFFFFFF``, the miner pool is
``numpy.random.default_rng(seed).choice(N, steps_per_window * target_batch_size, replace=False)``,
a rank takes ``pool[rank::world]``, and the validator rebuilds the pool with
``steps_per_window * batch_size`` rows and draws ``validation_bs`` of them with a time-seeded
generator cached per (uid, window).
"""

from __future__ import annotations

import time

import numpy as np
from torch.utils.data import Sampler


def _window_seed(uid: int, window: int) -> int:
    return (uid * 1_000_003 ^ window) & 0xFFFF_FFFF


class _WindowSampler(Sampler):
    def __init__(self, dataset, uid: int, window: int, *, steps_per_window: int, micro_bs: int, batch_size: int,
                 rank: int = 0, world_size: int = 1):
        self._source = dataset
        self.dataset_len = len(dataset)
        self.steps_per_window, self.micro_bs, self.batch_size = steps_per_window, micro_bs, batch_size
        self.rank, self.world_size = rank, world_size
        self.grad_accum_steps = batch_size // (micro_bs * world_size)
        self.set_window_uid(uid, window)

    def set_window_uid(self, uid: int, window: int) -> None:
        self.uid, self.window = uid, window
        self._mine = self._global_indices()[self.rank:: self.world_size].tolist()

    def __iter__(self):
        return iter(self._mine)

    def __len__(self):
        return len(self._mine)

    def ids_for_indices(self, idx_list) -> list[int]:
        return [self._source.sample_id(i) for i in idx_list]

    def _global_indices(self) -> np.ndarray:  # pragma: no cover - abstract
        raise NotImplementedError


class MinerSampler(_WindowSampler):
    def __init__(self, dataset, uid, window, *, steps_per_window, micro_bs, batch_size, target_batch_size,
                 rank: int = 0, world_size: int = 1):
        self.target_batch_size = target_batch_size
        super().__init__(dataset, uid, window, steps_per_window=steps_per_window, micro_bs=micro_bs,
                         batch_size=batch_size, rank=rank, world_size=world_size)

    def _global_indices(self) -> np.ndarray:
        wanted = self.steps_per_window * self.target_batch_size
        if wanted > self.dataset_len:
            raise ValueError(f"a window draws {wanted} samples; the dataset holds {self.dataset_len}")
        rng = np.random.default_rng(_window_seed(self.uid, self.window))
        return rng.choice(self.dataset_len, size=wanted, replace=False)


class EvalSampler(_WindowSampler):
    _subset_cache: dict[tuple[int, int], np.ndarray] = {}
    _cached_indices = _subset_cache        # the same dict under the name callers of the reference clear between windows

    def __init__(self, dataset, uid, window, *, steps_per_window, micro_bs, batch_size, validation_bs,
                 rank: int = 0, world_size: int = 1):
        if validation_bs > batch_size:
            raise ValueError("the validation subset cannot be larger than the batch it is drawn from")
        self.validation_bs = validation_bs
        super().__init__(dataset, uid, window, steps_per_window=steps_per_window, micro_bs=micro_bs,
                         batch_size=batch_size, rank=rank, world_size=world_size)

    def _eval_seed(self) -> int:
        return (self.uid * 0x9E3779B1 ^ self.window ^ int(time.time_ns())) & 0xFFFF_FFFF

    def _global_indices(self) -> np.ndarray:
        key = (self.uid, self.window)
        hit = self._subset_cache.get(key)
        if hit is not None:
            return hit
        total = self.steps_per_window * self.batch_size
        if total > self.dataset_len:
            raise ValueError("the reconstructed training pool does not fit the dataset")
        pool = np.random.default_rng(_window_seed(self.uid, self.window)).choice(self.dataset_len, size=total, replace=False)
        val = np.random.default_rng(self._eval_seed()).choice(pool, size=self.validation_bs, replace=False)
        self._subset_cache[key] = val
        return val
