"""Samplers (bit-exact seeding, rank partition, eval subset), shard schedule and dataset files."""

import numpy as np
import pytest
import torch

import templar_b200 as tplr
from templar_b200.sharded_sampler import _window_seed


class _DS:
    def __init__(self, n): self.n = n
    def __len__(self): return self.n
    def sample_id(self, i): return 1000 + i


def test_window_seed_and_pool_are_numpy_exact():
    assert _window_seed(7, 12345) == (7 * 1_000_003 ^ 12345) & 0xFFFFFFFF
    s = tplr.MinerSampler(_DS(5000), 7, 12345, steps_per_window=3, micro_bs=2, batch_size=8, target_batch_size=16)
    want = np.random.default_rng(_window_seed(7, 12345)).choice(5000, size=48, replace=False)
    assert list(s) == want.tolist() and s.grad_accum_steps == 4


@pytest.mark.parametrize("world", [1, 2, 4])
def test_rank_partition_is_disjoint_and_complete(world):
    parts = [list(tplr.MinerSampler(_DS(4000), 3, 9, steps_per_window=2, micro_bs=1, batch_size=8, target_batch_size=32,
                                    rank=r, world_size=world)) for r in range(world)]
    flat = sorted(sum(parts, []))
    assert len(flat) == 64 and len(set(flat)) == 64
    full = list(tplr.MinerSampler(_DS(4000), 3, 9, steps_per_window=2, micro_bs=1, batch_size=8, target_batch_size=32))
    for r in range(world):
        assert parts[r] == full[r::world]


def test_too_small_dataset_raises():
    with pytest.raises(ValueError):
        tplr.MinerSampler(_DS(10), 1, 1, steps_per_window=2, micro_bs=1, batch_size=8, target_batch_size=32)
    with pytest.raises(ValueError):
        tplr.EvalSampler(_DS(100), 1, 1, steps_per_window=1, micro_bs=1, batch_size=4, validation_bs=8)


def test_eval_sampler_is_subset_of_training_pool_and_cached():
    tplr.EvalSampler._subset_cache.clear()
    ds = _DS(3000)
    ev = tplr.EvalSampler(ds, 5, 77, steps_per_window=2, micro_bs=1, batch_size=16, validation_bs=8)
    pool = set(np.random.default_rng(_window_seed(5, 77)).choice(3000, size=32, replace=False).tolist())
    got = list(ev)
    assert len(got) == 8 and len(set(got)) == 8 and set(got) <= pool
    ev2 = tplr.EvalSampler(ds, 5, 77, steps_per_window=2, micro_bs=1, batch_size=16, validation_bs=8)
    assert list(ev2) == got                      # cached per (uid, window)
    assert ev.ids_for_indices(got[:2]) == [1000 + got[0], 1000 + got[1]]


@pytest.mark.parametrize("step,per,reset,want", [(0, 10, None, (0, 0)), (25, 10, None, (0, 2)), (25, 10, 20, (1, 0)),
                                                  (45, 10, 20, (1, 2)), (5, 0, None, (0, 0)), (19, 10, 20, (0, 1))])
def test_compute_shard_state(step, per, reset, want):
    assert tplr.compute_shard_state(step, per, reset) == want


def test_shared_sharded_dataset_reads_npy_shards(tmp_path):
    seq = 16
    tokens = np.arange(10 * seq, dtype=np.uint32)
    np.save(tmp_path / "train_000003.npy", tokens)
    np.save(tmp_path / "sample_ids_000003.npy", np.arange(10, dtype=np.uint64) + 500)
    ds = tplr.SharedShardedDataset(3, seq, 0, 1, custom_path=str(tmp_path))
    assert len(ds) == 10 and ds.sample_id(4) == 504
    assert ds[2].tolist() == list(range(32, 48))
    with pytest.raises(IndexError):
        ds[10]
    with pytest.raises(FileNotFoundError):
        tplr.SharedShardedDataset(4, seq, 0, 1, custom_path=str(tmp_path))
    assert tplr.SharedShardedDataset.locate_shards(5, "/x", "anneal")[1].endswith("sample_ids_anneal_000005.npy")
    assert tplr.ShardedDatasetManager.remap_shard_index(7) == 13 and tplr.ShardedDatasetManager.remap_shard_index(6) == 6


def test_synthetic_dataset_is_deterministic():
    a, b = tplr.SyntheticDataset(50, 32, 1000, seed=1), tplr.SyntheticDataset(50, 32, 1000, seed=1)
    assert torch.equal(a[7], b[7]) and not torch.equal(a[7], a[8]) and int(a[7].max()) < 1000
