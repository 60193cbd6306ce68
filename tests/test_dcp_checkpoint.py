"""DCP checkpointer in one process against the in-memory object store: save, upload, discovery by pointer
and by listing, download into another root, load, existence check, local clean-up."""

import asyncio
import json
from types import SimpleNamespace

import torch

import templar_b200 as tplr
from templar_b200.backends.chain import StaticChain, StaticWallet
from templar_b200.backends.store import MemoryStore
from templar_b200.models.llama import ModelArgs, build_model


def _comms(uid, store, chain):
    hp = SimpleNamespace(topk_compression=4, blocks_per_window=4, recent_windows=2, active_check_interval=1)
    c = tplr.Comms(wallet=StaticWallet(f"hotkey-{uid}"), config=SimpleNamespace(netuid=3, device="cpu"), hparams=hp, uid=uid,
                   store=store, subtensor=chain)
    c.try_commit(c.wallet, c.bucket)
    return c


def _model(seed):
    args = ModelArgs(dim=64, n_layers=1, n_heads=2, vocab_size=64, intermediate_size=128, max_seq_len=16)
    return build_model(args, seed=seed)


def test_save_upload_discover_download_load_roundtrip(tmp_path):
    store, chain = MemoryStore(), StaticChain(n=4, manual=True)
    writer, reader = _comms(0, store, chain), _comms(1, store, chain)

    async def go():
        for c in (writer, reader):
            c.commitments = await c.get_commitments()
        src = _model(1)
        ck = tplr.DCPCheckpointer(writer, uid=0, version="t1", repo_root=tmp_path / "w")
        for window, step in ((5, 2), (9, 4)):
            with torch.no_grad():
                for p in src.parameters():
                    p.add_(0.01 * window)
            await ck.save_local(model=src, window=window, sync_window=window - 1, global_step=step)
            await ck.upload(window=window, background=False, delete_local_on_success=False, initial_sleep_s=0.0,
                            pointer_poll_timeout_s=1.0, pointer_poll_interval_s=0.05)
        assert await ck.check_checkpoint_exists(window=9, prefer_highest_staked=False)
        assert not await ck.check_checkpoint_exists(window=7, prefer_highest_staked=False)
        side = json.loads((tmp_path / "w" / "checkpoints" / "t1" / "9" / "extra_metadata.json").read_text())
        assert side["window"] == 9 and side["sync_window"] == 8 and side["global_step"] == 4 and side["uid"] == 0

        # reader: another root, reads the writer's bucket; latest window found through the pointer file
        rk = tplr.DCPCheckpointer(reader, uid=1, version="t1", repo_root=tmp_path / "r")
        rk.comms = SimpleNamespace(**{**vars(reader), "bucket": writer.bucket, "store": store,
                                      "s3_get_object": writer.s3_get_object,
                                      "_get_highest_stake_validator_bucket": writer._get_highest_stake_validator_bucket})
        assert await rk._discover_latest(prefer_highest_staked=False) == 9
        dst = _model(2)
        got = await rk.download_and_load(model=dst, shared_fs=False, prefer_highest_staked=False)
        assert got == (8, 4)
        for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
            assert torch.equal(a.detach(), b.detach()), n

        # without the pointer the prefix listing gives the same answer; an explicit older window loads too
        await store.delete(writer.bucket, ["checkpoints/t1/_LATEST.json"])
        assert await rk._discover_latest(prefer_highest_staked=False) == 9
        old = _model(3)
        assert await rk.download_and_load(model=old, window=5, shared_fs=False, prefer_highest_staked=False) == (4, 2)
        assert not torch.equal(next(old.parameters()).detach(), next(src.parameters()).detach())
        assert await rk.download_and_load(model=old, window=77, shared_fs=False, prefer_highest_staked=False) is None

        base = tmp_path / "r" / "checkpoints" / "t1"
        assert not (base / "77").exists()                        # a missing window leaves no directory behind
        (base / "3").mkdir()                                     # empty left-over
        (base / "7").mkdir(); (base / "7" / "__0_0.distcp").write_bytes(b"x")      # stale partial save
        (base / "12").mkdir(); (base / "12" / "__0_0.distcp").write_bytes(b"x")    # newer, maybe still being written
        rk.cleanup_local_checkpoints(keep_latest=1)
        left = sorted(p.name for p in base.iterdir() if p.is_dir())
        assert left == ["12", "9"]

    asyncio.run(go())
