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


def test_checkpoint_fallback_ladder_current_version_bootstrap_version_nothing(tmp_path, monkeypatch):
    """`load_checkpoint_with_fallback` (reference tests/test_checkpoint_fallback.py): the current version's newest
    checkpoint wins; without one the configured bootstrap version is read (its newest window, or the window the
    hparams pin); a sidecar without a global step gets ``window - start_window`` of the version it came from; with
    nothing to load the model is left alone and the call says so."""
    monkeypatch.chdir(tmp_path)
    store, chain = MemoryStore(), StaticChain(n=4, manual=True)
    val, node = _comms(0, store, chain), _comms(2, store, chain)          # uid 0 has the highest stake

    async def save(version, window, step, delta):
        m = _model(1)
        with torch.no_grad():
            for p in m.parameters():
                p.add_(delta)
        ck = tplr.DCPCheckpointer(val, uid=0, version=version, repo_root=tmp_path / "val")
        await ck.save_local(model=m, window=window, sync_window=window, global_step=step)
        await ck.upload(window=window, background=False, delete_local_on_success=True, initial_sleep_s=0.0,
                        pointer_poll_timeout_s=1.0, pointer_poll_interval_s=0.05)
        return m

    def instance(version, bootstrap=None, pinned=None):
        hp = SimpleNamespace(checkpoint_init_window=pinned)
        return SimpleNamespace(model=_model(7), comms=node, uid=2, hparams=hp, start_window=10, bootstrap_version=bootstrap,
                               ckpt=tplr.DCPCheckpointer(node, uid=2, version=version, repo_root=tmp_path / "node"),
                               model_initialized=False, global_step=0)

    def same(a, b):
        return all(torch.equal(x.detach(), y.detach()) for x, y in zip(a.parameters(), b.parameters()))

    async def go():
        for c in (val, node):
            c.commitments = await c.get_commitments()
        # nothing anywhere
        inst = instance("cur", bootstrap="boot")
        untouched = _model(7)
        assert await tplr.neurons.load_checkpoint_with_fallback(inst) == (False, 0, 0, False)
        assert same(inst.model, untouched) and not inst.model_initialized
        # only the bootstrap version has checkpoints: newest one, flagged as bootstrap
        await save("boot", 20, 5, 0.25)
        b30 = await save("boot", 30, 9, 0.5)
        inst = instance("cur", bootstrap="boot")
        assert await tplr.neurons.load_checkpoint_with_fallback(inst) == (True, 30, 9, True)
        assert same(inst.model, b30) and inst.model_initialized and inst.global_step == 9
        # the hparams pin an older bootstrap window
        inst = instance("cur", bootstrap="boot", pinned=20)
        assert await tplr.neurons.load_checkpoint_with_fallback(inst) == (True, 20, 5, True)
        # a pinned window that does not exist, and no bootstrap version at all: nothing is loaded
        inst = instance("cur", bootstrap="boot", pinned=25)
        assert (await tplr.neurons.load_checkpoint_with_fallback(inst))[0] is False
        inst = instance("cur", bootstrap=None)
        assert (await tplr.neurons.load_checkpoint_with_fallback(inst))[0] is False
        # the current version gets a checkpoint: it wins over the bootstrap version
        c40 = await save("cur", 40, 12, 1.0)
        inst = instance("cur", bootstrap="boot")
        assert await tplr.neurons.load_checkpoint_with_fallback(inst) == (True, 40, 12, False)
        assert same(inst.model, c40)
        # a sidecar without a global step: derived from the start window of the version the checkpoint belongs to
        real = tplr.DCPCheckpointer.download_and_load

        async def no_step(self, **kw):
            res = await real(self, **kw)
            return None if res is None else (res[0], -1)
        monkeypatch.setattr(tplr.DCPCheckpointer, "download_and_load", no_step)
        inst = instance("cur", bootstrap="boot")
        assert await tplr.neurons.load_checkpoint_with_fallback(inst) == (True, 40, 30, False)        # 40 - start_window 10
        await val.post_start_window(17)
        boot_sw = await node.get_start_window(retries=1, retry_delay=0.01)

        async def start_of(version=None, **kw):
            return boot_sw if version == "boot" else None
        monkeypatch.setattr(node, "get_start_window", start_of)
        inst = instance("other", bootstrap="boot")
        assert await tplr.neurons.load_checkpoint_with_fallback(inst) == (True, 30, 13, True)         # 30 - 17
    asyncio.run(go())
