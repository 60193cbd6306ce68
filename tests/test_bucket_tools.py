"""Operator tools over the object-store interface (in-memory store)."""

import asyncio
import io

import torch

from templar_b200 import bucket_tools as bt
from templar_b200.backends.store import MemoryStore
from templar_b200.schemas import Bucket

B = Bucket(name="b", account_id="a", access_key_id="k", secret_access_key="s")


def _blob(obj):
    buf = io.BytesIO()
    torch.save(obj, buf)
    return buf.getvalue()


def test_classify_names():
    assert bt.classify("gradient-12-3-v2.1.28.pt") == ("gradient", 12, "2.1.28")
    assert bt.classify("aggregator-7-v2.1.28.pt") == ("aggregator", 7, "2.1.28")
    assert bt.classify("debug-5-0-v2.1.27.pt") == ("debug", 5, "2.1.27")
    assert bt.classify("peers_40_v2.1.28.json")[0] == "peers"
    assert bt.classify("checkpoints/2.1.28/30/__0_0.distcp") == ("checkpoint", 30, "2.1.28")
    assert bt.classify("notes.txt") == ("other", None, None)


def test_validate_summary_cleanup_and_versions():
    async def go():
        st = MemoryStore()
        assert await bt.validate(st, B) == {"put": True, "head": True, "get": True, "delete": True}
        for w in range(1, 6):
            await st.put_bytes(B, f"gradient-{w}-3-v2.1.28.pt", _blob({"state_dict": {"a.vals": torch.zeros(4), "a.idxs": torch.zeros(6, dtype=torch.uint8),
                                                                                      "a.quant_params": None, "metadata": {"window": w}},
                                                                       "global_step": w}))
            await st.put_bytes(B, f"debug-{w}-3-v2.1.28.pt", b"x")
        await st.put_bytes(B, "gradient-1-3-v2.1.20.pt", b"old")
        await st.put_bytes(B, "checkpoints/2.1.28/4/.metadata", b"m")
        s = await bt.summary(st, B)
        assert s["gradient@2.1.28"]["objects"] == 5 and s["gradient@2.1.20"]["objects"] == 1 and s["checkpoint@2.1.28"]["objects"] == 1
        would = await bt.cleanup(st, B, keep_windows=2, dry_run=True)
        assert len(would) == 7 and len(await st.list(B, "")) == 12          # nothing deleted on a dry run
        gone = await bt.cleanup(st, B, keep_windows=2)
        assert sorted(gone) == sorted(would)
        left = [o.key for o in await st.list(B, "")]
        assert "gradient-5-3-v2.1.28.pt" in left and "gradient-4-3-v2.1.28.pt" in left and "gradient-3-3-v2.1.28.pt" not in left
        assert "checkpoints/2.1.28/4/.metadata" in left                        # checkpoints are not window litter
        await st.put_bytes(B, "gradient-9-3-v2.1.20.pt", b"old")
        assert await bt.clean_versions(st, B, keep="2.1.28") == ["gradient-9-3-v2.1.20.pt"]
        obj = await bt.get_gradient(st, B, 3, 5, "2.1.28")
        d = bt.describe_gradient(obj)
        assert d["global_step"] == 5 and d["tensors"] == 1 and d["values"] == 4 and d["index_bytes"] == 6 and not d["quantised"]
        assert await bt.get_gradient(st, B, 3, 99, "2.1.28") is None
    asyncio.run(go())


def test_delete_by_selector_version_and_gather_results(tmp_path, monkeypatch):
    import os
    import time

    import pytest

    from templar_b200.backends.store import LocalFSStore

    async def go():
        st = LocalFSStore(tmp_path)
        names = ["gradient-1-3-v2.1.20.pt", "gradient-2-3-v2.1.28.pt", "debug-2-3-v2.1.28.pt", "peers_4_v2.1.20.json",
                 "checkpoints/2.1.20/4/.metadata", "gathers/2.1.20/3.pt", "gathers/2.1.28/9.pt", "notes.txt"]
        for n in names:
            await st.put_bytes(B, n, b"x")
        with pytest.raises(ValueError):
            await bt.delete_selected(st, B)                                   # no selector: refuses
        assert await bt.delete_gather(st, B, "2.1.28", dry_run=True) == ["gathers/2.1.28/9.pt"]
        assert sorted(await bt.delete_version(st, B, "2.1.20")) == sorted(n for n in names if "2.1.20" in n)
        left = sorted(o.key for o in await st.list(B, ""))
        assert left == sorted(["gradient-2-3-v2.1.28.pt", "debug-2-3-v2.1.28.pt", "gathers/2.1.28/9.pt", "notes.txt"])
        assert sorted(await bt.delete_selected(st, B, prefix="g", suffix=".pt", dry_run=True)) == ["gathers/2.1.28/9.pt", "gradient-2-3-v2.1.28.pt"]
        # age: only the object that was last written two hours ago
        old = st._path(B, "notes.txt")
        os.utime(old, (time.time() - 7200, time.time() - 7200))
        assert await bt.delete_selected(st, B, older_than_hours=1.0) == ["notes.txt"]
        assert len(await bt.delete_selected(st, B, everything=True)) == 3 and await st.list(B, "") == []
    asyncio.run(go())

    # the command line on the offline store of the environment
    monkeypatch.setenv("TPLR_STORE", "local")
    monkeypatch.setenv("TPLR_STORE_ROOT", str(tmp_path / "cli"))
    from templar_b200.backends.chain import StaticWallet
    from templar_b200.comms import Comms
    c = Comms(wallet=StaticWallet("hotkey-0"), uid=0)
    asyncio.run(c.store.put_bytes(c.bucket, "gathers/9.9.9/1.pt", b"x"))
    bt.main(["delete-gather", "--version", "9.9.9", "--dry-run"])
    assert asyncio.run(c.store.head(c.bucket, "gathers/9.9.9/1.pt")) is not None
    bt.main(["delete-gather", "--version", "9.9.9"])
    assert asyncio.run(c.store.head(c.bucket, "gathers/9.9.9/1.pt")) is None
