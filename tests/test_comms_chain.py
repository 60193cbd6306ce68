"""Comms over the in-memory / local stores, chain commitments, decorators, config and schemas.
Failures are injected on the host (dropped, late, corrupt and malformed objects)."""

import asyncio
import os
from datetime import datetime, timedelta, timezone
from types import SimpleNamespace

import pytest
import torch

import templar_b200 as tplr
from templar_b200 import chain as chain_mod
from templar_b200 import compress as C
from templar_b200.backends.chain import StaticChain, StaticWallet
from templar_b200.backends.store import LocalFSStore, MemoryStore, S3Store
from templar_b200.schemas import Bucket


def run(coro):
    return asyncio.run(coro)


def make_comms(uid, store, chain, topk=4):
    hp = SimpleNamespace(topk_compression=topk, blocks_per_window=4, recent_windows=2, active_check_interval=1)
    c = tplr.Comms(wallet=StaticWallet(f"hotkey-{uid}"), config=SimpleNamespace(netuid=3, device="cpu"), hparams=hp, uid=uid,
                   store=store, subtensor=chain)
    c.try_commit(c.wallet, c.bucket)
    return c


def payload(seed=0, k=4, shape=(2, 2, 64, 64), bad=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    idx, val, xshape, totalk = C.TopKCompressor().compress(x, k)
    if bad == "nan":
        val = val.clone(); val[0, 0, 0] = float("nan")
    if bad == "index":
        idx = C.pack_12bit_indices(torch.full(val.shape, 4095, dtype=torch.int64))
    return {"w.idxs": idx, "w.vals": val, "w.quant_params": None}


@pytest.fixture()
def net():
    store, chain = MemoryStore(), StaticChain(n=6, manual=True)
    comms = {u: make_comms(u, store, chain) for u in range(4)}

    async def sync():
        for c in comms.values():
            c.commitments = await c.get_commitments()
    run(sync())
    return store, chain, comms


def test_commitment_roundtrip_and_validation():
    b = Bucket(name="x" * 32, account_id="a" * 32, access_key_id="k" * 32, secret_access_key="s" * 64)
    s = chain_mod.encode_commitment(b)
    assert len(s) == 128
    d = chain_mod.decode_commitment(s)
    assert d.name == d.account_id == "a" * 32 and d.access_key_id == "k" * 32
    with pytest.raises(ValueError):
        chain_mod.decode_commitment("short")
    with pytest.raises(ValueError):
        chain_mod.encode_commitment(Bucket(name="n", account_id="a", access_key_id="k", secret_access_key="s"))
    assert hash(b) == hash(Bucket(**b.model_dump())) and b == Bucket(**b.model_dump())


def test_put_get_remote_and_local(net, tmp_path):
    store, chain, comms = net

    async def go():
        await comms[1].put(payload(1), window=5, key="gradient", uid="1", global_step=9, local=False)
        r = await comms[2].get(uid="1", window=5, key="gradient", local=False)
        assert r.success and r.global_step == 9 and torch.equal(r.data["w.vals"], payload(1)["w.vals"])
        assert (await comms[2].get(uid="1", window=6, key="gradient", local=False)).status == "NOT_FOUND"
        assert (await comms[2].get(uid="5", window=5, key="gradient", local=False)).status == "NOT_FOUND"
        await comms[1].put(payload(2), window=5, key="gradient", uid="1", local=True)
        r = await comms[1].get(uid="1", window=5, key="gradient", local=True)
        assert r.success
    run(go())


def test_time_window_too_early_too_late(net):
    store, chain, comms = net

    async def go():
        await comms[1].put(payload(1), window=3, key="gradient", uid="1", local=False)
        now = datetime.now(timezone.utc)
        r = await comms[2].get(uid="1", window=3, key="gradient", local=False, time_min=now + timedelta(seconds=60))
        assert r.status == "TOO_EARLY"
        r = await comms[2].get(uid="1", window=3, key="gradient", local=False, time_max=now - timedelta(seconds=60))
        assert r.status == "TOO_LATE"
        naive = (now - timedelta(seconds=60)).replace(tzinfo=None)
        r = await comms[2].get(uid="1", window=3, key="gradient", local=False, time_min=naive, time_max=now + timedelta(seconds=60))
        assert r.success
        assert await comms[2].get_with_retry(uid="1", window=3, key="gradient", timeout=5, local=False,
                                             time_max=now - timedelta(seconds=60)) is None
    run(go())


def test_gather_validates_and_reserve_fills_in(net):
    store, chain, comms = net
    totalks, xshapes = {"w.": 4096}, {"w.": (2, 2, 64, 64)}

    async def go():
        await comms[0].put(payload(0), window=7, key="gradient", uid="0", local=False)
        await comms[1].put(payload(1, bad="nan"), window=7, key="gradient", uid="1", local=False)
        await comms[2].put(payload(2, bad="index") | {"w.idxs": C.pack_12bit_indices(torch.full((2, 2, 4), 4095))},
                           window=7, key="gradient", uid="2", local=False)
        await comms[3].put(payload(3), window=7, key="gradient", uid="3", local=False)
        res = await comms[0].gather(my_uid=0, uids=[0, 1, 2], window=7, key="gradient", timeout=2, device="cpu",
                                    totalks={"w.": 4000}, local=False, xshapes=xshapes,
                                    expected_compressed_params={"w.idxs", "w.vals", "w.quant_params"})
        assert res.uids == [0] and sorted(res.skipped_uids) == [1, 2]      # NaN values, index >= totalk
        res = await comms[0].gather_with_reserve(my_uid=0, gather_uids=[0, 1], reserve_uids=[3], window=7, key="gradient",
                                                 timeout=2, device="cpu", totalks=totalks, local=False, xshapes=xshapes)
        assert res.uids == [0, 3] and res.success_rate == 1.0 and len(res.state_dict.__dict__["w.vals"]) == 2
        # sharded payload (wrong chunk grid) is rejected
        await comms[1].put(payload(5, shape=(1, 2, 64, 64)), window=8, key="gradient", uid="1", local=False)
        res = await comms[0].gather(my_uid=0, uids=[1], window=8, key="gradient", timeout=1, device="cpu", totalks=totalks,
                                    local=False, xshapes=xshapes)
        assert res is None
        # missing expected key
        await comms[1].put({"w.idxs": payload(1)["w.idxs"], "w.vals": payload(1)["w.vals"]}, window=9, key="gradient", uid="1", local=False)
        res = await comms[0].gather(my_uid=0, uids=[1], window=9, key="gradient", timeout=1, device="cpu", totalks=totalks,
                                    local=False, expected_compressed_params={"w.idxs", "w.vals", "w.quant_params"})
        assert res is None
    run(go())


def test_host_side_fault_injection_drop_corrupt_delay(net):
    store, chain, comms = net
    totalks = {"w.": 4096}

    async def go():
        for u in (1, 2, 3):
            await comms[u].put(payload(u), window=11, key="gradient", uid=str(u), local=False)
        store.faults = {"gradient-11-1-": "drop", "gradient-11-2-": "corrupt"}
        res = await comms[0].gather(my_uid=0, uids=[1, 2, 3], window=11, key="gradient", timeout=2, device="cpu",
                                    totalks=totalks, local=False)
        assert res.uids == [3] and sorted(res.skipped_uids) == [1, 2] and abs(res.success_rate - 1 / 3) < 1e-9
        store.faults = {"gradient-11-3-": ("delay", 5.0)}
        comms[0].gather_timeout = 1
        res = await comms[0].gather(my_uid=0, uids=[3], window=11, key="gradient", timeout=1, device="cpu", totalks=totalks, local=False)
        assert res is None                                  # whole gather timed out, nothing hangs
    run(go())


def test_check_compressed_indices(net):
    _, _, comms = net
    c = comms[0]
    vals = torch.zeros(3, 4)
    good = C.pack_12bit_indices(torch.randint(0, 64, (3, 4)))
    c.check_compressed_indices("p", good, 64, allowed_topk=4, vals=vals)
    for bad_idx, kw in ((good.to(torch.int64), {}), (good, {"vals": None}), (good[:3], {}),
                        (C.pack_12bit_indices(torch.full((3, 4), 70)), {}), (good, {"allowed_topk": 2})):
        with pytest.raises(ValueError):
            c.check_compressed_indices("p", bad_idx, 64, **({"allowed_topk": 4, "vals": vals} | kw))


def test_peer_list_start_window_and_activity(net):
    store, chain, comms = net

    async def go():
        v = comms[0]                     # uid 0 has the highest stake on the static chain
        await v.post_start_window(42)
        assert await comms[2].get_start_window(retries=1, retry_delay=0.01) == 42
        await v.post_peer_list(peers=[1, 2], reserve_peers=[3], first_effective_window=10, sync_window=9, initial_selection=True)
        await v.post_peer_list(peers=[2, 3], reserve_peers=[], first_effective_window=12, sync_window=11, initial_selection=False)
        assert await comms[2].get_peer_list() == ([2, 3], [], 12)
        assert await comms[2].get_peer_list(fetch_previous=True) == ([1, 2], [3], 10)
        comms[2].current_window = 20
        assert not await comms[2].is_miner_active(1, recent_windows=2)
        await comms[1].put(payload(1), window=19, key="gradient", uid="1", local=False)
        assert await comms[2].is_miner_active(1, recent_windows=2)
        assert await comms[2].refresh_active_peers() == {1}
        comms[2].update_peers_with_buckets()
        assert comms[2].eval_peers == {1: 1}
        comms[2].active_peers = set()
        comms[2].eval_peers = {1: 1}
        comms[2].active_peers = {3}
        comms[2].update_peers_with_buckets()
        assert comms[2].inactive_peers == {1} and 3 in comms[2].eval_peers
    run(go())


def test_weighted_sampling_and_stale_cleanup(net, tmp_path):
    store, chain, comms = net
    c = comms[1]
    assert c.weighted_random_sample_no_replacement([], [], 3) == []
    got = c.weighted_random_sample_no_replacement([1, 2, 3, 4], [0, 1, 1, 5], 3)
    assert len(got) == 3 and 1 not in got and len(set(got)) == 3

    async def go():
        for w in (1, 2, 30):
            await c.put(payload(w), window=w, key="gradient", uid="1", local=False)
        await c.cleanup_s3_data(uid="1", current_window=30, stale_retention=10)
        keys = [o.key for o in await store.list(c.bucket, "gradient-")]
        assert len(keys) == 1 and "gradient-30-1-" in keys[0]
    run(go())


def test_local_fs_store_roundtrip(tmp_path):
    st = LocalFSStore(tmp_path)
    b = Bucket(name="bkt", account_id="a" * 32, access_key_id="k" * 32, secret_access_key="s" * 64)

    async def go():
        await st.put_bytes(b, "dir/x.bin", b"hello")
        assert await st.get_bytes(b, "dir/x.bin") == b"hello" and (await st.head(b, "dir/x.bin")).size == 5
        assert [o.key for o in await st.list(b, "dir/")] == ["dir/x.bin"]
        assert await st.get_to_file(b, "dir/x.bin", str(tmp_path / "out.bin")) and not await st.get_to_file(b, "nope", "/tmp/z")
        await st.delete(b, ["dir/x.bin"])
        assert await st.head(b, "dir/x.bin") is None
    run(go())


class _FakeS3:
    """aiobotocore-shaped client: multipart upload with a vanishing upload id and flaky parts."""

    def __init__(self):
        self.objects, self.uploads, self.fail_parts, self.forget_once = {}, {}, 2, True

    async def create_multipart_upload(self, Bucket, Key):
        uid = f"u{len(self.uploads)}"
        self.uploads[uid] = {}
        return {"UploadId": uid}

    async def upload_part(self, Bucket, Key, PartNumber, UploadId, Body, ContentMD5=None):
        if self.forget_once and PartNumber == 2:
            self.forget_once = False
            raise RuntimeError("NoSuchUpload")
        if self.fail_parts > 0 and PartNumber == 1:
            self.fail_parts -= 1
            raise IOError("transient")
        self.uploads[UploadId][PartNumber] = Body
        return {"ETag": f"e{PartNumber}"}

    async def complete_multipart_upload(self, Bucket, Key, UploadId, MultipartUpload):
        self.objects[Key] = b"".join(self.uploads[UploadId][p["PartNumber"]] for p in MultipartUpload["Parts"])

    async def abort_multipart_upload(self, **kw):
        return None


def test_s3_multipart_upload_retries_and_restarts(tmp_path, monkeypatch):
    monkeypatch.setattr(asyncio, "sleep", _fast_sleep(asyncio.sleep))
    fake = _FakeS3()
    st = S3Store(client_factory=lambda b: fake, part_size=1024, concurrency=2, max_retries=4)
    data = os.urandom(5000)
    p = tmp_path / "big.bin"
    p.write_bytes(data)
    b = Bucket(name="bkt", account_id="a" * 32, access_key_id="k" * 32, secret_access_key="s" * 64)
    run(st.upload_large_file(b, "big.bin", str(p)))
    assert fake.objects["big.bin"] == data and len(fake.uploads) == 2      # restarted once with a new upload id
    chunk, workers = st.download_plan(10 * 1024 ** 3, workers=8)
    assert 64 * 1024 ** 2 <= chunk <= 1024 ** 3 and 1 <= workers <= 8


def _fast_sleep(real):
    async def s(t, *a, **k):
        return await real(0)
    return s


def test_decorators_and_config(monkeypatch):
    from templar_b200 import config, decos

    calls = {"n": 0}

    @decos.retry_on_failure(retries=3, delay=0.0)
    async def flaky():
        calls["n"] += 1
        return None if calls["n"] < 3 else "ok"
    assert run(flaky()) == "ok" and calls["n"] == 3

    @decos.sync_exception_catcher(on_error_return=lambda e: -1)
    def boom():
        raise ValueError("x")
    assert boom() == -1

    class Node:
        is_master = False

        @decos.master_only
        def f(self):
            return 1
    assert Node().f() is None
    for v in config.REQUIRED_VARS:
        monkeypatch.delenv(v, raising=False)
    with pytest.raises(ImportError):
        config.load_bucket_secrets(strict=True)
    assert "gradients" in config.load_bucket_secrets(strict=False)
    monkeypatch.setenv("R2_DATASET_BUCKET_LIST", '[{"name": "d1"}, {"name": "d2"}]')
    assert config.load_bucket_secrets(strict=False)["dataset"]["multiple"][1]["name"] == "d2"
    r = tplr.CommsGetResult(status="OK")
    assert not r.success and tplr.CommsGetResult(data={}, status="OK").success


class _RangeBody:
    def __init__(self, data):
        self.data = data

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc):
        return None

    async def read(self):
        return self.data


class _FakeRangedS3:
    """get_object with Range; the first ``flaky`` requests of chunk 1 return short data, ``dead`` chunks always fail."""

    def __init__(self, data, flaky=0, dead=()):
        self.data, self.flaky, self.dead, self.requests = data, flaky, set(dead), []

    async def head_object(self, Bucket, Key):
        from datetime import datetime, timezone
        return {"ContentLength": len(self.data), "LastModified": datetime.now(timezone.utc)}

    async def get_object(self, Bucket, Key, Range=None):
        lo, hi = (int(x) for x in Range.split("=")[1].split("-"))
        self.requests.append((lo, hi))
        if lo in self.dead:
            raise IOError("connection reset")
        if self.flaky > 0 and lo > 0:
            self.flaky -= 1
            return {"Body": _RangeBody(self.data[lo: hi])}            # one byte short
        return {"Body": _RangeBody(self.data[lo: hi + 1])}


def test_ranged_download_retries_short_chunks_and_resumes(tmp_path, monkeypatch):
    monkeypatch.setattr(asyncio, "sleep", _fast_sleep(asyncio.sleep))
    data = os.urandom(10_000)
    b = Bucket(name="bkt", account_id="a" * 32, access_key_id="k" * 32, secret_access_key="s" * 64)
    out = tmp_path / "big.bin"

    # 1. short reads are retried; the file is complete and the progress file is gone
    fake = _FakeRangedS3(data, flaky=2)
    st = S3Store(client_factory=lambda bk: fake, max_retries=4)
    monkeypatch.setattr(st, "download_plan", lambda size, workers=None: (3000, 2))
    assert run(st.download_large_file(b, "big.bin", len(data), str(out)))
    assert out.read_bytes() == data and not (tmp_path / "big.bin.progress").exists()
    assert len(fake.requests) == 4 + 2

    # 2. a chunk that never arrives: the call reports failure and records the finished chunks
    out.unlink()
    fake = _FakeRangedS3(data, dead=(6000,))
    st = S3Store(client_factory=lambda bk: fake, max_retries=2)
    monkeypatch.setattr(st, "download_plan", lambda size, workers=None: (3000, 2))
    assert not run(st.download_large_file(b, "big.bin", len(data), str(out)))
    done = {int(x) for x in (tmp_path / "big.bin.progress").read_text().split()}
    assert done == {0, 1, 3}

    # 3. the next attempt fetches only the missing chunk
    fake = _FakeRangedS3(data)
    st = S3Store(client_factory=lambda bk: fake, max_retries=2)
    monkeypatch.setattr(st, "download_plan", lambda size, workers=None: (3000, 2))
    assert run(st.download_large_file(b, "big.bin", len(data), str(out)))
    assert fake.requests == [(6000, 8999)] and out.read_bytes() == data


def test_ranged_read_on_every_transport(net, tmp_path):
    """Inclusive byte ranges through the S3 client, the local store and the in-memory store, and through
    Comms.s3_get_object_range; a range past the end, a short answer and a missing object read as None."""
    data = os.urandom(5000)
    b = Bucket(name="bkt", account_id="a" * 32, access_key_id="k" * 32, secret_access_key="s" * 64)
    fake = _FakeRangedS3(data)
    s3 = S3Store(client_factory=lambda bk: fake)
    assert run(s3.get_range(b, "x", 10, 19)) == data[10:20] and fake.requests == [(10, 19)]
    assert run(s3.get_range(b, "x", 4990, 5200)) is None               # the fake answers with fewer bytes
    assert run(s3.get_range(b, "x", 5, 4)) is None
    fs = LocalFSStore(tmp_path)
    run(fs.put_bytes(b, "x", data))
    assert run(fs.get_range(b, "x", 0, 0)) == data[:1] and run(fs.get_range(b, "x", 4000, 4999)) == data[4000:]
    assert run(fs.get_range(b, "x", 4000, 5000)) is None and run(fs.get_range(b, "nope", 0, 1)) is None
    comms = net[2][0]
    run(comms.store.put_bytes(comms.bucket, "blob", data))
    assert run(comms.s3_get_object_range(comms.bucket, "blob", 100, 163)) == data[100:164]
    assert run(comms.s3_get_object_range(comms.bucket, "missing", 0, 3)) is None


def test_large_file_calls_on_comms_and_chain_metadata_decoding(net, tmp_path, monkeypatch):
    """Comms.upload_large_file / download_large_file reach the transport's multipart upload and ranged download where it
    has them and fall back to whole objects where it has not; ChainManager.decode_metadata reads one commitment entry."""
    store, chain, comms = net
    c = comms[1]
    src = tmp_path / "blob.bin"
    src.write_bytes(os.urandom(9000))
    run(c.upload_large_file(str(src), "big/blob.bin"))                     # in-memory store: one object
    assert run(store.get_bytes(c.bucket, "big/blob.bin")) == src.read_bytes()
    assert run(c.download_large_file(c.bucket, "big/blob.bin", 9000, str(tmp_path / "back.bin")))
    assert (tmp_path / "back.bin").read_bytes() == src.read_bytes()
    assert not run(c.download_large_file(c.bucket, "big/none.bin", 1, str(tmp_path / "none.bin")))

    fake = _FakeS3()
    fake.fail_parts, fake.forget_once = 0, False
    s3 = S3Store(client_factory=lambda bk: fake, part_size=4000, max_retries=2)
    c3 = tplr.Comms(wallet=StaticWallet("hotkey-9"), config=SimpleNamespace(netuid=3, device="cpu"),
                    hparams=SimpleNamespace(topk_compression=4, blocks_per_window=4), uid=9, store=s3, subtensor=chain)
    run(c3.upload_large_file(str(src), "big/blob.bin"))
    assert fake.objects["big/blob.bin"] == src.read_bytes() and len(fake.uploads["u0"]) == 3      # three parts
    ranged = _FakeRangedS3(src.read_bytes())
    c3.store = S3Store(client_factory=lambda bk: ranged)
    monkeypatch.setattr(c3.store, "download_plan", lambda size, workers=None: (4000, 2))
    assert run(c3.download_large_file(c3.bucket, "big/blob.bin", 9000, str(tmp_path / "r.bin")))
    assert (tmp_path / "r.bin").read_bytes() == src.read_bytes() and sorted(ranged.requests) == [(0, 3999), (4000, 7999), (8000, 8999)]

    text = "x" * 128
    entry = {"info": {"fields": [[{"Raw128": [tuple(text.encode())]}]]}}
    got = tplr.ChainManager.decode_metadata((b"\x01" * 32,), entry, decode_account_id=lambda raw: "5F" + raw.hex()[:6])
    assert got == ("5F010101", text)


def test_gather_accepts_quantised_payloads_and_rejects_bad_tables(net):
    store, chain, comms = net
    totalks, xshapes = {"w.": 4096}, {"w.": (2, 2, 64, 64)}
    comp = C.TopKCompressor(use_quantization=True, quantization_bins=16)

    def qpayload(seed, *, shift=None, scale=None, lookup_nan=False, drop_params=False, lookup_edit=None):
        g = torch.Generator().manual_seed(seed)
        idx, q, xshape, totalk, qp = comp.compress(torch.randn(2, 2, 64, 64, generator=g), 4)
        sh, sc, off, lut, dt = qp
        lut = lut.clone()
        if lookup_nan:
            lut[3] = float("nan")
        if lookup_edit is not None:
            lut = lookup_edit(lut, q)
        qp = (sh if shift is None else torch.tensor(shift), sc if scale is None else scale, off, lut, dt)
        return {"w.idxs": idx, "w.vals": q, "w.quant_params": None if drop_params else qp}

    async def go():
        await comms[0].put(qpayload(0), window=5, key="gradient", uid="0", local=False)
        await comms[1].put(qpayload(1, shift=float("inf")), window=5, key="gradient", uid="1", local=False)
        await comms[2].put(qpayload(2, scale=0.0), window=5, key="gradient", uid="2", local=False)
        await comms[3].put(qpayload(3, lookup_nan=True), window=5, key="gradient", uid="3", local=False)
        res = await comms[0].gather(my_uid=0, uids=[0, 1, 2, 3], window=5, key="gradient", timeout=2, device="cpu",
                                    totalks=totalks, local=False, xshapes=xshapes, compressor=comp)
        assert res.uids == [0] and sorted(res.skipped_uids) == [1, 2, 3]
        sd = vars(res.state_dict)
        assert sd["w.vals"][0].dtype == torch.uint8 and len(sd["w.quant_params"]) == 1      # codes kept, tables beside them
        deq = comp.maybe_dequantize_values(sd["w.vals"], sd["w.quant_params"], "cpu")
        assert deq[0].dtype == torch.float32 and torch.isfinite(deq[0]).all()
        # a table that the codes would index out of range, or that is not a 1-D float table, is refused on the host
        bad_tables = [lambda lut, q: lut[: int(q.max())],                  # shorter than the largest code
                      lambda lut, q: lut.view(4, 4),                        # not 1-D
                      lambda lut, q: lut.to(torch.int64),                   # not floating point
                      lambda lut, q: torch.cat((lut, lut) * 16)]            # more entries than a byte can address
        for n, edit in enumerate(bad_tables):
            await comms[1].put(qpayload(10 + n, lookup_edit=edit), window=7 + n, key="gradient", uid="1", local=False)
            assert await comms[0].gather(my_uid=0, uids=[1], window=7 + n, key="gradient", timeout=1, device="cpu",
                                         totalks=totalks, local=False, xshapes=xshapes, compressor=comp) is None, n
        # codes without their table are refused
        await comms[1].put(qpayload(4, drop_params=True), window=6, key="gradient", uid="1", local=False)
        assert await comms[0].gather(my_uid=0, uids=[1], window=6, key="gradient", timeout=1, device="cpu", totalks=totalks,
                                     local=False, xshapes=xshapes, compressor=comp) is None
    run(go())


def test_background_activity_tracker_starts_once_and_stops_on_close(net, tmp_path):
    store, chain, comms = net

    async def go():
        c = comms[0]
        c.active_check_interval = 0.01
        await comms[1].put(payload(1), window=c.current_window, key="gradient", uid="1", local=False)
        c.start_background_tasks()
        task = c._active_task
        c.start_background_tasks()
        assert c._active_task is task                      # started once
        await asyncio.sleep(0.1)
        assert not task.done()
        await c.close_all_s3_clients()
        await asyncio.sleep(0)
        assert task.cancelled() or task.done()
        d = tmp_path / "x" / "y"
        d.mkdir(parents=True)
        c.delete_local_directory(str(tmp_path / "x"))
        c.delete_local_directory(str(tmp_path / "x"))        # missing path: no error
        assert not (tmp_path / "x").exists()
    run(go())


class ClientError(Exception):
    """Shaped like botocore's: the store recognises it by class name and reads ``response['Error']['Code']``."""

    def __init__(self, code):
        super().__init__(code)
        self.response = {"Error": {"Code": code}}


class _FakeObjS3:
    def __init__(self, objects):
        self.objects, self.made = dict(objects), 0

    async def head_object(self, Bucket, Key):
        if Key not in self.objects:
            raise ClientError("404")
        return {"ContentLength": len(self.objects[Key]), "LastModified": datetime(2026, 1, 1)}       # naive time stamp

    async def get_object(self, Bucket, Key, Range=None):
        if Key == "boom":
            raise ClientError("InternalError")
        if Key not in self.objects:
            raise ClientError("NoSuchKey")
        return {"Body": _RangeBody(self.objects[Key])}

    async def list_objects_v2(self, Bucket, Prefix, ContinuationToken=None):
        keys = sorted(k for k in self.objects if k.startswith(Prefix))
        start = int(ContinuationToken or 0)
        page = keys[start: start + 2]
        more = start + 2 < len(keys)
        return {"Contents": [{"Key": k, "Size": len(self.objects[k])} for k in page], "IsTruncated": more,
                "NextContinuationToken": str(start + 2) if more else None}

    async def put_object(self, Bucket, Key, Body):
        self.objects[Key] = Body


def test_s3_store_head_get_list_pagination_and_client_purge():
    b = Bucket(name="bkt", account_id="a" * 32, access_key_id="k" * 32, secret_access_key="s" * 64)
    made = []

    def factory(bucket):
        made.append(_FakeObjS3({f"p/{i}": bytes([i]) * (i + 1) for i in range(5)}))
        return made[-1]

    st = S3Store(client_factory=factory)

    async def go():
        assert await st.head(b, "p/9") is None and await st.get_bytes(b, "p/9") is None      # missing: None, no raise
        info = await st.head(b, "p/3")
        assert info.size == 4 and info.last_modified.tzinfo is not None                       # naive stamps become UTC
        assert await st.get_bytes(b, "p/2") == bytes([2]) * 3
        assert [o.key for o in await st.list(b, "p/")] == [f"p/{i}" for i in range(5)]         # three pages of two
        assert len(made) == 1                                                                 # one cached client so far
        with pytest.raises(ClientError):
            await st.get_bytes(b, "boom")                                                     # a real failure propagates
        await st.put_bytes(b, "q", b"x")
        assert len(made) == 2                                          # the client was purged after the ClientError
    run(go())


def test_commitment_map_of_a_substrate_chain_is_keyed_by_uid(monkeypatch):
    """The bittensor path: walk Commitments.CommitmentOf, decode account ids, keep registered hotkeys, skip garbage."""
    import sys
    import types

    mod = types.ModuleType("bittensor.core.chain_data")
    mod.decode_account_id = lambda raw: f"hk-{raw}"
    for name in ("bittensor", "bittensor.core"):
        monkeypatch.setitem(sys.modules, name, types.ModuleType(name))
    monkeypatch.setitem(sys.modules, "bittensor.core.chain_data", mod)

    def entry(account, text):
        return ([account], SimpleNamespace(value={"info": {"fields": [[{"Raw128": [text.encode()]}]]}}))

    good = "a" * 32 + "b" * 32 + "c" * 64
    asked = {}

    class _Substrate:
        def get_block_hash(self, block):
            return f"hash-{block}"

        def query_map(self, module, storage_function, params, block_hash):
            asked.update(module=module, fn=storage_function, params=params, block_hash=block_hash)
            return [entry(0, good), entry(1, "too short"), entry(7, good),            # 7 is not in the metagraph
                    ([2], SimpleNamespace(value={"info": {}}))]                        # undecodable entry

    cm = chain_mod.ChainManager.__new__(chain_mod.ChainManager)
    cm.netuid = 9
    cm.metagraph = SimpleNamespace(hotkeys=["hk-0", "hk-1", "hk-2"], uids=[0, 1, 2])
    cm.subtensor = SimpleNamespace(substrate=_Substrate())
    got = run(cm.get_commitments(block=5))
    assert asked == {"module": "Commitments", "fn": "CommitmentOf", "params": [9], "block_hash": "hash-5"}
    assert set(got) == {0} and got[0].account_id == "a" * 32 and got[0].secret_access_key == "c" * 64


def test_make_subtensor_never_falls_back_silently(monkeypatch):
    import builtins

    from templar_b200.backends.chain import make_subtensor

    assert isinstance(make_subtensor(SimpleNamespace(network="static", netuid=5, static_chain={"n": 3})), StaticChain)
    real_import = builtins.__import__

    def no_bittensor(name, *a, **k):
        if name == "bittensor":
            raise ImportError("no bittensor here")
        return real_import(name, *a, **k)

    monkeypatch.setattr(builtins, "__import__", no_bittensor)
    with pytest.raises(RuntimeError, match="bittensor package is not installed"):
        make_subtensor(SimpleNamespace(network="finney", netuid=5))
