"""Page-addressed streaming dataset on an in-memory row source (no network)."""

import asyncio
import os

import numpy as np
import torch

from templar_b200.dataset import DatasetLoader, MemoryRowSource, SubsetLoader


class _Tok:
    """One token per word (its length), EOS = 0."""

    eos_token_id = 0

    def encode(self, text, truncation=True, max_length=None):
        ids = [len(w) for w in text.split()]
        return ids[:max_length] if (truncation and max_length) else ids


def _source(n_cfg=3, n_rows=400):
    rng = np.random.default_rng(0)
    docs = {f"cfg{c}": [" ".join("x" * int(k) for k in rng.integers(1, 9, size=int(rng.integers(3, 40))))
                        for _ in range(n_rows)] for c in range(n_cfg)}
    return MemoryRowSource(docs)


def test_next_pages_is_deterministic_and_offset_dependent():
    src = _source()
    a = asyncio.run(DatasetLoader.next_pages(offset=5, n_pages=4, seed="miner-7", source=src))
    b = asyncio.run(DatasetLoader.next_pages(offset=5, n_pages=4, seed="miner-7", source=src))
    c = asyncio.run(DatasetLoader.next_pages(offset=6, n_pages=4, seed="miner-7", source=src))
    assert a == b and a != c
    for cfg, row, split in a:
        assert cfg in src.docs and split == "train" and 0 <= row < 400 - 1 - 100


def test_padded_batches_hold_one_document_per_sequence_group():
    src, tok = _source(), _Tok()
    pages = asyncio.run(DatasetLoader.next_pages(0, 2, 3, source=src))
    ds = asyncio.run(DatasetLoader.create(batch_size=4, sequence_length=16, pages_info=pages, tokenizer=tok,
                                          source=src))
    assert ds.get_page_names() == [f"{c}_{r}_{s}" for c, r, s in pages]
    first = [b.copy() for b in ds]
    assert first and all(b.shape == (4, 16) and b.dtype == np.int64 for b in first)
    flat = np.concatenate([b.reshape(-1) for b in first])
    # documents in page order, each padded with EOS to a multiple of 16 (their own EOS dropped)
    expect = []
    for page in pages:
        for text in asyncio.run(src.rows(page, 100)):
            body = tok.encode(text, max_length=16)
            expect += body + [0] * ((-len(body)) % 16)
    assert np.array_equal(flat, np.asarray(expect[: flat.size]))
    again = [b.copy() for b in ds]                       # a second pass replays the same documents
    assert len(again) == len(first) and all(np.array_equal(x, y) for x, y in zip(first, again))


def test_packed_batches_join_documents_with_one_eos():
    tok = _Tok()
    sl = SubsetLoader(batch_size=2, sequence_length=8, tokenizer=tok, pack_samples=True)
    sl.add_documents([[1, 2, 3], [4, 5, 0], [6] * 9, [7] * 20])
    out = np.concatenate([b.reshape(-1) for b in sl])
    stream = [1, 2, 3, 0, 4, 5, 0] + [6] * 9 + [0] + [7] * 20 + [0]
    assert out.size == 32 and np.array_equal(out, np.asarray(stream[:32]))
    assert sl._get_pad_size([1, 2, 3]) == 1
    sl.pack_samples = False
    assert sl._get_pad_size([1] * 8) == 0 and sl._get_pad_size([1] * 9) == 7


def test_random_pages_and_raw_rows():
    src, tok = _source(), _Tok()
    ds = asyncio.run(DatasetLoader.create(batch_size=2, sequence_length=8, num_pages=2, tokenizer=tok, source=src))
    assert len(ds.pages) == 2 and len(ds.buffer) > 0
    rows = asyncio.run(ds.fetch_data_to_rows(3))
    assert len(rows) == 300 and all(isinstance(r, str) for r in rows)
    cfgs = asyncio.run(DatasetLoader.fetch_dataset_configs(source=src))
    assert cfgs == {f"cfg{c}": {"num_rows": 400, "split": "train"} for c in range(3)}


def test_dataset_prep_shards_ids_and_reader(tmp_path):
    """pretokenize -> fixed-size shards with documents split across shard ends; ids = BLAKE2b-8 of each sequence;
    the sharded dataset reads what was written."""
    import hashlib
    import struct

    import templar_b200 as tplr
    from templar_b200 import dataset_prep as P

    tok = _Tok()
    docs = [" ".join("y" * (1 + (i * 7 + j) % 9) for j in range(5 + i % 11)) for i in range(200)]
    stream = []
    for d in docs:
        stream += tok.encode(d) + [0]
    paths = P.pretokenize(docs, tok, str(tmp_path), shard_size=512, seq_len=16)
    assert len(paths) == len(stream) // 512 and len(paths) >= 3
    for i, path in enumerate(paths):
        arr = np.load(path)
        assert arr.dtype == np.uint32 and arr.shape == (512,)
        assert np.array_equal(arr, np.asarray(stream[i * 512: (i + 1) * 512], dtype=np.uint32))
        ids = np.load(tmp_path / f"sample_ids_{i:06d}.npy")
        assert ids.dtype == np.uint64 and ids.shape == (32,)
        want = struct.unpack("<Q", hashlib.blake2b(arr[16:32].tobytes(), digest_size=8).digest())[0]
        assert int(ids[1]) == want == P.sample_id(arr[16:32])
    ds = tplr.SharedShardedDataset(1, 16, 0, 1, custom_path=str(tmp_path))
    assert len(ds) == 32
    assert np.array_equal(np.asarray(ds[3]), np.asarray(stream[512 + 48: 512 + 64]))
    assert int(ds.sample_id(3)) == P.sample_id(np.load(paths[1])[48:64])


def test_dataset_prep_cli_synthetic_and_ids(tmp_path, capsys):
    from templar_b200 import dataset_prep as P

    assert P.main(["synthetic", "--dir", str(tmp_path), "--shards", "2", "--tokens", "4096", "--seq-len", "64",
                   "--vocab-size", "1000"]) == 0
    a = np.load(tmp_path / "train_000001.npy")
    assert a.shape == (4096,) and int(a.max()) < 1000
    ids = np.load(tmp_path / "sample_ids_000001.npy").copy()
    (tmp_path / "sample_ids_000001.npy").unlink()
    assert P.main(["ids", "--dir", str(tmp_path), "--seq-len", "64", "--workers", "3"]) == 0
    assert np.array_equal(np.load(tmp_path / "sample_ids_000001.npy"), ids)
    assert P.shard_names(5, "anneal") == ("anneal_000005.npy", "sample_ids_anneal_000005.npy")


def test_http_row_source_against_a_local_rows_service():
    """HttpRowSource on a datasets-server shaped service started in-process: size listing, row pages, retry on 503."""
    from aiohttp import web

    from templar_b200.dataset import HttpRowSource

    tok = _Tok()
    docs = {"cfgA": [f"w{'x' * (i % 5)} yy z" for i in range(300)], "default": ["skip me"]}
    hits = {"rows": 0}

    async def size(request):
        assert request.query["dataset"] == "org/name"
        return web.json_response({"size": {"splits": [{"config": c, "split": "train", "num_rows": len(d)} for c, d in docs.items()]}})

    async def rows(request):
        hits["rows"] += 1
        if hits["rows"] == 1:
            return web.Response(status=503)                     # the first request fails: the source retries
        q = request.query
        off, lim = int(q["offset"]), int(q["limit"])
        return web.json_response({"rows": [{"row": {"text": t}} for t in docs[q["config"]][off: off + lim]]})

    async def go():
        app = web.Application()
        app.add_routes([web.get("/size", size), web.get("/rows", rows)])
        runner = web.AppRunner(app)
        await runner.setup()
        site = web.TCPSite(runner, "127.0.0.1", 0)
        await site.start()
        port = site._server.sockets[0].getsockname()[1]
        try:
            src = HttpRowSource("org/name", f"http://127.0.0.1:{port}/rows", f"http://127.0.0.1:{port}/size",
                                retry_limit=3, retry_delay=0.0)
            cfgs = await DatasetLoader.fetch_dataset_configs(source=src)
            assert cfgs == {"cfgA": {"num_rows": 300, "split": "train"}}
            ds = await DatasetLoader.create(batch_size=2, sequence_length=8, pages_info=[("cfgA", 10, "train")],
                                            tokenizer=tok, source=src)
            assert hits["rows"] == 2 and ds.get_page_names() == ["cfgA_10_train"]
            first = next(iter(ds))
            assert first.shape == (2, 8)
            want = tok.encode(docs["cfgA"][10], max_length=8)
            assert first[0, : len(want)].tolist() == want and first[0, len(want):].tolist() == [0] * (8 - len(want))
            hits["rows"] = -10                                    # every request fails from here on
            app_rows_fail = HttpRowSource("org/name", f"http://127.0.0.1:{port}/nope", f"http://127.0.0.1:{port}/size",
                                          retry_limit=2, retry_delay=0.0)
            try:
                await app_rows_fail.rows(("cfgA", 0, "train"), 5)
                raise AssertionError("a missing end point must raise after the retries")
            except RuntimeError as e:
                assert "Maximum retry attempts exceeded" in str(e)
        finally:
            await runner.cleanup()

    asyncio.run(go())


def test_shards_travel_through_the_dataset_bucket_and_the_manager_rotates_them(tmp_path, monkeypatch):
    """Shards uploaded with the prep tool are what a node's dataset manager downloads under a RELATIVE dataset path
    (the key is the path): the active shard on demand, the next one ahead of time, and after a swap the old files go."""
    import asyncio
    import json

    from templar_b200 import dataset_prep as P
    from templar_b200.backends.chain import StaticWallet
    from templar_b200.backends.store import MemoryStore
    from templar_b200.comms import Comms
    from templar_b200.sharded_dataset import ShardedDatasetManager

    seq, src = 8, tmp_path / "src"
    for i in range(3):
        P.synthetic_shard(str(src), i, seq * 5, seq, 100, seed=7)
    os.remove(src / "sample_ids_000002.npy")
    recs = P.scan_shards(str(src), "train", seq)
    assert [r["shard"] for r in recs] == [0, 1, 2] and recs[0]["sequences"] == 5 and recs[0]["leftover_tokens"] == 0
    assert recs[0]["ids_ok"] and recs[2]["ids"] is None and not recs[2]["ids_ok"]
    P.synthetic_shard(str(tmp_path / "ragged"), 4, seq * 5 + 3, seq, 100, seed=7)
    rag = P.scan_shards(str(tmp_path / "ragged"), "train", seq)[0]
    assert (rag["shard"], rag["sequences"], rag["leftover_tokens"], rag["ids_ok"], rag["dtype"]) == (4, 5, 3, True, "uint32")

    from templar_b200 import profilers
    prof = profilers.ShardProfiler("t", slow_read_s=60.0)
    monkeypatch.setattr(profilers, "ENABLE_SHARD_PROFILER", True)        # as if TPLR_ENABLE_SHARD_PROFILER were set
    monkeypatch.setattr(profilers, "_shard", prof)
    work = tmp_path / "node"
    work.mkdir()
    monkeypatch.chdir(work)
    monkeypatch.setenv("DATASET_BINS_PATH", "remote/tokenized")
    comms = Comms(wallet=StaticWallet("hotkey-1"), uid=1, store=MemoryStore())

    async def go():
        keys = await P.upload_shards(comms, str(src), [0, 1, 2], seq_len=seq)       # computes the missing ids of shard 2
        assert "remote/tokenized/train_000001.npy" in keys and len(keys) == 6 and (src / "sample_ids_000002.npy").exists()
        mgr = ShardedDatasetManager(seq, 0, 1, comms)
        mgr.max_dataset_idx = 3
        await mgr.initialize_datasets(0)
        assert len(mgr.active_dataset) == 5 and os.path.exists("remote/tokenized/train_000000.npy")
        await mgr.upcoming_dataset
        assert os.path.exists("remote/tokenized/train_000001.npy") and os.path.exists("remote/tokenized/sample_ids_000001.npy")
        assert not [f for f in os.listdir("remote/tokenized") if ".part" in f]
        first = mgr.active_dataset[1].clone()
        assert await mgr.swap_datasets() == 1
        assert not os.path.exists("remote/tokenized/train_000000.npy") and mgr.active_dataset.tokens_file.endswith("train_000001.npy")
        assert not torch.equal(first, mgr.active_dataset[1])
        await mgr.upcoming_dataset
        # the stand-alone downloader: keeps what is there, reports a shard that the bucket does not have
        done = await P.download_shards(comms, str(tmp_path / "dl"), [2, 9])
        assert done == {2: True, 9: False} and sorted(os.listdir(tmp_path / "dl")) == ["sample_ids_000002.npy", "train_000002.npy"]
    asyncio.run(go())
    assert P.main(["scan", "--dir", str(tmp_path / "dl"), "--seq-len", str(seq)]) == 0
    # the shard profiler saw the downloads and the opens of the shards the manager touched
    st = prof.get_stats()
    first, second = st["remote/tokenized/train_000000.npy"], st["remote/tokenized/train_000001.npy"]
    assert first["reads"] == 2 and first["min_time"] <= first["max_time"] <= first["total_time"]      # one download, one open
    assert sorted(r["what"] for r in second["timings"]) == ["download", "open"]
    assert second["num_rows"] == 5 and second["file_size"] > 0 and second["row_groups"] == 1
    prof.log_read_details("x", 1, 2, 0, 5); prof.log_read_complete("remote/tokenized/train_000000.npy", 0.1); prof.log_analysis()
    prof.export_data(str(tmp_path / "shards.json"))
    rep = json.loads((tmp_path / "shards.json").read_text())
    assert set(rep) == {"shard_statistics", "summary"} and rep["summary"]["reads"] >= 4
    assert rep["shard_statistics"]["remote/tokenized/train_000000.npy"]["file_size"] > 0
    prof.reset("remote/tokenized/train_000000.npy")
    assert "remote/tokenized/train_000000.npy" not in prof.get_stats() and prof.get_stats()
    prof.reset()
    assert prof.get_stats() == {} and profilers.get_profiler() is prof
    d = profilers.DummyShardProfiler()
    assert d.start_read("a") == "dummy_timer" and d.end_read("dummy_timer") == 0.0 and d.log_parquet_metadata("a", 1, 1, 1) is None and d.reset("a") is None
