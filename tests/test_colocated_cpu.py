"""Nodes that share a box (``neurons/miner.py --colocated``): gradients of co-located uids are taken from the peer
group (GPU peer memory on a B200 box, an all-gather on this CPU tier), never downloaded; uploads still happen."""

import torch

from templar_b200.backends.store import MemoryStore, PeerMemoryStore
from templar_b200.models.llama import ModelArgs, build_model
from templar_b200.parallel.peer_group import LocalPeerGroup
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine
from templar_b200.utils.synthetic import synthetic_payload
from test_distributed_cpu import launch


def test_two_colocated_miners_exchange_through_the_peer_group(tmp_path):
    res = launch(2, [tmp_path], worker="_gloo_colocated_worker.py", port=29653, timeout=600)
    assert [r["uid"] for r in res] == [2, 3]
    for r in res:
        assert r["success"] == [1.0, 1.0] and r["steps"] == 2 and r["ef"] > 0, r
        assert r["gradient_downloads"] == [], r                   # nothing of a co-located peer came through the store
    assert len(res[0]["uploaded"]) >= 4                           # yet both nodes uploaded both windows for everyone else
    assert res[0]["peers_agree"] < 1e-6                           # same peers, same update
    assert res[0]["vs_object_store"] < 1e-6 and res[0]["moved"] > 1e-5   # and the same as through the object store


def test_rank_addressed_peers_equal_slot_peers_in_the_engine():
    """``peers=[("rank", r)]`` reads the payload from where the owner compressed it; the result is that of the same
    payload staged in a slot."""
    args = ModelArgs(dim=128, n_layers=1, n_heads=2, vocab_size=256, intermediate_size=256, max_seq_len=32)

    def engine():
        eng = WindowEngine(build_model(args, seed=3), EngineConfig(max_peers=3))
        eng.snapshot()
        eng.store.master_shard.add_(torch.randn(eng.store.master_shard.shape, generator=torch.Generator().manual_seed(1)) * 1e-3)
        return eng

    a, b = engine(), engine()
    pay = [synthetic_payload(a.layout, 7 + j) for j in range(2)]
    for j in range(2):
        a.load_peer_payload(j, pay[j])
    a.outer_step(peers=[0, 1], include_own=False)
    b.load_peer_payload(0, pay[0])
    b.rank_payloads = {5: pay[1]}                                 # what LocalPeerGroup.exchange() provides on CPU
    b.outer_step(peers=[0, ("rank", 5)], include_own=False)
    assert torch.equal(a.store.master_shard, b.store.master_shard)


def test_peer_memory_store_answers_for_local_uids_only():
    import asyncio

    from templar_b200.schemas import Bucket

    group = LocalPeerGroup(7, rank=0, world_size=1)
    st = PeerMemoryStore(MemoryStore(), group)
    assert st.local_rank(7, 3) is None                            # nothing posted yet
    group.publish(3)
    assert st.local_rank(7, 3) == 0 and st.local_rank(7, 4) is None and st.local_rank(8, 3) is None
    b = Bucket(name="b", account_id="a", access_key_id="k", secret_access_key="s")
    assert asyncio.run(st.head(b, "gradient-3-7-v1.pt")) is not None          # liveness without touching the bucket
    assert asyncio.run(st.head(b, "gradient-3-8-v1.pt")) is None
    asyncio.run(st.put_bytes(b, "x", b"1"))
    assert asyncio.run(st.get_bytes(b, "x")) == b"1" and st.faults == {}      # everything else is the inner store
