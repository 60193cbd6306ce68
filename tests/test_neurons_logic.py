"""Protocol logic on CPU: gradient preparation (error feedback maths, null rounds), outer step,
engine path == generic path, sync metric, index overlap, slashing levels, peer rotation, catch-up."""

import asyncio
import math
from types import SimpleNamespace

import pytest
import torch

import templar_b200 as tplr
from templar_b200 import compress as C
from templar_b200.models.llama import ModelArgs, build_model
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine


def run(c):
    return asyncio.run(c)


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.a = torch.nn.Parameter(torch.randn(128, 64))
        self.b = torch.nn.Parameter(torch.randn(64))


def make_miner(use_dct=True, topk=8, quant=False):
    model = Tiny()
    m = SimpleNamespace(model=model, use_engine=False,
                        hparams=SimpleNamespace(use_dct=use_dct, topk_compression=topk, momentum_decay=0.9),
                        transformer=C.ChunkingTransformer(model, 64),
                        compressor=C.TopKCompressor(use_quantization=quant, quantization_bins=256),
                        owned_params={"a", "b"}, error_feedback={"a": None, "b": None}, error_feedback_cpu_buffers={})
    return m


@pytest.mark.parametrize("use_dct", [False, True])
def test_prepare_gradient_dict_error_feedback_maths(use_dct):
    m = make_miner(use_dct)
    g1 = {n: torch.randn_like(p) for n, p in m.model.named_parameters()}
    for n, p in m.model.named_parameters():
        p.grad = g1[n].clone()
    grad, xshapes, totalks = tplr.prepare_gradient_dict(m, step_window=3)
    assert grad["metadata"] == {"window": 3} and set(xshapes) == {"a", "b"} and totalks == {"a": 4096, "b": 64}
    assert grad["aidxs"].dtype == torch.uint8 and grad["avals"].shape == (2, 1, 8) and grad["aquant_params"] is None
    for n, p in m.model.named_parameters():
        sent = m.transformer.decode(m.compressor.decompress(p, grad[n + "idxs"], grad[n + "vals"], xshapes[n], totalks[n]),
                                    use_dct=use_dct)
        assert torch.allclose(m.error_feedback[n], g1[n] - sent, atol=1e-5)       # e = 0*gamma + g - sent
        assert p.grad is None
    e1 = {n: m.error_feedback[n].clone() for n in ("a", "b")}
    for n, p in m.model.named_parameters():
        p.grad = g1[n].clone()
    grad2, _, _ = tplr.prepare_gradient_dict(m, 4)
    for n, p in m.model.named_parameters():
        sent = m.transformer.decode(m.compressor.decompress(p, grad2[n + "idxs"], grad2[n + "vals"], xshapes[n], totalks[n]),
                                    use_dct=use_dct)
        assert torch.allclose(m.error_feedback[n], 0.9 * e1[n] + g1[n] - sent, atol=1e-5)
    for n, p in m.model.named_parameters():
        p.grad = g1[n].clone()
    grad3, _, _ = tplr.prepare_gradient_dict(m, 5, null_round=True)
    assert all(float(m.error_feedback[n].abs().max()) == 0 for n in ("a", "b")) and float(grad3["avals"].abs().max()) == 0


def test_prepare_gradient_dict_quantised_and_ownership():
    m = make_miner(quant=True)
    m.owned_params = {"a"}
    for n, p in m.model.named_parameters():
        p.grad = torch.randn_like(p)
    grad, xs, tk = tplr.prepare_gradient_dict(m, 1)
    assert "bidxs" not in grad and grad["avals"].dtype == torch.uint8 and len(grad["aquant_params"]) == 5
    assert m.model.b.grad is None


def _gather_result(model, n_peers, topk=8, use_dct=True, seed=0):
    tr, comp = C.ChunkingTransformer(model, 64), C.TopKCompressor()
    sd, xs, tk = {}, {}, {}
    g = torch.Generator().manual_seed(seed)
    for n, p in model.named_parameters():
        idxs, vals = [], []
        for j in range(n_peers):
            enc = tr.encode(torch.randn(p.shape, generator=g) * (1 + j), use_dct=use_dct)
            i, v, xs[n], tk[n] = comp.compress(enc, topk)
            idxs.append(i), vals.append(v)
        sd[n + "idxs"], sd[n + "vals"], sd[n + "quant_params"] = idxs, vals, [None] * n_peers
    return SimpleNamespace(state_dict=SimpleNamespace(**sd), uids=list(range(n_peers)), skipped_uids=[], success_rate=1.0), tr, comp, xs, tk


def test_outer_step_matches_manual_aggregation():
    model = Tiny()
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    gr, tr, comp, xs, tk = _gather_result(model, 3)
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    fp = tplr.outer_step(model, opt, gather_result=gr, transformer=tr, compressor=comp, xshapes=xs, totalks=tk, device="cpu",
                         is_master=True, world_size=1, use_dct=True)
    assert set(fp) >= {"param_norms", "param_means", "global_l2_norm", "total_elements"} and fp["total_elements"] == 128 * 64 + 64
    for n, p in model.named_parameters():
        sd = vars(gr.state_dict)
        g = tr.decode(comp.batch_decompress(p, sd[n + "idxs"], sd[n + "vals"], xs[n], tk[n], clip_norm=True), use_dct=True)
        assert torch.allclose(p.detach(), before[n] - 0.5 * g, atol=1e-6)
        assert abs(fp["param_norms"][n] - float(g.norm())) < 1e-4
    assert tplr.outer_step(model, opt, gather_result=None, transformer=tr, compressor=comp, xshapes=xs, totalks=tk,
                           device="cpu", is_master=True, world_size=1)["total_elements"] == 0


def test_outer_step_skips_non_finite_parameter():
    model = Tiny()
    before = model.a.detach().clone()
    gr, tr, comp, xs, tk = _gather_result(model, 2)
    vars(gr.state_dict)["avals"][0][0, 0, 0] = float("inf")
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    tplr.outer_step(model, opt, gather_result=gr, transformer=tr, compressor=comp, xshapes=xs, totalks=tk, device="cpu",
                    is_master=True, world_size=1, use_dct=True)
    assert torch.equal(model.a.detach(), before) and not torch.equal(model.b.detach(), Tiny().b.detach())


@pytest.mark.parametrize("update", ["sgd", "sign"])
def test_engine_window_equals_generic_functions(update):
    """The fused-path engine (CPU arithmetic) and the reference-semantics functions give the same weights."""
    args = ModelArgs(dim=64, n_layers=1, n_heads=2, vocab_size=128, intermediate_size=128, max_seq_len=32)
    torch.manual_seed(1)
    tok = torch.randint(0, 128, (2, 33))
    m1 = build_model(args, seed=3)
    eng = WindowEngine(m1, EngineConfig(topk=8, use_dct=True, momentum_decay=0.9, outer_lr=0.3, outer_update=update,
                                        inner_lr=1e-2, max_peers=3))
    eng.snapshot()
    eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0)
    eng.optimizer_step()
    eng.compress()
    own = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in eng.own_payload().items()}
    m2 = build_model(args, seed=3)
    opt = torch.optim.AdamW(m2.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    theta0 = {n: p.detach().clone() for n, p in m2.named_parameters()}
    m2.loss(tok[:, :-1], tok[:, 1:]).backward()
    torch.nn.utils.clip_grad_norm_(m2.parameters(), 1.0)
    opt.step()
    for n, p in m2.named_parameters():
        assert torch.allclose(p.detach(), dict(m1.named_parameters())[n].detach(), atol=2e-6), n
    miner = SimpleNamespace(model=m2, use_engine=False, hparams=SimpleNamespace(use_dct=True, topk_compression=8, momentum_decay=0.9),
                            transformer=C.ChunkingTransformer(m2, 64), compressor=C.TopKCompressor(),
                            owned_params={n for n, _ in m2.named_parameters()},
                            error_feedback={n: None for n, _ in m2.named_parameters()}, error_feedback_cpu_buffers={})
    with torch.no_grad():
        for n, p in m2.named_parameters():
            p.grad = theta0[n] - p.detach()
            p.copy_(theta0[n])
    grad, xs, tk = tplr.prepare_gradient_dict(miner, 0)
    for n, _ in m2.named_parameters():
        a = C.unpack_12bit_indices(own[n + "idxs"], own[n + "vals"].shape).sort(-1).values
        b = C.unpack_12bit_indices(grad[n + "idxs"], grad[n + "vals"].shape).sort(-1).values
        assert torch.equal(a, b), n
        assert torch.allclose(own[n + "vals"].abs().sort(-1).values, grad[n + "vals"].abs().sort(-1).values, atol=1e-6)
        assert torch.allclose(eng.store.view(eng.ef, n), miner.error_feedback[n], atol=1e-6)
    if update == "sgd":
        gr = SimpleNamespace(state_dict=SimpleNamespace(**{k: [v] for k, v in grad.items() if k != "metadata"}), uids=[0],
                             skipped_uids=[], success_rate=1.0)
        tplr.outer_step(m2, torch.optim.SGD(m2.parameters(), lr=0.3), gather_result=gr, transformer=miner.transformer,
                        compressor=miner.compressor, xshapes=xs, totalks=tk, device="cpu", is_master=True, world_size=1, use_dct=True)
        eng.outer_step(1)
        for n, p in m2.named_parameters():
            assert torch.allclose(p.detach(), dict(m1.named_parameters())[n].detach(), atol=2e-6), n
    else:
        eng.outer_step(1)
        g = C.ChunkingTransformer(m1, 64)
        moved = (eng.store.master_shard - eng.theta0).abs()
        assert float(moved.max()) <= 0.3 + 1e-6 and float(moved[moved > 0].min()) >= 0.3 - 1e-6


def test_engine_outer_step_through_public_api_and_fingerprint():
    args = ModelArgs(dim=64, n_layers=1, n_heads=2, vocab_size=128, intermediate_size=128, max_seq_len=32)
    m = build_model(args, seed=3)
    eng = WindowEngine(m, EngineConfig(topk=8, use_dct=True, max_peers=4))
    ref = build_model(args, seed=3)
    gr, tr, comp, xs, tk = _gather_result(ref, 3, seed=5)
    lr = 0.25
    tplr.outer_step(ref, torch.optim.SGD(ref.parameters(), lr=lr), gather_result=gr, transformer=tr, compressor=comp,
                    xshapes=xs, totalks=tk, device="cpu", is_master=True, world_size=1, use_dct=True)
    fp = tplr.outer_step(m, torch.optim.SGD(m.parameters(), lr=lr), gather_result=gr, transformer=tr, compressor=comp,
                         xshapes=xs, totalks=tk, device="cpu", is_master=True, world_size=1, use_dct=True)
    for n, p in ref.named_parameters():
        assert torch.allclose(p.detach(), dict(m.named_parameters())[n].detach(), atol=2e-6), n
    assert fp["global_l2_norm"] > 0


def test_compare_model_with_debug_dict():
    model = Tiny()
    dbg = {n + "_debug": p.detach().flatten()[:2].tolist() for n, p in model.named_parameters()}
    r = run(tplr.compare_model_with_debug_dict(model, dbg, learning_rate=0.01))
    assert r["success"] and r["l2_norm"] == 0 and r["avg_steps_behind"] == 0 and r["param_count"] == 4
    dbg["a_debug"] = [x + 0.02 for x in dbg["a_debug"]]
    r = run(tplr.compare_model_with_debug_dict(model, dbg, learning_rate=0.01))
    assert abs(r["max_steps_behind"] - 2.0) < 1e-3 and abs(r["max_diff"] - 0.02) < 1e-6
    r = run(tplr.compare_model_with_debug_dict(model, dbg, 0.01, param_avg_change={"a": torch.tensor([0.04, 0.04])}))
    assert abs(r["max_steps_behind"] - 0.5) < 1e-3
    r = run(tplr.compare_model_with_debug_dict(model, {}, 0.01))
    assert math.isinf(r["avg_steps_behind"]) and math.isinf(r["avg_l2_norm"])


class _OverlapComms:
    def __init__(self, ts): self.ts = ts
    async def gradient_timestamp(self, uid, window): return self.ts[uid]


def _overlap_case(idx_per_peer, ts, thr=0.9):
    model = torch.nn.Module()
    model.w = torch.nn.Parameter(torch.zeros(64, 64))
    vals = [torch.zeros(i.shape) for i in idx_per_peer]
    sd = SimpleNamespace(**{"widxs": [C.pack_12bit_indices(i) for i in idx_per_peer], "wvals": vals})
    gr = SimpleNamespace(uids=list(ts), state_dict=sd)
    neuron = SimpleNamespace(model=model, comms=_OverlapComms(ts), config=SimpleNamespace(device="cpu"))
    return run(tplr.check_uid_index_overlap(neuron, gr, window=5, overlap_threshold=thr))


def test_index_overlap_full_partial_none_and_offender_by_timestamp():
    a = torch.arange(8).view(1, 1, 8)
    full = _overlap_case([a, a.clone()], {10: 1.0, 11: 2.0})
    assert full["pairs_high_ovlap"] == 1 and full["uids_over_thresh"] == {11: "mega"} and full["max_overlap"] == 1.0
    half = _overlap_case([a, torch.tensor([[[0, 1, 2, 3, 100, 101, 102, 103]]])], {10: 5.0, 11: 2.0}, thr=0.5)
    assert abs(half["mean_overlap"] - 0.5) < 1e-6 and half["uids_over_thresh"] == {10: "max"}
    none = _overlap_case([a, a + 100, a + 200], {1: 1.0, 2: 2.0, 3: 3.0})
    assert none["pairs_checked"] == 3 and none["pairs_high_ovlap"] == 0 and none["mean_overlap"] == 0
    assert _overlap_case([a], {1: 1.0})["pairs_checked"] == 0


def test_slash_levels():
    assert [tplr.determine_slash_egregiousness(x) for x in (0.1, 0.5, 0.59, 0.6, 1.0)] == ["high", "max", "max", "mega", "mega"]
    with pytest.raises(ValueError):
        tplr.determine_slash_egregiousness(1.5)
    assert tplr.instantiate_slashing_multiplier() == {"high": 0.5, "max": 0.0, "mega": 0.0}


class _PeerComms:
    def __init__(self, lists):
        self.lists, self.peers, self.reserve_peers = lists, [], []
    async def get_peer_list(self, fetch_previous=False):
        return self.lists.get("prev" if fetch_previous else "cur")


def test_update_peers_rotation():
    inst = SimpleNamespace(comms=_PeerComms({"prev": ([1, 2], [3], 4), "cur": ([5, 6], [7], 10)}), next_peers=None,
                           next_reserve_peers=None, peers_update_window=8,
                           hparams=SimpleNamespace(peer_replacement_frequency=2, peer_list_window_margin=1))
    run(tplr.update_peers(inst, window=9, peer_start=tplr.T()))
    assert inst.comms.peers == [1, 2] and inst.next_peers == [5, 6] and inst.peers_update_window == 10
    run(tplr.update_peers(inst, window=10, peer_start=tplr.T()))
    assert inst.comms.peers == [5, 6] and inst.comms.reserve_peers == [7] and inst.next_peers is None


def test_handle_checkpoint_catchup_replays_scheduler(monkeypatch):
    calls = []

    async def fake_catchup(instance, start, aggregator_device=None):
        calls.append(start)
    monkeypatch.setattr(tplr.neurons, "catchup_with_aggregation_server", fake_catchup)
    sched = SimpleNamespace(n=0)
    sched.step = lambda: setattr(sched, "n", sched.n + 1)
    hp = SimpleNamespace(inner_steps=3, anneal_mode={"enabled": False},
                         optimizer={"type": "adamw", "adamw": {"scheduler": {"warmup_inner_steps": 5, "initial_warmup_inner_steps": 9,
                                                                             "replay_rewind_inner_steps": 4}}})
    inst = SimpleNamespace(hparams=hp, start_window=10, current_window=20, inner_scheduler=sched, inner_scheduler_step_count=0,
                           warmup_inner_steps=0, warmup_steps_taken=7, should_skip_scheduler_step=lambda: False)
    run(tplr.handle_checkpoint_catchup(inst, True, 15, 6, False))
    assert calls == [15] and sched.n == 6 * 3 - 4 and inst.warmup_inner_steps == 5 and inst.warmup_steps_taken == 0
    run(tplr.handle_checkpoint_catchup(inst, True, 15, 6, True))
    assert calls[-1] == 10 and inst.warmup_inner_steps == 9
    run(tplr.handle_checkpoint_catchup(inst, False, 0, 0, False))
    assert calls[-1] == 10
    run(tplr.handle_checkpoint_catchup(inst, True, 20, 2, False))
    assert len(calls) == 3                       # up to date: no replay
    hp.anneal_mode = {"enabled": True, "start_global_step": 4, "warmup_inner_steps": 2}
    sched.n = 0
    run(tplr.handle_checkpoint_catchup(inst, True, 20, 6, False))
    assert sched.n == 6 and inst.warmup_steps_taken == 2


def test_validator_gather_offload_round_trip():
    """offload / reload of a gathered state dict keeps values and structure (lists, tuples with non-tensor leaves)."""
    from neurons.validator import Validator

    v = Validator.__new__(Validator)
    v.hparams = SimpleNamespace(offload_gather_results=True)
    lookup = torch.arange(4.0)
    sd = SimpleNamespace(**{"w.idxs": [torch.arange(6, dtype=torch.uint8), torch.ones(6, dtype=torch.uint8)],
                            "w.vals": [torch.randn(4), torch.randn(4)],
                            "w.quant_params": [(0.5, 0.1, 128, lookup, torch.float32), None]})
    keep = [t.clone() for t in sd.__dict__["w.vals"]]
    res = SimpleNamespace(state_dict=sd, uids=[3, 4])
    v.offload_gather_results(res, log=False)
    assert res._offloaded == "cpu" and res.state_dict is sd
    assert all(t.device.type == "cpu" for t in sd.__dict__["w.vals"])
    qp = sd.__dict__["w.quant_params"]
    assert qp[1] is None and qp[0][0] == 0.5 and qp[0][4] is torch.float32 and torch.equal(qp[0][3], lookup)
    v.offload_gather_results(res, log=False)                       # second call is a no-op
    v.load_gather_results_to_device(res, torch.device("cpu"), log=False)
    assert res._offloaded is None
    assert all(torch.equal(a, b) for a, b in zip(sd.__dict__["w.vals"], keep))
    v.hparams.offload_gather_results = False
    v.offload_gather_results(res, log=False)
    assert res._offloaded is None


def test_engine_quantised_window_equals_generic_functions():
    """Engine with ``quantize`` against the reference-semantics functions with a quantising compressor: same
    codes, same tables, same error feedback, and the same weights after the outer step on the sent payload."""
    args = ModelArgs(dim=64, n_layers=1, n_heads=2, vocab_size=128, intermediate_size=128, max_seq_len=32)
    torch.manual_seed(1)
    tok = torch.randint(0, 128, (2, 33))
    m1 = build_model(args, seed=3)
    eng = WindowEngine(m1, EngineConfig(topk=8, use_dct=True, momentum_decay=0.9, outer_lr=0.3, inner_lr=1e-2,
                                        max_peers=3, quantize=True, quant_bins=16))
    hp = SimpleNamespace(use_dct=True, topk_compression=8, momentum_decay=0.9)
    node = SimpleNamespace(model=m1, use_engine=True, hparams=hp)
    eng.snapshot()
    eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0)
    eng.optimizer_step()
    sent, xs, tk = tplr.prepare_gradient_dict(node, 0)                   # engine path: codes + tables
    m2 = build_model(args, seed=3)
    opt = torch.optim.AdamW(m2.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    theta0 = {n: p.detach().clone() for n, p in m2.named_parameters()}
    m2.loss(tok[:, :-1], tok[:, 1:]).backward()
    torch.nn.utils.clip_grad_norm_(m2.parameters(), 1.0)
    opt.step()
    comp = C.TopKCompressor(use_quantization=True, quantization_bins=16, quantization_range=6)
    miner = SimpleNamespace(model=m2, use_engine=False, hparams=hp, transformer=C.ChunkingTransformer(m2, 64),
                            compressor=comp, owned_params={n for n, _ in m2.named_parameters()},
                            error_feedback={n: None for n, _ in m2.named_parameters()}, error_feedback_cpu_buffers={})
    with torch.no_grad():
        for n, p in m2.named_parameters():
            p.grad = theta0[n] - p.detach()
            p.copy_(theta0[n])
    grad, _, _ = tplr.prepare_gradient_dict(miner, 0)
    for n, _ in m2.named_parameters():
        assert sent[n + "vals"].dtype == torch.uint8 and grad[n + "vals"].dtype == torch.uint8
        qa, qb = sent[n + "quant_params"], grad[n + "quant_params"]
        assert abs(float(qa[0]) - float(qb[0])) < 1e-7 and abs(float(qa[1]) / float(qb[1]) - 1) < 1e-5
        da = comp._dequantize_values(sent[n + "vals"], qa).reshape(-1, sent[n + "vals"].shape[-1])
        db = comp._dequantize_values(grad[n + "vals"], qb).reshape(da.shape)
        ia = C.unpack_12bit_indices(sent[n + "idxs"], da.shape)
        ib = C.unpack_12bit_indices(grad[n + "idxs"], db.shape)
        oa, ob = ia.argsort(-1), ib.argsort(-1)
        assert torch.equal(ia.gather(-1, oa), ib.gather(-1, ob)), n
        assert torch.allclose(da.gather(-1, oa), db.gather(-1, ob), atol=2e-6), n
        assert torch.allclose(eng.store.view(eng.ef, n), miner.error_feedback[n], atol=2e-6), n
    # a receiver that stages the sent dict sees exactly the node's own (dequantised) payload
    from templar_b200.parallel.window_engine import peer_slice
    eng.load_peer_payload(0, peer_slice({k: [v] for k, v in sent.items() if k != "metadata"}, 0), non_blocking=False)
    assert torch.allclose(eng.peer_val[0], eng.own_val, atol=1e-7)


class _CatchupComms:
    """Serves the leader's aggregated gradients / debug dicts per window; records what was asked for."""

    def __init__(self, aggregated: dict, debug: dict, live=None):
        self.aggregated, self.debug, self.live = aggregated, debug, live
        self.metagraph = SimpleNamespace(S=torch.tensor([1.0, 9.0, 2.0]))       # leader = uid 1
        self.peers, self.asked, self.gathers = [0, 2], [], []

    async def get(self, uid, window, key, **kw):
        self.asked.append((uid, window, key))
        src = self.aggregated if key == "aggregator" else self.debug
        data = src.get(window)
        return SimpleNamespace(success=data is not None, data=data)

    async def gather(self, **kw):
        self.gathers.append(kw["window"])
        return self.live


def _catchup_instance(model, comms, current_window, tr, comp, xs, tk, lr=0.5):
    sched_steps = []
    inst = SimpleNamespace(
        model=model, comms=comms, start_window=10, current_window=current_window, is_master=True, world_size=1, uid=0,
        config=SimpleNamespace(device="cpu"), hparams=SimpleNamespace(blocks_per_window=4, inner_steps=3, use_dct=True,
                                                                      time_window_delta_seconds=12),
        outer_optimizer=torch.optim.SGD(model.parameters(), lr=lr), transformer=tr, compressor=comp, xshapes=xs, totalks=tk,
        global_step=0, inner_scheduler=SimpleNamespace(step=lambda: sched_steps.append(1)), inner_scheduler_step_count=0,
        should_skip_scheduler_step=lambda: False, query_block_timestamp=lambda b: 1000.0 + b, local_rank=0)
    return inst, sched_steps


def _as_payload(gr):
    return {"state_dict": vars(gr.state_dict), "uids": gr.uids, "skipped_uids": [], "success_rate": 1.0}


def test_catchup_replays_available_windows_skips_gaps_and_falls_back_to_a_live_gather():
    model, ref = Tiny(), Tiny()
    ref.load_state_dict(model.state_dict())
    g11, tr, comp, xs, tk = _gather_result(model, 2, seed=11)
    g13 = _gather_result(model, 2, seed=13)[0]
    g14 = _gather_result(model, 2, seed=14)[0]
    # windows 11 and 13 were aggregated by the leader, 12 is missing, 14 (the last one) only exists as live gradients
    comms = _CatchupComms({11: _as_payload(g11), 13: _as_payload(g13)}, {}, live=g14)
    inst, sched = _catchup_instance(model, comms, current_window=15, tr=tr, comp=comp, xs=xs, tk=tk)
    asyncio.run(tplr.neurons.catchup_with_aggregation_server(inst, 10))
    opt = torch.optim.SGD(ref.parameters(), lr=0.5)
    for gr in (g11, g13, g14):
        tplr.outer_step(ref, opt, gather_result=gr, transformer=tr, compressor=comp, xshapes=xs, totalks=tk, device="cpu",
                        is_master=True, world_size=1, use_dct=True)
    for (n, a), (_, b) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(a.detach(), b.detach(), atol=1e-6), n
    assert inst.global_step == 3 and len(sched) == 9 and inst.inner_scheduler_step_count == 9       # 3 applied windows x 3
    assert comms.gathers == [14]                                # live gather only for the last window
    assert [w for (_, w, k) in comms.asked if k == "aggregator"] == [11, 12, 13, 14]
    assert all(uid == "1" for uid, _, _ in comms.asked)


def test_catchup_follows_the_chain_head_and_survives_a_failed_fallback():
    model = Tiny()
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    g11, tr, comp, xs, tk = _gather_result(model, 2, seed=21)
    g12 = _gather_result(model, 2, seed=22)[0]
    comms = _CatchupComms({11: _as_payload(g11), 12: _as_payload(g12)}, {}, live=None)
    inst, _ = _catchup_instance(model, comms, current_window=12, tr=tr, comp=comp, xs=xs, tk=tk)
    real_get = comms.get

    async def get_and_advance(uid, window, key, **kw):
        if key == "aggregator" and window == 11:
            inst.current_window = 14                           # the chain moved on while we were replaying
        return await real_get(uid, window, key, **kw)

    comms.get = get_and_advance
    asyncio.run(tplr.neurons.catchup_with_aggregation_server(inst, 10))
    # 11 and 12 applied; 13 has neither aggregated nor live gradients and is skipped without an error
    assert inst.global_step == 2 and comms.gathers == [13]
    assert any(not torch.equal(p.detach(), before[n]) for n, p in model.named_parameters())
