"""End-to-end offline network on CPU: two miners and a validator exchanging gradients through an
in-memory object store on a static chain; plus unit tests of the validator's scoring state,
the trainer's LR warm-up / flatten rules, the model factory and small modules."""

import asyncio
import math
import os
import time
from types import SimpleNamespace

import pytest
import torch

import templar_b200 as tplr
from neurons.burn import get_config as burn_config, run as burn_run
from neurons.evaluator import Evaluator, ModelCache, compute_bpb
from neurons.miner import Miner
from neurons.trainer import Trainer
from neurons.validator import Validator, min_power_normalization
from templar_b200 import model_factory as mf
from templar_b200.backends.chain import StaticChain
from templar_b200.backends.store import MemoryStore
from templar_b200.utils.rating import PlackettLuce


def run(c):
    return asyncio.run(c)


@pytest.fixture()
def cwd_tmp(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("TPLR_LOG_LEVEL", "WARNING")
    monkeypatch.setenv("TPLR_METRICS_JSONL", str(tmp_path / "metrics.jsonl"))
    return tmp_path


def _node(cls, cfg_fn, argv, store, chain):
    return cls(config=cfg_fn(["--local", "--device", "cpu", *argv]), store=store, subtensor=chain)


def test_two_miners_and_a_validator_stay_in_sync(cwd_tmp):
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        miners = [_node(Miner, Miner.miner_config, ["--uid", str(u), "--peers", "2", "3"], store, chain) for u in (2, 3)]
        for n in miners + [v]:
            n.loop = asyncio.get_running_loop()
            n.comms.commitments = await n.comms.get_commitments()
            n.comms.peers = [2, 3]
            n.gather_timeout = 5
            await n.dataset_manager.initialize_datasets(0)
        for m in miners:
            m.set_dataloader()
        v.set_dataloader(validator=True)
        start = {n: p.detach().clone() for n, p in miners[0].model.named_parameters()}
        for w in range(1, 4):
            for m in miners:
                m.current_window = m.comms.current_window = w
            res = await asyncio.gather(*(m.run_window(w) for m in miners))
            assert all(r["gather_success_rate"] == 1.0 and r["global_step"] == w for r in res)
            v.current_window, v.comms.current_window, v.sync_window = w + 1, w, w
            out = await v.run_window()
            assert sorted(out["gathered"]) == [2, 3] and len(out["scored"]) == 2 and out["global_step"] == w
        await v.ckpt.flush_background_uploads()
        pm = [dict(m.model.named_parameters()) for m in miners]
        pv = dict(v.model.named_parameters())
        for n in pm[0]:
            assert torch.allclose(pm[0][n], pm[1][n], atol=1e-6), n          # same peers, same update
            assert torch.allclose(pm[0][n], pv[n], atol=1e-5), n             # the validator followed
            assert not torch.equal(pm[0][n], start[n]) or pm[0][n].numel() < 4
        assert v.evaluated_uids == {2, 3} and float(v.weights.sum()) == pytest.approx(1.0, abs=1e-5)
        assert os.path.exists(v.state_path)
        # the measurements of a validator window reached the metrics sink
        for n in miners + [v]:
            n.metrics_logger.close()                      # drains the writer thread's queue into the sink
        import json as _json
        seen = {}
        for line in (cwd_tmp / "metrics.jsonl").read_text().splitlines():
            rec = _json.loads(line)
            seen.setdefault(rec["measurement"].split("_", 0)[-1], rec)
        names = {k for k in seen}
        want = {"validator_window_v2", "validator_gradient_stats", "timing", "validator_scores", "training_step_v2"}
        assert all(any(n.endswith(w) for n in names) for w in want), sorted(names)
        stats = next(r for n, r in seen.items() if n.endswith("validator_gradient_stats"))["fields"]
        assert stats["mean_grad_norm"] > 0 and stats["min_grad_norm"] <= stats["median_grad_norm"] <= stats["max_grad_norm"]
        assert stats["mean_weight_norm"] > 0 and stats["grad_to_weight_ratio"] > 0
        # checkpoint published at global_step 2 is complete and loadable by a fresh evaluator
        assert await v.ckpt.check_checkpoint_exists(window=2)
        e = _node(Evaluator, Evaluator.evaluator_config, ["--uid", "1", "--skip-lm-eval", "--custom-eval-batches", "1"], store, chain)
        e.comms.commitments = await e.comms.get_commitments()
        assert await e.check_latest_checkpoint() == 2
        rep = await e.evaluate_window(2)
        assert rep["global_step"] == 2 and rep["perplexity"] > 1 and rep["bits_per_byte"] > 0
        # a miner that joins late catches up from the checkpoint + the validator's aggregated gradients
        late = _node(Miner, Miner.miner_config, ["--uid", "1", "--peers", "2", "3"], store, chain)
        late.loop = asyncio.get_running_loop()
        late.comms.commitments = await late.comms.get_commitments()
        late.comms.peers = [2, 3]
        late.current_window, late.start_window = 4, 1
        ok, win, step, boot = await tplr.neurons.load_checkpoint_with_fallback(late)
        assert (ok, win, step, boot) == (True, 2, 2, False)
        await tplr.neurons.handle_checkpoint_catchup(late, ok, win, step, boot)
        assert late.global_step == 3
        pl = dict(late.model.named_parameters())
        for n in pv:
            assert torch.allclose(pl[n], pv[n], atol=1e-5), n
    run(go())


def test_nodes_with_sharded_parameters_follow_the_same_protocol(cwd_tmp, monkeypatch):
    """``torchtitan.shard_params`` in the hparams: miners and the validator hold weights and gradients as shards (one
    rank each here, so the whole machinery runs in-process); they publish debug slices, score and stay in sync as the
    nodes with whole weights do."""
    real = tplr.load_hparams

    def sharded(*a, **k):
        hp = real(*a, **k)
        hp.torchtitan.shard_params = True
        return hp
    monkeypatch.setattr(tplr, "load_hparams", sharded)

    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        miners = [_node(Miner, Miner.miner_config, ["--uid", str(u), "--peers", "2", "3"], store, chain) for u in (2, 3)]
        for n in miners + [v]:
            assert n.engine.fsdp and n.engine.store.compute is None
            n.loop = asyncio.get_running_loop()
            n.comms.commitments = await n.comms.get_commitments()
            n.comms.peers = [2, 3]
            n.gather_timeout = 5
            await n.dataset_manager.initialize_datasets(0)
        for m in miners:
            m.set_dataloader()
        v.set_dataloader(validator=True)
        for w in range(1, 3):
            for m in miners:
                m.current_window = m.comms.current_window = w
            res = await asyncio.gather(*(m.run_window(w) for m in miners))
            assert all(r["gather_success_rate"] == 1.0 and r["global_step"] == w for r in res)
            v.current_window, v.comms.current_window, v.sync_window = w + 1, w, w
            out = await v.run_window()
            assert sorted(out["gathered"]) == [2, 3] and len(out["scored"]) == 2 and out["global_step"] == w
        full = [n.engine.full_state_dict() for n in miners + [v]]
        for k, t in full[0].items():
            if t.is_floating_point():
                assert torch.allclose(t, full[1][k], atol=1e-6) and torch.allclose(t, full[2][k], atol=1e-5), k
        # the published debug slices are the master weights' elements, not whatever a gather buffer holds
        dbg = await v.comms.get(uid="2", window=2, key="debug", local=False)
        name = "layers.0.attention.wq.weight"
        assert dbg.data[name + "_debug"] == pytest.approx(full[0][name].flatten()[10:12].tolist(), abs=1e-7)
        v.sync_window = 3                          # the sync check reads the debug slices of sync_window - 1
        sync = await v.evaluate_miner_sync(2)
        assert sync["success"] and sync["sync_score"] > 0.9, sync
    run(go())


def test_miner_survives_missing_and_corrupt_peers(cwd_tmp):
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        m = _node(Miner, Miner.miner_config, ["--uid", "2", "--peers", "1", "3"], store, chain)
        m.loop = asyncio.get_running_loop()
        m.comms.commitments = await m.comms.get_commitments()
        m.comms.peers = [1, 3]                 # nobody else uploads
        m.gather_timeout = 1
        await m.dataset_manager.initialize_datasets(0)
        m.set_dataloader()
        before = {n: p.detach().clone() for n, p in m.model.named_parameters()}
        m.current_window = 1
        r = await m.run_window(1)
        assert r["gather_success_rate"] == 0.0 and r["global_step"] == 0
        for n, p in m.model.named_parameters():
            assert torch.equal(p.detach(), before[n]), n          # window skipped: weights restored
        assert float(m.engine.ef.abs().max()) > 0                 # but the error feedback kept the work
    run(go())


# --------------------------------------------------------------------------------------- #
def _bare_validator():
    v = object.__new__(Validator)
    z = lambda: torch.zeros(256)  # noqa: E731
    v.gradient_scores, v.sync_scores, v.binary_indicator_scores = z(), z(), z()
    v.final_scores, v.binary_moving_averages, v.weights = z(), z(), z()
    v.hparams = SimpleNamespace(burn_rate=0.5, gather_share=0.75, gather_peer_count=2, reserve_peer_count=2, gather_top_ratio=2.0,
                                reserve_decay_ratio=0.5, gather_peers_slash_threshold=0.4, consecutive_negative_threshold=3,
                                exclude_negative_peers=True, missing_gradient_penalty_score=-99.0, bma_threshold=0.1,
                                bma_warmup_windows=0, sync_max_steps_behind=2, reset_inactivity_windows=3, uids_per_window=2,
                                minimum_peers=1, peer_replacement_frequency=2, peer_list_window_margin=1)
    v.openskill_model, v.openskill_ratings, v.current_window_scores = PlackettLuce(beta=7, tau=0.1), {}, {}
    v.evaluated_uids, v.eval_peers, v.inactive_scores = set(), {}, {}
    v.peer_eval_history, v.consecutive_negative_count, v.consecutive_missing_gradient_count = {}, {}, {}
    v.missing_gradient_history, v.excluded_from_gather, v.exclusion_start_window = {}, set(), {}
    v.peers_last_eval_window, v.naughty_peers = {}, {}
    v.eval_history_limit, v.missing_gradient_history_limit, v.naughty_peer_timeout = 20, 10, 20
    v.missing_gradient_slash_rate, v.sync_score_slash_rate, v.inactivity_slash_rate, v.score_zero_threshold = 0.75, 0.75, 0.25, 1e-4
    v.idx_similarity_slashing_rate = tplr.neurons.instantiate_slashing_multiplier()
    v.burn_uid, v.sync_window, v.current_window, v.start_window, v.is_master = 1, 10, 11, 0, True
    v.metrics_logger = None
    v.comms = SimpleNamespace(metagraph=SimpleNamespace(uids=torch.arange(256)), active_peers=set(), inactive_peers=set(),
                              weighted_random_sample_no_replacement=lambda c, w, k: c[:k])
    return v


def test_update_weights_emission_schedule():
    v = _bare_validator()
    for u, s in ((5, 4.0), (6, 3.0), (7, 2.0), (8, 1.0), (9, 0.5), (10, -1.0)):
        v.final_scores[u] = s
        v.evaluated_uids.add(u)
    v.update_weights()
    w = v.weights
    assert float(w.sum()) == pytest.approx(1.0, abs=1e-6) and float(w[1]) == pytest.approx(0.5)
    assert w[5] > w[6] > w[7] > w[8] > 0 and w[9] == 0 and w[10] == 0
    assert float(w[5] / w[6]) == pytest.approx(2.0, rel=1e-4)             # linear ramp top_ratio : 1
    assert float(w[7]) <= float(w[6])                                       # reserve never above gather
    v.final_scores.zero_()
    v.update_weights()
    assert float(v.weights[1]) == 1.0


def test_missing_gradient_ladder_and_reset():
    v = _bare_validator()
    v.final_scores[7] = 1.0
    v.binary_moving_averages[7] = 1.0
    v.slash_for_missing_gradients([7], success_rate=0.9)
    assert float(v.final_scores[7]) == pytest.approx(0.75)
    v.slash_for_missing_gradients([7], success_rate=0.9)
    assert float(v.final_scores[7]) == pytest.approx(0.375)
    v.slash_for_missing_gradients([7], success_rate=0.9)
    assert float(v.final_scores[7]) == 0.0 and v.current_window_scores[7] == -99.0
    v.final_scores[8] = 1.0
    v.slash_for_missing_gradients([8], success_rate=0.1)                  # poor gather: straight to 0
    assert float(v.final_scores[8]) == 0.0
    v.final_scores[9] = 1.0
    for _ in range(8):
        v.slash_for_missing_gradients([9], success_rate=0.9)
    assert 9 in v.naughty_peers and 9 not in v.openskill_ratings or float(v.final_scores[9]) == 0.0
    v.note_delivered([7])
    assert v.consecutive_missing_gradient_count[7] == 0
    v.slash_for_invalid_gradient(5, ValueError("bad"))
    assert 5 in v.evaluated_uids


def test_negative_evaluation_penalties_and_fifth_rank_rule():
    v = _bare_validator()
    v.final_scores[3] = 1.0
    v.binary_moving_averages[3] = 1.0
    for i in range(8):
        v.gradient_scores[3] = -0.1 if i < 6 else 0.1
        v.track_negative_evaluation(3)
    v.current_window_scores = {3: 0.1, 4: 0.2}
    v.apply_negative_evaluation_penalties()
    assert float(v.final_scores[3]) == pytest.approx(0.25)
    for _ in range(3):
        v.gradient_scores[3] = -0.1
        v.track_negative_evaluation(3)
    v.current_window_scores = {u: -0.1 for u in range(5)}                 # everybody negative: no punishment
    assert v.should_skip_negative_penalty() and not v.should_exclude_from_gather(3)
    v.apply_negative_evaluation_penalties()
    assert 3 not in v.excluded_from_gather
    v.current_window_scores = {u: 0.1 for u in range(5)}
    assert v.should_exclude_from_gather(3)
    v.apply_negative_evaluation_penalties()
    assert 3 in v.excluded_from_gather
    v.gradient_scores[3] = 0.2
    v.track_negative_evaluation(3)
    assert 3 not in v.excluded_from_gather and v.consecutive_negative_count[3] == 0


def test_openskill_update_overlap_slash_bins_and_inactivity():
    v = _bare_validator()
    v.current_window_scores = {1: 0.3, 2: 0.1, 3: -0.2}
    for u in (1, 2, 3):
        v.evaluated_uids.add(u)
        v.sync_scores[u] = 1.0
        v.binary_moving_averages[u] = 0.5
    v.update_openskill_ratings()
    assert v.openskill_ratings[1].mu > v.openskill_ratings[2].mu > v.openskill_ratings[3].mu and v.current_window_scores == {}
    assert float(v.final_scores[1]) == pytest.approx(v.openskill_ratings[1].ordinal() * 0.5)
    v.final_scores[2] = 2.0
    v.slash_from_overlap({"uids_over_thresh": {2: "high", 3: "mega", 999: "max"}})
    assert float(v.final_scores[2]) == pytest.approx(1.0) and 3 in v.naughty_peers and 3 not in v.openskill_ratings
    v.eval_peers = {u: 1 for u in range(20)}
    bins = v.bin_evaluation_peers(5)
    assert len(bins) == 5 and sorted(sum(bins.values(), [])) == list(range(20))
    assert len(v.select_evaluation_uids_from_bin(bins, 99)) == 2
    assert v.bin_evaluation_peers(50) == {0: list(range(20))}
    v.eval_peers = {}
    v.comms.inactive_peers = {4}
    v.final_scores[4] = 1.0
    v.penalize_inactive_peers()
    assert float(v.final_scores[4]) == pytest.approx(0.75)
    v.current_window += 10
    v.penalize_inactive_peers()
    assert float(v.final_scores[4]) == 0.0 and 4 not in v.inactive_scores
    assert torch.allclose(min_power_normalization(torch.tensor([1.0, 3.0])), torch.tensor([0.1, 0.9]))
    assert float(min_power_normalization(torch.zeros(3)).sum()) == 0


def test_peer_selection():
    v = _bare_validator()
    v.comms.active_peers = {2, 3, 4, 5, 6}
    v.comms.metagraph.I = torch.zeros(256)
    v.comms.metagraph.I[torch.tensor([2, 3])] = torch.tensor([0.5, 0.9])
    g, r = v.select_initial_peers()
    assert g == [3, 2] and len(r) == 2 and set(r) <= {4, 5, 6}
    v.weights[torch.tensor([4, 5, 6])] = torch.tensor([0.3, 0.2, 0.1])
    v.naughty_peers = {6: 5}
    g, r = v.select_next_peers()
    assert g == [4, 5] and 6 not in g + r
    v.comms.active_peers = set()
    assert v.select_next_peers() is None


# --------------------------------------------------------------------------------------- #
def _trainer(sched=None, anneal=None, inner_steps=10):
    t = Trainer()
    t.hparams = SimpleNamespace(inner_steps=inner_steps, anneal_mode=anneal or {"enabled": False},
                                optimizer={"type": "adamw", "adamw": {"learning_rate": 1e-3, "scheduler": sched or {}}})
    return t


def test_lr_flatten_window():
    t = _trainer({"flatten_start_step": 3, "flatten_duration": 2})
    for count, want in ((0, False), (29, False), (30, True), (49, True), (50, False)):
        t.inner_scheduler_step_count = count
        assert t.should_skip_scheduler_step() is want
    for s in ({}, {"flatten_start_step": None, "flatten_duration": 2}, {"flatten_start_step": 3, "flatten_duration": 0},
              {"flatten_start_step": 0, "flatten_duration": 5}):
        t2 = _trainer(s)
        t2.inner_scheduler_step_count = 35
        assert t2.should_skip_scheduler_step() is False


def test_warmup_scale_and_schedulers():
    t = _trainer({"warmup_steps": 4, "t_max": 100, "eta_min_factor": 0.1})
    t.warmup_inner_steps, t.warmup_steps_taken = 4, 0
    assert [round(t._warmup_scale(), 2) for t.warmup_steps_taken in (0, 1, 3, 4, 9)] == [0.25, 0.5, 1.0, 1.0, 1.0]
    t.hparams.anneal_mode = {"enabled": True}
    t.warmup_steps_taken = 0
    assert t._warmup_scale() == 1.0
    t.hparams.anneal_mode = {"enabled": False}
    t.inner_optimizer = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1e-3)
    s = t.get_inner_scheduler()
    lrs = []
    for _ in range(6):
        lrs.append(t.inner_optimizer.param_groups[0]["lr"])
        t.inner_optimizer.step()
        s.step()
    assert lrs[0] < lrs[1] < lrs[3] and lrs[4] == pytest.approx(1e-3, rel=1e-3) and lrs[5] < lrs[4]
    t2 = _trainer(anneal={"enabled": True, "warmup_inner_steps": 2, "decay_outer_steps": 1, "peak_lr_factor": 0.5, "eta_min_factor": 0.0},
                  inner_steps=4)
    t2.inner_optimizer = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    s2 = t2.get_inner_scheduler()
    seq = []
    for _ in range(7):
        seq.append(t2.inner_optimizer.param_groups[0]["lr"])
        t2.inner_optimizer.step()
        s2.step()
    assert seq[2] == pytest.approx(0.5, rel=1e-3) and seq[6] == pytest.approx(0.0, abs=1e-6)


def test_model_factory_roles_and_errors():
    hp = lambda **tt: SimpleNamespace(torchtitan=SimpleNamespace(**tt))  # noqa: E731
    assert mf.create_parallel_dims(16, hp(), "evaluator").dp_shard == 8
    assert mf.create_parallel_dims(8, hp(), "validator").dp_replicate == 2
    with pytest.raises(ValueError):
        mf.create_parallel_dims(6, hp(), "validator")
    d = mf.create_parallel_dims(8, hp(dp_shard=4, tp_degree=2), "miner")
    assert (d.dp_shard, d.tp, d.world_size) == (4, 2, 8) and d.mesh_shape() == {"dp_shard": 4, "tp": 2}
    assert mf.create_parallel_dims(8, hp(dp_shard=-1, tp_degree=2), "miner").dp_shard == 4
    for bad, msg in ((dict(dp_shard=0), "dp_shard cannot be zero"), (dict(dp_replicate=2, dp_shard=2), "but not both"),
                     (dict(dp_replicate=2, tp_degree=2), "tp/pp/cp are all 1"), (dict(dp_shard=3), "must be divisible")):
        with pytest.raises(ValueError, match=msg):
            mf.create_parallel_dims(8, hp(**bad), "miner")
    hpar = tplr.load_hparams(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hparams"), True)
    args = mf.get_titan_model_args(hpar)
    assert (args.dim, args.ffn_hidden, args.vocab_size) == (128, 256, 512)
    job = mf.create_job_config(hpar, "evaluator")
    assert job.mixed_precision_param == "float32" and job.mixed_precision_reduce == "float32"
    a = mf.initialize_torchtitan_model(hpar, "miner", "cpu", 1)
    b = mf.initialize_torchtitan_model(hpar, "evaluator", "cpu", 1)
    assert all(torch.equal(p, q) for p, q in zip(a.parameters(), b.parameters()))        # deterministic init
    meta = mf.create_meta_model(hpar, "miner", 1)
    assert next(meta.parameters()).is_meta


def test_hf_export_matches_model_logits(tmp_path):
    hpar = tplr.load_hparams(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hparams"), True)
    model = mf.initialize_torchtitan_model(hpar, "miner", "cpu", 1)
    hf = mf.convert_titan_to_hf(model, hpar, save_path=str(tmp_path / "hf"), is_master=True)
    assert (tmp_path / "hf" / "config.json").exists()
    if not isinstance(hf, dict):
        tok = torch.randint(0, 512, (2, 16))
        with torch.no_grad():
            assert torch.allclose(model(tok), hf(tok).logits, atol=2e-4, rtol=1e-3)


def test_small_modules(tmp_path, monkeypatch):
    assert compute_bpb(math.log(2.0) * 80, 10) == pytest.approx(8.0) and math.isinf(compute_bpb(1.0, 0))
    from neurons.evaluator import loss_to_bpb
    from neurons.validator import timer
    from templar_b200.metrics import NullMetricsLogger
    from templar_b200.wandb_ops import NullRun as _Run
    assert loss_to_bpb(math.log(2.0) * 80, 40, total_bytes=10) == pytest.approx(8.0)
    assert loss_to_bpb(math.log(2.0) * 80, 40, bytes_per_token=0.25) == pytest.approx(8.0) and math.isinf(loss_to_bpb(1.0, 0))
    with pytest.raises(ValueError):
        loss_to_bpb(1.0, 4)
    wb, seen = _Run(), []
    with timer("phase", wb, step=3, metrics_logger=SimpleNamespace(log=lambda **kw: seen.append(kw))):
        pass
    with timer("quiet", wb, step=None, metrics_logger=NullMetricsLogger()):
        pass
    assert list(wb.history[0][0]) == ["validator/phase"] and wb.history[0][1] == 3 and len(wb.history) == 1
    assert seen[0]["measurement"] == "timing" and seen[0]["tags"] == {"window": 3} and "phase" in seen[0]["fields"]
    c = ModelCache(tmp_path / "cache", namespace="v")
    assert not c.exists(1) and c.get_path(1) == tmp_path / "cache" / "v" / "window_1"
    for w in (1, 5, 12):
        c.get_path(w).mkdir(parents=True)
        (c.get_path(w) / "config.json").write_text("{}")
    (c.get_path(1) / "model.safetensors").write_bytes(b"x")
    (c.get_path(5) / "model-00001-of-00002.safetensors").write_bytes(b"x")
    c.mark(1); c.mark(5); c.mark(12)
    assert c.exists(1) and c.exists(5) and not c.exists(12) and not c.exists(2)      # 12 has no weight file
    (c.base_dir / "window_old").mkdir()                                         # not a window directory: left alone
    assert c.windows() == [1, 5, 12] and c.cleanup(keep_latest=1) == [1, 5]
    assert c.windows() == [12] and (c.base_dir / "window_old").exists()
    out = tmp_path / "lm"
    (out / "model_name").mkdir(parents=True)
    (out / "model_name" / "results_1.json").write_text(
        '{"results": {"arc_easy": {"acc,none": 0.5, "acc_norm,none": 0.6}, "piqa": {"acc,none": 0.7}, "odd": {"f1": 1}}}')
    assert Evaluator.parse_lm_eval_results(out) == {"arc_easy": 0.6, "piqa": 0.7}
    assert Evaluator.parse_lm_eval_results(out, with_metric=True) == {"arc_easy": ("acc_norm,none", 0.6), "piqa": ("acc,none", 0.7)}
    (out / "broken.json").write_text("{")
    os.utime(out / "broken.json", (time.time() + 5, time.time() + 5))
    assert Evaluator.parse_lm_eval_results(out) == {} and Evaluator.parse_lm_eval_results(tmp_path / "nothing") == {}
    chain = StaticChain(n=3, manual=True)
    chain.advance(400)
    assert burn_run(burn_config(["--max-iterations", "3", "--poll-seconds", "0"]), subtensor=chain, sleep=lambda s: chain.advance(200)) == 2
    from templar_b200.metrics import MetricsLogger
    from templar_b200.profilers import TimerProfiler, ShardProfiler, DummyTimerProfiler
    from templar_b200.wandb_ops import NullRun, versioned
    ml = MetricsLogger(prefix="T", uid=1, role="miner", jsonl_path=str(tmp_path / "m.jsonl"), flush_interval=0.05,
                       config=SimpleNamespace(netuid=3, device="cpu", project="p", _private=1, nested={"a": 1}, nothing=None))
    ml.log("m", {"w": 1}, {"loss": 1.5, "xs": [1.0, 2, 3.0], "uids": [4, 5, 6], "t": torch.tensor([2.0, 4.0]), "flag": True,
                           "name": "x", "none": None, "empty": [], "one": torch.tensor(7.0), "count": 3},
           with_system_metrics=True)
    ml.log("skipped", {}, {"a": 1}, sample_rate=0.0)
    ml.close()
    import json
    lines = (tmp_path / "m.jsonl").read_text().splitlines()
    rec = json.loads(lines[0])
    f, t = rec["fields"], rec["tags"]
    assert len(lines) == 1 and rec["measurement"] == "Tm"
    assert (f["xs_mean"], f["xs_min"], f["xs_max"], f["xs_median"]) == (2, 1, 3, 2) and f["t_max"] == 4 and f["one"] == 7
    assert f["uids"] == "[4, 5, 6]" and f["none"] == 0.0 and f["empty"] == 0.0 and f["flag"] == 1 and f["name"] == "x"
    assert f["count"] == 3 and isinstance(f["count"], int) and "sys_cpu_usage" in f and "sys_mem_total" in f
    assert (t["role"], t["uid"], t["prefix"], t["w"], t["config_netuid"], t["config_project"]) == ("miner", "1", "T", "1", "3", "p")
    assert t["runtime_id"] and t["version"] == tplr.__version__ and "config__private" not in t and "config_nested" not in t
    assert "config_nothing" not in t
    assert versioned({"a": 1}, "9") == {"v9/a": 1, "latest/a": 1}
    r = NullRun()
    r.log({"a": 1}, step=2)
    assert r.history == [({"a": 1}, 2)]
    tp = TimerProfiler("t")

    @tp.profile("f")
    def f():
        return 3

    @tp.profile("g")
    async def g():
        return 4
    assert f() == 3 and run(g()) == 4 and tp.get_stats("f")["count"] == 1 and tp.get_stats()["g"]["count"] == 1

    @tp.profile("boom")
    def boom():
        raise KeyError("x")

    @tp.profile("aboom")
    async def aboom():
        raise KeyError("y")
    for _ in range(12):
        with pytest.raises(KeyError):
            boom()
    with pytest.raises(KeyError):
        run(aboom())
    sb = tp.get_stats("boom")
    assert (sb["count"], sb["errors"], len(sb["timings"]), sb["function"]) == (12, 12, 10, "boom") and sb["avg"] == sb["mean"]
    assert tp.get_stats("aboom")["errors"] == 1 and tp.get_stats("f")["errors"] == 0 and "error" in tp.get_stats("nope")
    tp.start_timer("region"); assert tp.end_timer("region") >= 0 and tp.end_timer("region") == 0.0
    tp.log_summary()
    tp.reset("boom")
    assert "boom" not in tp.get_stats() and "f" in tp.get_stats()
    tp.reset()
    assert tp.get_stats() == {}
    assert DummyTimerProfiler().profile("x")(f)() == 3
    sp = ShardProfiler("s", slow_read_s=10)
    sp.end_read(sp.start_read("a.npy", {"idx": 1, "num_rows": 9}), "a.npy", num_row_groups=3, rows_per_group=3)
    sp.export_data(str(tmp_path / "rep.json"))
    rec = sp.get_stats("a.npy")
    assert (rec["reads"], rec["num_rows"], rec["row_groups"], rec["timings"][0]["idx"]) == (1, 9, 3, 1)
    assert (tmp_path / "rep.json").exists() and sp.get_stats("never") == {}
    m = PlackettLuce()
    a, b = m.rate([[m.rating()], [m.rating()]], scores=[1.0, 0.0])
    assert a[0].mu > 25 > b[0].mu and a[0].sigma < 25 / 3
    tplr.log_with_context("info", "hello", window=3, uid=1)


def test_phase_ranges_show_up_in_a_profiler_trace():
    """Phases are record_function scopes: a torch.profiler run lists them by name; iteration is labelled too."""
    import torch.profiler as tp

    from templar_b200.utils.ranges import labelled, nvtx_enabled, phase

    with tp.profile(activities=[tp.ProfilerActivity.CPU]) as prof:
        seen = []
        for x in labelled([1, 2, 3], "Data Loading"):
            with phase("Forward + Backward Pass"):
                seen.append(torch.ones(4) * x)
    names = {e.key for e in prof.key_averages()}
    assert "Data Loading" in names and "Forward + Backward Pass" in names
    assert len(seen) == 3 and not nvtx_enabled()


def test_quantised_payloads_travel_through_the_store_and_keep_nodes_in_sync(cwd_tmp):
    """Miners send 8-bit codes with per-tensor tables (the reference wire format); peers and the validator decode
    them when they stage the gathered payloads and end with the same weights."""
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        miners = [_node(Miner, Miner.miner_config, ["--uid", str(u), "--peers", "2", "3"], store, chain) for u in (2, 3)]
        for n in miners + [v]:
            n.loop = asyncio.get_running_loop()
            n.comms.commitments = await n.comms.get_commitments()
            n.comms.peers = [2, 3]
            n.gather_timeout = 5
            await n.dataset_manager.initialize_datasets(0)
        for m in miners:
            m.set_dataloader()
            m.engine.cfg.quantize, m.engine.cfg.quant_bins = True, 64
        v.set_dataloader(validator=True)
        for w in range(1, 3):
            for m in miners:
                m.current_window = m.comms.current_window = w
            res = await asyncio.gather(*(m.run_window(w) for m in miners))
            assert all(r["gather_success_rate"] == 1.0 for r in res)
            got = await v.comms.get(uid="2", window=w, key="gradient", local=False, stale_retention=10)
            vals = [t for k, t in got.data.items() if k.endswith("vals")]
            assert vals and all(t.dtype == torch.uint8 and int(t.max()) < 64 for t in vals)
            assert all(got.data[k] is not None for k in got.data if k.endswith("quant_params"))
            v.current_window, v.comms.current_window, v.sync_window = w + 1, w, w
            out = await v.run_window()
            assert sorted(out["gathered"]) == [2, 3]
        await v.ckpt.flush_background_uploads()
        pm = [dict(m.model.named_parameters()) for m in miners]
        pv = dict(v.model.named_parameters())
        for n in pm[0]:
            assert torch.allclose(pm[0][n], pm[1][n], atol=1e-6), n
            assert torch.allclose(pm[0][n], pv[n], atol=1e-5), n
    run(go())


def test_miner_window_with_muon_as_the_inner_optimizer(cwd_tmp):
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        m = _node(Miner, Miner.miner_config, ["--uid", "2", "--peers", "2"], store, chain)
        m.loop = asyncio.get_running_loop()
        m.comms.commitments = await m.comms.get_commitments()
        m.comms.peers = [2]
        m.gather_timeout = 5
        await m.dataset_manager.initialize_datasets(0)
        m.set_dataloader()
        m.engine.cfg.inner_optimizer = "muon"
        before = {n: p.detach().clone() for n, p in m.model.named_parameters()}
        m.current_window = m.comms.current_window = 1
        res = await m.run_window(1)
        assert res["global_step"] == 1 and res["gather_success_rate"] == 1.0
        moved = [float((p.detach() - before[n]).abs().max()) for n, p in m.model.named_parameters()]
        assert all(x == x for x in moved) and max(moved) > 0            # finite, and the model changed
        assert float(m.engine.exp_avg.abs().max()) > 0                  # Muon momentum / Adam moment were written
    run(go())


def test_evaluator_cli_spellings_and_dataset_path_evaluation(cwd_tmp):
    from templar_b200 import dataset_prep

    a = Evaluator.evaluator_config(["--local", "--device", "cpu", "--eval_interval", "5", "--from_window", "3", "--to_window", "4",
                                    "--no_follow", "--force_reval", "--custom_eval_path", "/x", "--cache_dir", "c", "--batch_size", "2"])
    b = Evaluator.evaluator_config(["--local", "--device", "cpu", "--eval-interval", "5", "--backfill-start", "3", "--backfill-end", "4",
                                    "--no-follow", "--force-reval", "--custom-eval-path", "/x", "--cache-dir", "c", "--batch-size", "2"])
    for k in ("eval_interval", "backfill_start", "backfill_end", "no_follow", "force_reval", "custom_eval_path", "cache_dir", "batch_size"):
        assert getattr(a, k) == getattr(b, k), k
    assert (a.backfill_start, a.backfill_end, a.no_follow, a.force_reval, a.batch_size) == (3, 4, True, True, 2)
    # "--offline" is "--local" under a name that a torchrun command line accepts in front of the script's own options
    assert Miner.miner_config(["--offline", "--device", "cpu"]).local and not Miner.miner_config(["--device", "cpu"]).local

    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        e = _node(Evaluator, Evaluator.evaluator_config, ["--uid", "1", "--skip-lm-eval", "--batch_size", "2"], store, chain)
        seq, vocab = e.hparams.sequence_length, e.hparams.model_config.vocab_size
        dataset_prep.synthetic_shard(str(cwd_tmp / "evalset"), 0, seq * 6, seq, vocab, seed=3, prefix="val")
        e.config.custom_eval_path = str(cwd_tmp / "evalset")
        synth = await e.run_custom_eval(1)                                   # no tokenizer: 4 bytes per token assumed
        assert synth["bytes_exact"] == 0.0 and 0.9 * 6 * (seq - 1) < synth["tokens"] <= 6 * (seq - 1)   # pad ids are masked
        e.tokenizer = SimpleNamespace(batch_decode=lambda ids, **kw: ["ab" * len(row) for row in ids],
                                      pad_token_id=getattr(e.tokenizer, "pad_token_id", 0),
                                      eos_token_id=getattr(e.tokenizer, "eos_token_id", 0))
        rep = await e.run_custom_eval(1)
        assert rep["bytes_exact"] == 1.0 and rep["bytes"] == 6 * seq * 2     # two bytes per token of every sequence
        assert rep["loss"] == pytest.approx(synth["loss"]) and rep["perplexity"] > 1
        assert rep["bits_per_byte"] == pytest.approx(compute_bpb(rep["loss"] * rep["tokens"], 6 * seq * 2))
    run(go())


FAKE_HARNESS = """#!/usr/bin/env python3
import json, os, sys
a = sys.argv[1:]
out, tasks = a[a.index("--output_path") + 1], a[a.index("--tasks") + 1].split(",")
model = dict(kv.split("=", 1) for kv in a[a.index("--model_args") + 1].split(","))["pretrained"]
assert os.path.exists(os.path.join(model, "config.json")), model
leaked = [k for k in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "NCCL_DEBUG", "TORCHELASTIC_RUN_ID") if k in os.environ]
os.makedirs(os.path.join(out, "model"), exist_ok=True)
if os.environ.get("FAKE_HARNESS_FAIL"):
    sys.exit(3)
json.dump({"results": {t: {"acc,none": 0.25, "acc_norm,none": 0.5 - 0.1 * len(leaked)} for t in tasks}},
          open(os.path.join(out, "model", "results_x.json"), "w"))
"""


def test_evaluator_baseline_then_checkpoints_with_a_task_harness(cwd_tmp, monkeypatch):
    """Nothing published: the untrained weights are evaluated once at step 0.  Then a checkpoint appears and is
    evaluated with the downstream-task child process, which gets the exported model and an environment without the
    launcher's variables; the per-window export cache keeps one window; a failing child leaves no scores."""
    import json as _json
    import stat

    bindir = cwd_tmp / "bin"
    bindir.mkdir()
    (bindir / "lm_eval").write_text(FAKE_HARNESS)
    (bindir / "lm_eval").chmod((bindir / "lm_eval").stat().st_mode | stat.S_IXUSR)
    monkeypatch.setenv("PATH", f"{bindir}{os.pathsep}{os.environ['PATH']}")

    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        v.comms.commitments = await v.comms.get_commitments()
        await v.comms.post_start_window(3)
        e = _node(Evaluator, Evaluator.evaluator_config,
                  ["--uid", "1", "--tasks", "arc_easy,piqa", "--custom-eval-batches", "1", "--no-follow"], store, chain)
        monkeypatch.setenv("RANK", "0"); monkeypatch.setenv("NCCL_DEBUG", "INFO")      # must not reach the child
        await e.run()
        assert e.start_window == 3 and e.baseline_evaluated and e.evaluated_windows == {3} and e.eval_counter == 1
        assert e.cache.windows() == [3] and e.cache.exists(3)
        # a checkpoint of window 5 (global step 2) is published; the follow loop picks it up and keeps one export
        v.global_step = 2
        await v.ckpt.save_local(model=v.model, window=5, sync_window=5, global_step=2)
        await v.ckpt.upload(window=5, background=False)
        await e.run()
        assert e.evaluated_windows == {3, 5} and e.last_eval_window == 5 and e.cache.windows() == [5]
        again = await e.evaluate_window(5)
        assert again["skipped"] and e.eval_counter == 2
        # failing child: custom metrics still there, no task scores, export still pruned to one window
        monkeypatch.setenv("FAKE_HARNESS_FAIL", "1")
        e.force_reval = True
        rep = await e.evaluate_window(5)
        assert rep["tasks"] == {} and rep["perplexity"] > 1 and rep["global_step"] == 2
        e.metrics_logger.close()
    run(go())
    recs = [_json.loads(l) for l in (cwd_tmp / "metrics.jsonl").read_text().splitlines()]
    tasks = [r for r in recs if r["measurement"].endswith("benchmark_task")]
    assert len(tasks) == 4 and {r["tags"]["task"] for r in tasks} == {"arc_easy", "piqa"}
    assert all(r["fields"]["score"] == pytest.approx(0.5) and r["tags"]["metric"] == "acc_norm,none" for r in tasks)
    custom = [r for r in recs if r["measurement"].endswith("custom_evaluation")]
    assert [int(r["tags"]["baseline"]) for r in custom] == [1, 0, 0] and [int(r["tags"]["global_step"]) for r in custom] == [0, 2, 2]
    summ = [r for r in recs if r["measurement"].endswith("benchmark_summary")]
    assert len(summ) == 2 and all(r["fields"]["num_tasks"] == 2 for r in summ)


def test_offline_evaluator_without_any_validator_evaluates_the_untrained_weights(cwd_tmp):
    """No validator, hence no start window and no checkpoint: an offline evaluator does not wait for ever; it counts its
    steps from the window it starts in and reports the baseline."""
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        e = _node(Evaluator, Evaluator.evaluator_config, ["--uid", "1", "--skip-lm-eval", "--custom-eval-batches", "1", "--no-follow"],
                  store, chain)
        e.current_window = 7
        await asyncio.wait_for(e.run(), timeout=60)
        assert e.start_window == 7 and e.baseline_evaluated and e.evaluated_windows == {7}
    run(go())


def test_miner_without_fixed_peers_finds_the_published_list_and_does_not_wait_for_ever(cwd_tmp):
    """A miner started without --peers asks for the validators' peer list every window: with no validator in sight it
    gives up after a bounded number of tries (offline) and runs a null round; once a list is published it adopts it
    when the list comes into effect.  Offline, a gather waits one window at most, not the network time-out."""
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        m = _node(Miner, Miner.miner_config, ["--uid", "2", "--block-time", "0.5"], store, chain)
        m.loop = asyncio.get_running_loop()
        m.comms.commitments = await m.comms.get_commitments()
        await m.dataset_manager.initialize_datasets(0)
        m.set_dataloader()
        assert m.gather_wait_seconds() == 2.0                    # 4 blocks x 0.5 s, not the 90 s of a network run
        m.config.local = False
        assert m.gather_wait_seconds() == 90.0
        m.config.local = True
        m.current_window = m.comms.current_window = 5
        t0 = time.time()
        res = await asyncio.wait_for(m.run_window(5), timeout=60)                    # nobody publishes a list
        assert m.comms.peers == [] and res["gather_success_rate"] == 0.0 and time.time() - t0 < 30
        # uid 0 (highest stake) commits its bucket and publishes a list that takes effect at window 7
        v = tplr.Comms(wallet=tplr.backends.chain.StaticWallet("hotkey-0"), config=m.config, hparams=m.hparams, uid=0,
                       store=store, subtensor=chain)
        v.try_commit(v.wallet, v.bucket)
        await v.post_peer_list(peers=[2], reserve_peers=[], first_effective_window=7, sync_window=6, initial_selection=True)
        m.comms.commitments = await m.comms.get_commitments()
        m.current_window = m.comms.current_window = 6
        await m.run_window(6)
        assert m.next_peers == [2] and m.comms.peers == [] and m.peers_update_window == 7
        m.current_window = m.comms.current_window = 7
        res = await m.run_window(7)
        assert m.comms.peers == [2] and m.next_peers is None and res["gather_success_rate"] == 1.0
    run(go())


def test_miner_runs_null_rounds_until_the_validators_can_know_it(cwd_tmp):
    """Outside local mode the first validator_offset + peer_list_window_margin windows after the start window, and
    windows without gather peers, are null rounds: no inner update is kept and nothing is fed into the error feedback."""
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        m = _node(Miner, Miner.miner_config, ["--uid", "2", "--peers", "2"], store, chain)
        m.loop = asyncio.get_running_loop()
        m.comms.commitments = await m.comms.get_commitments()
        m.comms.peers = [2]
        m.gather_timeout = 2
        await m.dataset_manager.initialize_datasets(0)
        m.set_dataloader()
        m.config.local, m.start_window = False, 10
        before = {n: p.detach().clone() for n, p in m.model.named_parameters()}
        def tick(to_window):           # outside local mode a miner waits for the chain before it uploads
            asyncio.get_running_loop().call_later(0.3, lambda: setattr(m, "current_window", to_window))

        m.current_window = m.comms.current_window = 11                 # offset 1 < warm-up of 3 windows
        tick(12)
        await m.run_window(11)
        assert float(m.engine.ef.abs().max()) == 0.0 and float(m.engine.own_val.abs().max()) == 0.0
        for n, p in m.model.named_parameters():
            assert torch.equal(p.detach(), before[n]), n
        m.comms.peers = []                                             # warm-up over, but nobody to gather from
        m.current_window = m.comms.current_window = 14
        tick(15)
        await m.run_window(14)
        assert float(m.engine.ef.abs().max()) == 0.0
        for n, p in m.model.named_parameters():
            assert torch.equal(p.detach(), before[n]), n
    run(go())


def test_upload_times_and_own_uploads_decide_who_is_gathered_scored_and_slashed(cwd_tmp):
    """The protocol on a chain with a clock (no ``--local``).  Miners finish training early, wait for the window to
    end and upload after the first block of the next window; everyone accepts an upload only from that block's
    time until ``time_window_delta_seconds`` later.  The validator scores every evaluation peer from that peer's
    OWN upload: a miner that is not on the gather list is scored all the same, an upload stamped before the window
    opened or after it closed is slashed as missing, and a malformed one is zeroed."""
    from datetime import datetime, timedelta, timezone
    import io
    import time as _time

    async def go():
        bpw, w = 4, 6
        store = MemoryStore()
        chain = StaticChain(n=7, manual=True, block_time=1.0)
        chain._manual_block = w * bpw
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        miners = {u: _node(Miner, Miner.miner_config, ["--uid", str(u), "--peers", "2", "3", "5"], store, chain) for u in (2, 3, 4)}
        ghosts = {u: tplr.Comms(wallet=tplr.backends.chain.StaticWallet(f"hotkey-{u}"), config=miners[2].config,
                                hparams=miners[2].hparams, uid=u, store=store, subtensor=chain) for u in (1, 5, 6)}
        for c in ghosts.values():
            c.try_commit(c.wallet, c.bucket)
        waiting = {u: asyncio.Event() for u in miners}
        for u, m in miners.items():
            m.config.local = False                       # a clock, acceptance times, the wait before the upload
            m.hparams.blocks_per_window = bpw
            m.loop = asyncio.get_running_loop()
            m.comms.commitments = await m.comms.get_commitments()
            m.comms.peers = [2, 3, 5]
            m.gather_timeout = 3
            m.start_window = 0
            await m.dataset_manager.initialize_datasets(0)
            m.set_dataloader()
            m.current_window = m.comms.current_window = w
            orig = m.wait_until_window

            async def waits(target, _orig=orig, _u=u):
                waiting[_u].set()
                await _orig(target)
            m.wait_until_window = waits

        async def clock():
            """Once every miner has trained and waits: the ghosts' uploads appear (copies of miner 4's payload, one
            of them malformed), the next window's first block is stamped `now`, and the chain moves on."""
            await asyncio.gather(*(e.wait() for e in waiting.values()))
            pay = {k: (t.clone() if torch.is_tensor(t) else t) for k, t in miners[4].engine.own_payload().items()}
            pay["metadata"] = {"window": w}
            bad = dict(pay)
            name = next(k for k in pay if k.endswith("vals") and pay[k].numel() > 8)
            bad[name] = torch.full_like(pay[name].float(), float("nan"))
            bad[name[:-4] + "quant_params"] = None
            for u, c in ghosts.items():
                await c.put(state_dict=bad if u == 6 else pay, uid=str(u), window=w, key="gradient", local=False)
            chain.genesis = _time.time() - (w + 1) * bpw * chain.block_time
            t_open = datetime.fromtimestamp(chain.block_timestamp((w + 1) * bpw), tz=timezone.utc)
            delta = timedelta(seconds=miners[2].hparams.time_window_delta_seconds)
            store.faults[f"gradient-{w}-5-"] = ("mtime", t_open - timedelta(seconds=5))           # before the window opened
            store.faults[f"gradient-{w}-1-"] = ("mtime", t_open + delta + timedelta(seconds=5))   # after it closed
            store.faults[f"gradient-{w}-6-"] = ("mtime", t_open + timedelta(seconds=1))
            chain._manual_block = (w + 1) * bpw
            for m in miners.values():
                m._on_block(chain.block)

        res, _ = await asyncio.gather(asyncio.gather(*(m.run_window(w) for m in miners.values())), clock())
        for r in res:                                      # peer 5's upload carries a stamp from before the window opened
            assert r["skipped_uids"] == [5] and r["global_step"] == 1, r
        for u in (2, 3, 4):                               # the real uploads were made after the window had opened
            key = next(k for (b, k) in store.objects if k.startswith(f"gradient-{w}-{u}-"))
            stamp = next(v_[1] for (b, k), v_ in store.objects.items() if k == key)
            assert stamp.timestamp() >= chain.block_timestamp((w + 1) * bpw) - 1e-3
        # the validator: gather list [2, 3]; evaluation peers are everybody who uploads
        v.config.local = False
        v.hparams.blocks_per_window, v.hparams.uids_per_window = bpw, 6
        v.loop = asyncio.get_running_loop()
        v.comms.commitments = await v.comms.get_commitments()
        v.gather_timeout = 3
        await v.dataset_manager.initialize_datasets(0)
        v.set_dataloader(validator=True)
        v.current_window, v.comms.current_window, v.sync_window = w + 1, w + 1, w
        slashed = {"missing": [], "invalid": []}
        for kind, name in (("missing", "slash_for_missing_gradient"), ("invalid", "slash_for_invalid_gradient")):
            def spy(uid, *a, _orig=getattr(v, name), _kind=kind):
                slashed[_kind].append((uid, float(v.final_scores[uid])))
                _orig(uid, *a)
                slashed[_kind][-1] += (float(v.final_scores[uid]),)
            setattr(v, name, spy)
        for u in (1, 5, 6):
            v.final_scores[u] = 1.0
        out = await v.run_window()
        assert sorted(out["gathered"]) == [2, 3]
        scored = sorted(r["uid"] for r in out["scored"])
        assert scored == [2, 3, 4], out["scored"]          # 4 is on nobody's gather list and is scored from its own upload
        # too early / too late: the score is scaled by the missing-gradient rate; malformed: zeroed
        assert sorted(slashed["missing"]) == [(1, 1.0, pytest.approx(0.75)), (5, 1.0, pytest.approx(0.75))]
        assert slashed["invalid"] == [(6, 1.0, 0.0)]
        assert {1, 5, 6} <= v.evaluated_uids
        for n in [*miners.values(), v]:
            n.metrics_logger.close()
        import json as _json
        slashes = [_json.loads(l) for l in (cwd_tmp / "metrics.jsonl").read_text().splitlines() if "validator_slash" in l]
        assert any(r["tags"].get("reason_code") == "invalid_gradient" and r["tags"].get("eval_uid") == "6" for r in slashes)
    run(go())


def test_validator_leaves_the_evaluation_loop_when_the_window_changes(cwd_tmp):
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        miners = [_node(Miner, Miner.miner_config, ["--uid", str(u), "--peers", "2", "3"], store, chain) for u in (2, 3)]
        for n in miners + [v]:
            n.loop = asyncio.get_running_loop()
            n.comms.commitments = await n.comms.get_commitments()
            n.comms.peers = [2, 3]
            n.gather_timeout = 5
            await n.dataset_manager.initialize_datasets(0)
        for m in miners:
            m.set_dataloader()
            m.current_window = m.comms.current_window = 1
        v.set_dataloader(validator=True)
        await asyncio.gather(*(m.run_window(1) for m in miners))
        v.current_window, v.comms.current_window, v.sync_window = 2, 1, 1
        v.config.local = False                         # the loop watches the clock only outside local mode
        v.hparams.uids_per_window = 2
        fetched = []
        orig = v.fetch_eval_gradient

        async def fetch(uid, tmin, tmax):
            fetched.append(uid)
            v.current_window = 3                       # the chain moves on while the first uid is being scored
            return await orig(uid, None, None)
        v.fetch_eval_gradient = fetch
        v.query_block_timestamp = lambda block: None   # no acceptance window: this test is about the loop exit
        out = await v.run_window()
        assert len(fetched) == 1 and len(out["scored"]) == 1 and out["global_step"] == 1
    run(go())


def test_shard_schedule_swaps_and_resets_with_the_global_step():
    from neurons.trainer import Trainer

    calls = []

    async def init(idx):
        calls.append(("init", idx))

    async def swap():
        calls.append(("swap",))

    t = Trainer.__new__(Trainer)
    t.hparams = SimpleNamespace(outer_steps_per_shard=10, shard_reset_outer_step=35, anneal_mode={})
    t.dataset_manager = SimpleNamespace(initialize_datasets=init, swap_datasets=swap)
    t.set_dataloader = lambda validator=False: calls.append(("loader", validator))
    t.local_rank = 0

    async def go():
        t.global_step = 12
        await t.init_shard_schedule()
        assert calls == [("init", 1), ("loader", False)] and (t._shard_epoch, t._shard_index) == (0, 1)
        calls.clear()
        t.global_step = 19
        assert not await t.maybe_switch_shard(5) and calls == []
        t.global_step = 20                                             # next shard of the same epoch: swap
        assert await t.maybe_switch_shard(6) and calls == [("swap",), ("loader", False)] and t._shard_index == 2
        calls.clear()
        t.global_step = 36                                             # past the reset step: schedule re-opened at shard 0
        assert await t.maybe_switch_shard(7, validator=True)
        assert calls == [("init", 0), ("loader", True)] and (t._shard_epoch, t._shard_index) == (1, 0)
        calls.clear()
        t.hparams.anneal_mode = {"enabled": True}
        t.global_step = 80
        assert not await t.maybe_switch_shard(8) and calls == []        # anneal mode stays on its shard
    run(go())


def test_validator_state_round_trip(cwd_tmp):
    async def go():
        store, chain = MemoryStore(), StaticChain(n=4, manual=True)
        v = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        v.global_step = 7
        v.final_scores[2], v.gradient_scores[3], v.weights[2] = 0.25, -0.5, 1.0
        v.binary_moving_averages[3], v.sync_scores[2], v.binary_indicator_scores[2] = 0.75, 0.9, 1.0
        v.openskill_ratings[2] = v.openskill_model.rating(mu=31.0, sigma=4.0, name="2")
        v.naughty_peers, v.consecutive_negative_count = {3: 5}, {2: 1}
        await v.save_state()
        w = _node(Validator, Validator.validator_config, ["--uid", "0", "--peers", "2", "3"], store, chain)
        w.state_path = v.state_path
        w.load_state()
        assert w.global_step == 7 and w.naughty_peers == {3: 5} and w.consecutive_negative_count == {2: 1}
        for name in ("final_scores", "gradient_scores", "weights", "binary_moving_averages", "sync_scores",
                     "binary_indicator_scores"):
            assert torch.equal(getattr(w, name), getattr(v, name).float()), name
        assert w.openskill_ratings[2].mu == pytest.approx(31.0) and w.openskill_ratings[2].sigma == pytest.approx(4.0)
        # a state file of another metagraph size is ignored tensor by tensor, an unreadable one entirely
        w.final_scores = torch.zeros(3)
        w.load_state()
        assert w.final_scores.shape == (3,) and float(w.final_scores.sum()) == 0.0
        with open(v.state_path, "wb") as f:
            f.write(b"not a checkpoint")
        w.global_step = 1
        w.load_state()
        assert w.global_step == 1
        torch.save([1, 2, 3], v.state_path)                      # readable, but not a state dictionary
        w.load_state()
        assert w.global_step == 1
        # only rank 0 writes the file; nothing half-written is left beside it
        os.remove(v.state_path)
        v.is_master = False
        await v.save_state()
        assert not os.path.exists(v.state_path)
        v.is_master = True
        await v.save_state()
        assert os.path.exists(v.state_path) and not [f for f in os.listdir(".") if ".tmp" in f]
    run(go())
