"""Worker for test_hsdp_cpu.py: 4 gloo ranks run the same two windows as one sharded group of four (the known-good
layout), as two replicas of two shards (hybrid) and as four replicas of one rank (plain data parallelism); the
weights and the losses must agree."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine  # noqa: E402
from templar_b200.utils.synthetic import synthetic_payload  # noqa: E402

ARGS = ModelArgs(dim=128, n_layers=2, n_heads=2, vocab_size=256, intermediate_size=256, max_seq_len=32)


def run(grank, world, replicas, groups, shard_params=False, muon=False):
    shards = world // replicas
    shard_group, rep_group = groups[replicas]
    model = build_model(ARGS, seed=3)
    extra = dict(inner_optimizer="muon", inner_lr=0.02, muon_momentum=0.9) if muon else {}
    eng = WindowEngine(model, EngineConfig(shard_params=shard_params, max_peers=2, **extra), rank=grank % shards,
                       world_size=shards, group=shard_group, replicate_group=rep_group, replicate_size=replicas)
    eng.REPLICATE_BUCKET = 10_000                  # several all-reduce buckets per step even on this small model
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, 256, (2, 2, world, 2, 33), generator=g)           # [window, step, rank, batch, seq + 1]
    losses = []
    for w in range(2):
        eng.snapshot()
        for step in range(2):
            t = toks[w, step, grank]
            losses.append(float(eng.micro_step(t[:, :-1], t[:, 1:], 1.0)))
            eng.optimizer_step()
        eng.compress()
        eng.merge_own_payload()
        eng.load_peer_payload(1, synthetic_payload(eng.layout, 5 + w))
        eng.outer_step(2)
    own = eng.own_val.clone()
    state = eng.full_state_dict()
    return losses, {k: v.clone() for k, v in state.items() if v.is_floating_point()}, own


def trainer_case(grank, world, replicas):
    """Through the neurons' own path: ``Trainer.engine_topology`` / ``attach_engine`` from ``torchtitan.dp_replicate``,
    two inner steps, then the public ``outer_step`` with a gather result that only the master rank holds."""
    import asyncio
    import threading
    from types import SimpleNamespace

    import templar_b200 as tplr
    from neurons.trainer import Trainer
    from templar_b200 import compress as C
    from templar_b200.distributed import dist_helper

    dist_helper.rank, dist_helper.world_size = grank, world
    t = Trainer()
    t.hparams = SimpleNamespace(inner_steps=2, outer_learning_rate=0.4, topk_compression=8, use_dct=True,
                                optimizer={"type": "adamw", "adamw": {"learning_rate": 1e-3}}, anneal_mode={},
                                tokenizer=SimpleNamespace(pad_token_id=0), torchtitan={"dp_replicate": replicas},
                                gather_peer_count=2, reserve_peer_count=0)
    t.tokenizer = t.hparams.tokenizer
    t.device, t.rank, t.world_size, t.is_master = torch.device("cpu"), grank, world, grank == 0
    t.model = build_model(ARGS, seed=3)
    t.attach_engine(heap=t.make_heap())
    t.init_optimizers_schedulers()
    t.sampler = SimpleNamespace(grad_accum_steps=2)
    t.stop_event = threading.Event()
    t.current_window = 10
    g = torch.Generator().manual_seed(100 + grank)
    loader = [torch.randint(0, 256, (2, 16), generator=g) for _ in range(4)]
    t.engine.snapshot()
    out = asyncio.run(t.inner_steps(loader, step_window=10))
    gather = None
    if grank == 0:
        tr, comp = C.ChunkingTransformer(t.model, 64), C.TopKCompressor()
        sd = {}
        gg = torch.Generator().manual_seed(7)
        for n, p in t.model.named_parameters():
            idxs, vals = [], []
            for j in range(2):
                i, v, _, _ = comp.compress(tr.encode(torch.randn(p.shape, generator=gg) * 1e-3, use_dct=True), 8)
                idxs.append(i), vals.append(v)
            sd[n + "idxs"], sd[n + "vals"], sd[n + "quant_params"] = idxs, vals, [None, None]
        gather = SimpleNamespace(state_dict=SimpleNamespace(**sd), uids=[0, 1], skipped_uids=[], success_rate=1.0)
    tplr.neurons.outer_step(t.model, t.outer_optimizer, gather_result=gather, transformer=None, compressor=None, xshapes=None,
                            totalks=None, device="cpu", is_master=grank == 0, world_size=world, use_dct=True)
    state = t.engine.full_state_dict()
    topo = t.engine_topology()
    return out["inner_steps"], {k: v.clone() for k, v in state.items() if v.is_floating_point()}, \
        [topo["shard_rank"], topo["shard_world"], topo["replicas"], t.engine.replica]


def main():
    grank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    groups = {1: (None, None)}
    for replicas in (2, 4):
        shards = world // replicas
        sg = [dist.new_group(list(range(r * shards, (r + 1) * shards))) for r in range(replicas)]
        rg = [dist.new_group(list(range(s, world, shards))) for s in range(shards)]
        groups[replicas] = (sg[grank // shards] if shards > 1 else None, rg[grank % shards])
    out = {}
    for tag, kw in (("adamw", {}), ("muon", {"muon": True})):
        ref_l, ref_s, ref_own = run(grank, world, 1, groups, **kw)
        start = build_model(ARGS, seed=3).state_dict()
        out[tag + "_moved"] = max(float((ref_s[k] - start[k]).abs().max()) for k in ref_s)
        for name, replicas, shard_params in (("hybrid", 2, False), ("hybrid_sharded_params", 2, True), ("replicated", 4, False)):
            l, s, own = run(grank, world, replicas, groups, shard_params=shard_params, **kw)
            out[f"{tag}_{name}"] = {"loss": max(abs(a - b) for a, b in zip(l, ref_l)),
                                    "weights": max(float((s[k] - ref_s[k]).abs().max()) for k in ref_s),
                                    "payload": float((own - ref_own).abs().max())}
    steps1, ref_s, _ = trainer_case(grank, world, 1)
    start = build_model(ARGS, seed=3).state_dict()
    out["trainer_moved"] = max(float((ref_s[k] - start[k]).abs().max()) for k in ref_s)
    for replicas in (2, 4):
        steps, s_, topo = trainer_case(grank, world, replicas)
        out[f"trainer_{replicas}"] = {"steps": [steps1, steps], "topology": topo,
                                      "weights": max(float((s_[k] - ref_s[k]).abs().max()) for k in ref_s)}
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if grank == 0:
        print("RESULT " + json.dumps(gathered))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
