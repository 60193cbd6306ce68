"""Worker for test_fsdp_cpu.py: two windows of the engine with sharded parameters on 2 gloo ranks against the
engine that keeps weights and gradients whole on every rank; same data, same peers."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine  # noqa: E402
from templar_b200.utils.synthetic import synthetic_payload  # noqa: E402


def run(rank, world, shard_params, ckpt=False, quantize=False, muon=False):
    args = ModelArgs(dim=128, n_layers=3, n_heads=2, vocab_size=256, intermediate_size=256, max_seq_len=32)
    model = build_model(args, seed=3)
    model.activation_checkpointing = ckpt
    extra = dict(inner_optimizer="muon", inner_lr=0.02, muon_momentum=0.9) if muon else {}
    eng = WindowEngine(model, EngineConfig(shard_params=shard_params, max_peers=2, quantize=quantize, **extra), rank=rank,
                       world_size=world)
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, 256, (2, 2, 2, world, 2, 33), generator=g)       # [window, step, micro, rank, batch, seq + 1]
    losses = []
    for w in range(2):
        eng.snapshot()
        for step in range(2):
            for mb in range(2):
                t = toks[w, step, mb, rank]
                losses.append(float(eng.micro_step(t[:, :-1], t[:, 1:], 0.5)))
            eng.optimizer_step()
        eng.compress()
        eng.merge_own_payload()
        eng.load_peer_payload(1, synthetic_payload(eng.layout, 5 + w))
        eng.outer_step(2)
    with torch.no_grad():
        t = toks[0, 0, 0, 0]
        losses.append(float(model.loss(t[:, :-1], t[:, 1:])))
    state = eng.full_state_dict()
    return losses, {k: v.clone() for k, v in state.items() if v.is_floating_point()}, eng


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    ref_l, ref_s, ref_e = run(rank, world, False)
    out = {}
    for name, kw in (("fsdp", {}), ("fsdp_ckpt", {"ckpt": True})):
        l, s, e = run(rank, world, True, **kw)
        out[name] = {"loss": max(abs(a - b) for a, b in zip(l, ref_l)),
                     "weights": max(float((s[k] - ref_s[k]).abs().max()) for k in ref_s),
                     "moved": max(float((ref_s[k] - v).abs().max()) for k, v in
                                  build_model(ModelArgs(dim=128, n_layers=3, n_heads=2, vocab_size=256,
                                                        intermediate_size=256, max_seq_len=32), seed=3).state_dict().items()
                                  if k in ref_s),
                     "shard_elems": e.store.n_shard, "total": e.layout.total, "gathers": e.store.gather.gathers,
                     "full_buffers": e.store.compute is None and e.store.grad is None}
    ql, qs, _ = run(rank, world, False, quantize=True)
    l, s, _ = run(rank, world, True, quantize=True)
    out["fsdp_quant"] = {"loss": max(abs(a - b) for a, b in zip(l, ql)),
                         "weights": max(float((s[k] - qs[k]).abs().max()) for k in qs)}
    ml, ms, _ = run(rank, world, False, muon=True)
    l, s, _ = run(rank, world, True, muon=True)
    out["fsdp_muon"] = {"loss": max(abs(a - b) for a, b in zip(l, ml)),
                        "weights": max(float((s[k] - ms[k]).abs().max()) for k in ms),
                        "vs_adamw": max(float((ms[k] - ref_s[k]).abs().max()) for k in ms)}
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print("RESULT " + json.dumps(gathered))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
