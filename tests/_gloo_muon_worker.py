"""Worker for test_muon.py: sharded Muon on dim-0 sharded DTensor parameters (gloo, 2 ranks)."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torch.distributed.device_mesh import init_device_mesh  # noqa: E402
from torch.distributed.tensor import Shard, distribute_tensor  # noqa: E402

from templar_b200.muon import Muon  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    mesh = init_device_mesh("cpu", (world,))
    torch.manual_seed(0)
    shapes = [(64, 32), (32, 96), (128, 64)]
    full_w = [torch.randn(*s) for s in shapes]
    full_g = [[torch.randn(*s) for s in shapes] for _ in range(2)]
    bias, bias_g = torch.randn(16), [torch.randn(16) for _ in range(2)]

    # sharded: every rank holds rows [rank * n / world, (rank + 1) * n / world) of each matrix
    params = [torch.nn.Parameter(distribute_tensor(w.clone(), mesh, [Shard(0)])) for w in full_w]
    aux = torch.nn.Parameter(bias.clone())
    opt = Muon([dict(params=params, use_muon=True, lr=0.03, weight_decay=0.01),
                dict(params=[aux], use_muon=False, lr=1e-3)])
    # single rank, full matrices, same class (plain tensors take the local path)
    ref_params = [torch.nn.Parameter(w.clone()) for w in full_w]
    ref_aux = torch.nn.Parameter(bias.clone())
    ref = Muon([dict(params=ref_params, use_muon=True, lr=0.03, weight_decay=0.01),
                dict(params=[ref_aux], use_muon=False, lr=1e-3)])
    for step in range(2):
        for p, q, g in zip(params, ref_params, full_g[step]):
            p.grad = distribute_tensor(g.clone(), mesh, [Shard(0)])
            q.grad = g.clone()
        aux.grad, ref_aux.grad = bias_g[step].clone(), bias_g[step].clone()
        opt.step()
        ref.step()
    worst = moved = 0.0
    for p, q, w in zip(params, ref_params, full_w):
        got = p.detach().full_tensor()
        worst = max(worst, float((got - q.detach()).abs().max()))
        moved = max(moved, float((got - w).abs().max()))
    out = {"max_diff": worst, "moved": moved, "aux_diff": float((aux.detach() - ref_aux.detach()).abs().max())}

    # window engine with Muon as the inner optimizer: 2 ranks (each its own micro-batch) == 1 rank (both)
    from templar_b200.models.llama import ModelArgs, build_model
    from templar_b200.parallel.window_engine import EngineConfig, WindowEngine

    args = ModelArgs(dim=64, n_layers=2, n_heads=2, vocab_size=128, intermediate_size=128, max_seq_len=32)
    cfg = EngineConfig(inner_optimizer="muon", inner_lr=0.02, muon_momentum=0.9)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 128, (2, world, 2, 33), generator=g)          # [step, rank, batch, seq + 1]
    eng = WindowEngine(build_model(args, seed=3), cfg, rank=rank, world_size=world)
    one = WindowEngine(build_model(args, seed=3), cfg)
    for step in range(2):
        t = toks[step, rank]
        eng.micro_step(t[:, :-1], t[:, 1:], 1.0)
        eng.optimizer_step()
        for r in range(world):
            t = toks[step, r]
            one.micro_step(t[:, :-1], t[:, 1:], 1.0 / world)
        one.optimizer_step()
    full, ref = eng.full_state_dict(), one.full_state_dict()             # fp32 master weights by name (collective)
    d = torch.cat([(full[k] - ref[k]).abs().reshape(-1) for k in ref])
    out["engine_exact_frac"] = float((d < 1e-6).float().mean())
    out["engine_max_diff"] = float(d.max())
    mine, theirs = dict(eng.model.named_parameters()), dict(one.model.named_parameters())
    out["engine_compute_diff"] = max(float((mine[k].detach().float() - theirs[k].detach().float()).abs().max()) for k in theirs)
    start = dict(build_model(args, seed=3).named_parameters())
    out["engine_moved"] = max(float((ref[k] - start[k].detach()).abs().max()) for k in start)
    res = [None] * world
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
