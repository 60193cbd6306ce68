"""Validator scoring throughput on the 1B model: for each of 8 peers' compressed payloads, the loss of a
batch before and after applying that peer's decoded update, then the restore of the weights.

    python -m templar_b200.bench.config5_validator --peers 8 --iters 3                       (one GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
        -m templar_b200.bench.config5_validator --peers 8 --iters 3 [--shard-params]          (sharded engine)

What is timed per peer (CUDA events on every rank, max over ranks): forward-only loss on ``--batch`` x ``--seq-len``
tokens per GPU with the window's snapshot weights, ``WindowEngine.apply_single_peer`` (every rank pulls the peer's
packed payload from the slot of the rank that holds it, unpacks, clips to the median norm, inverse-DCTs and updates
the master and bf16 weights of its own shard in one kernel), the forward-only loss again, and
``WindowEngine.restore``.  The four phases are also reported separately.  This is the reference's evaluation
step (neurons/validator.py:3563-3770 and :1974-2179: loss before, apply, loss after, restore) without its per-tensor
Python loop on rank 0; ``python -m baseline.reference_config5`` times the unmodified reference on the same
payloads.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1B")
    ap.add_argument("--peers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--shard-params", action="store_true")
    a = ap.parse_args()

    from ..models.llama import PRESETS, build_model
    from ..ops import native
    from ..parallel.symmetric import SymmetricHeap
    from ..parallel.window_engine import EngineConfig, WindowEngine
    from ..utils.synthetic import synthetic_payload

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    heap = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        heap = SymmetricHeap.create(dev, rank, world, timeout_s=30.0)
    args = PRESETS[a.model]
    model = build_model(args, device=dev, dtype=torch.bfloat16, seed=0)
    eng = WindowEngine(model, EngineConfig(topk=a.topk, use_dct=True, max_peers=a.peers, shard_params=a.shard_params),
                       device=dev, rank=rank, world_size=world, heap=heap)
    for j in range(a.peers):                                   # peer j's payload lives on rank j % world
        owner, slot = eng.slot_of(j)
        if owner == rank:
            eng.load_peer_payload(slot, synthetic_payload(eng.layout, 500 + j, device=dev))
    eng._barrier()
    g = torch.Generator().manual_seed(5 + rank)
    tok = torch.randint(0, args.vocab_size, (a.batch, a.seq_len + 1), generator=g).to(dev)
    x, y = tok[:, :-1], tok[:, 1:]
    eng.snapshot()
    median = eng.compute_peer_norms(a.peers).clone()       # per-tensor median norm over the gathered peers
    phases = ("loss_before", "apply", "loss_after", "restore")

    def score_all(marks=None):
        out = []

        def mark():
            if marks is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)

        mark()
        for j in range(a.peers):
            with torch.no_grad():
                before = model.loss(x, y)
                mark()
                eng.apply_single_peer(j, lr=1.0, median=median)
                mark()
                after = model.loss(x, y)
                mark()
            eng.restore()
            mark()
            out.append(before - after)
        return torch.stack(out)

    score_all()
    torch.cuda.synchronize()
    times, per_phase = [], []
    for _ in range(a.iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        l0 = native.launch_count
        marks = []
        deltas = score_all(marks)
        torch.cuda.synchronize()
        launches = native.launch_count - l0
        seg = [marks[i].elapsed_time(marks[i + 1]) for i in range(len(marks) - 1)]
        t = torch.tensor([sum(seg)] + [sum(seg[p::4]) for p in range(4)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t[0]))
        per_phase.append([float(v) for v in t[1:]])
    order = sorted(range(len(times)), key=lambda i: times[i])
    mid = order[len(order) // 2]
    ms = times[mid]
    status = eng.check_status()
    if rank == 0:
        rec = {"case": "config5_validator_scoring", "impl": "ours", "model": a.model, "world": world, "peers": a.peers,
               "ms_per_peer": ms / a.peers, "peers_per_s": a.peers / ms * 1e3,
               "ms_per_peer_by_phase": {n: round(v / a.peers, 3) for n, v in zip(phases, per_phase[mid])},
               "tokens_per_eval_per_gpu": a.batch * a.seq_len, "own_kernel_launches": launches,
               "sharding": "weights, gradients and optimizer state sharded" if a.shard_params else
               ("optimizer state sharded, weights whole" if world > 1 else "single GPU"),
               "kernel_status": status, "loss_delta_first_peer": float(deltas[0]), "dtype": "bf16",
               "data": "synthetic uniform-random tokens, random-init weights, seeded synthetic peer payloads"}
        print(json.dumps(rec))
    if world > 1:
        heap.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
