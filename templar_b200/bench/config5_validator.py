"""Validator scoring throughput on the 1B model: for each of 8 peers' compressed payloads, the loss of a
batch before and after applying that peer's decoded update, then the restore of the weights.

    python -m templar_b200.bench.config5_validator --peers 8 --iters 3

What is timed per peer (CUDA events, one GPU): forward-only loss on ``--batch`` x ``--seq-len`` tokens with
the window's snapshot weights, ``WindowEngine.apply_single_peer`` (unpack + clip to the median norm +
inverse DCT + update of master and bf16 weights in one kernel), the forward-only loss again, and
``WindowEngine.restore``.  This is the reference's evaluation step (neurons/validator.py:3563-3770 and
:1890-2080: loss before, apply, loss after, restore) without its per-tensor Python loop.
"""

from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1B")
    ap.add_argument("--peers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()

    from ..models.llama import PRESETS, build_model
    from ..ops import native
    from ..parallel.window_engine import EngineConfig, WindowEngine
    from ..utils.synthetic import synthetic_payload

    dev = torch.device("cuda", 0)
    args = PRESETS[a.model]
    model = build_model(args, device=dev, dtype=torch.bfloat16, seed=0)
    eng = WindowEngine(model, EngineConfig(topk=a.topk, use_dct=True, max_peers=a.peers), device=dev)
    for j in range(a.peers):
        eng.load_peer_payload(j, synthetic_payload(eng.layout, 500 + j, device=dev))
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, args.vocab_size, (a.batch, a.seq_len + 1), generator=g).to(dev)
    x, y = tok[:, :-1], tok[:, 1:]
    eng.snapshot()
    median = eng.compute_peer_norms(a.peers).clone()       # per-tensor median norm over the gathered peers

    def score_all():
        out = []
        for j in range(a.peers):
            with torch.no_grad():
                before = model.loss(x, y)
                eng.apply_single_peer(j, lr=1.0, median=median)
                after = model.loss(x, y)
            eng.restore()
            out.append(before - after)
        return torch.stack(out)

    score_all()
    torch.cuda.synchronize()
    times = []
    for _ in range(a.iters):
        l0 = native.launch_count
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        deltas = score_all()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        launches = native.launch_count - l0
    times.sort()
    ms = times[len(times) // 2]
    rec = {"case": "config5_validator_scoring", "model": a.model, "peers": a.peers, "ms_per_peer": ms / a.peers,
           "peers_per_s": a.peers / ms * 1e3, "tokens_per_eval": a.batch * a.seq_len, "own_kernel_launches": launches,
           "kernel_status": eng.check_status(), "loss_delta_first_peer": float(deltas[0]), "dtype": "bf16",
           "data": "synthetic uniform-random tokens, random-init weights, seeded synthetic peer payloads"}
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
