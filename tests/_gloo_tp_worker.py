"""Worker for test_distributed_cpu.py: tensor-parallel LLaMA sharding logic on CPU (gloo, fp32) against the
unsharded model.  The projections run through CollectiveTensorParallel (torch.distributed collectives)."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.models.llama_tp import TPLlamaModel  # noqa: E402
from templar_b200.parallel.tensor_parallel import CollectiveTensorParallel  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    torch.manual_seed(0)
    args = ModelArgs(dim=128, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=500, intermediate_size=256, max_seq_len=64)
    B, S = 2, 64
    full = build_model(args, device="cpu", dtype=torch.float32, seed=9)
    model = TPLlamaModel(args, rank, world)
    model.freqs_cis = full.freqs_cis
    model.load_from_full(full)
    model.attach(CollectiveTensorParallel(B * S, args.dim, rank, world))
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, args.vocab_size, (B, S + 1), generator=g)
    labels = toks[:, 1:].clone()
    labels[0, :5] = -100
    loss = model.loss(toks[:, :-1], labels)
    loss.backward()
    model.reduce_replicated_grads()
    ref = full.loss(toks[:, :-1], labels)
    ref.backward()
    fg = {n: p.grad for n, p in full.named_parameters()}
    worst = 0.0
    for name, p in model.named_parameters():
        f = fg[name]
        if name in ("tok_embeddings.weight", "output.weight"):
            n = model.vocab_padded // world
            pad = torch.zeros(model.vocab_padded, f.shape[1])
            pad[: f.shape[0]] = f
            f = pad[rank * n:(rank + 1) * n]
        elif name.endswith(("wq.weight", "wk.weight", "wv.weight", "w1.weight", "w3.weight")):
            n = f.shape[0] // world
            f = f[rank * n:(rank + 1) * n]
        elif name.endswith(("wo.weight", "w2.weight")):
            n = f.shape[1] // world
            f = f[:, rank * n:(rank + 1) * n]
        worst = max(worst, ((p.grad - f).norm() / (f.norm() + 1e-12)).item())
    # the same step with activation checkpointing: identical loss and gradients
    g1 = {n: p.grad.clone() for n, p in model.named_parameters()}
    for p in model.parameters():
        p.grad = None
    model.activation_checkpointing = True
    loss2 = model.loss(toks[:, :-1], labels)
    loss2.backward()
    model.reduce_replicated_grads()
    ckpt_diff = max(float((p.grad - g1[n]).abs().max()) for n, p in model.named_parameters())
    out = {"loss": float(loss), "ref_loss": float(ref), "worst_rel": worst, "vocab_padded": model.vocab_padded,
           "ckpt_loss_diff": abs(float(loss2) - float(loss)), "ckpt_grad_diff": ckpt_diff}
    res = [None] * world
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
