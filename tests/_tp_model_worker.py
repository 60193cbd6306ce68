"""Worker launched by test_gpu_multi.py under torchrun: tensor-parallel LLaMA vs the unsharded model on one GPU."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.models.llama_tp import TPLlamaModel  # noqa: E402
from templar_b200.ops import functional as OF  # noqa: E402
from templar_b200.parallel.symmetric import SymmetricHeap  # noqa: E402
from templar_b200.parallel.tensor_parallel import TensorParallel  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    heap = SymmetricHeap.create(dev, rank, world, timeout_s=20.0)
    args = ModelArgs(dim=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1000, intermediate_size=1024, max_seq_len=256)
    B, S = 2, 256
    full = build_model(args, device=dev, dtype=torch.bfloat16, seed=9)
    model = TPLlamaModel(args, rank, world).to(device=dev, dtype=torch.bfloat16)
    model.freqs_cis = full.freqs_cis
    model.load_from_full(full)
    model.attach(TensorParallel(heap, rows=B * S, width=args.dim))
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, args.vocab_size, (B, S + 1), generator=g).to(dev)
    loss = model.loss(toks[:, :-1], toks[:, 1:])
    loss.backward()
    model.reduce_replicated_grads()
    ref = full.loss(toks[:, :-1], toks[:, 1:])
    ref.backward()
    torch.cuda.synchronize()
    model.tp.check()
    # the oracle for both bf16 pipelines: the same model in fp32 (PyTorch ops; fp32 operands never reach the own GEMM)
    oracle = build_model(args, device=dev, dtype=torch.float32, seed=None)
    oracle.load_state_dict({k: (v.float() if v.is_floating_point() else v) for k, v in full.state_dict().items()})
    o_loss = oracle.loss(toks[:, :-1], toks[:, 1:])
    o_loss.backward()
    out = {"loss": float(loss), "ref_loss": float(ref), "oracle_loss": float(o_loss),
           "status": int(OF.status_word(dev).item())}
    fg = {n: p.grad for n, p in full.named_parameters()}
    og = {n: p.grad for n, p in oracle.named_parameters()}
    n_sh = world

    def shard(name, f):
        if name in ("tok_embeddings.weight", "output.weight"):
            n = model.vocab_padded // n_sh
            pad = torch.zeros(model.vocab_padded, f.shape[1], device=f.device)
            pad[: f.shape[0]] = f
            return pad[rank * n:(rank + 1) * n]
        if name.endswith(("wq.weight", "wk.weight", "wv.weight", "w1.weight", "w3.weight")):
            n = f.shape[0] // n_sh
            return f[rank * n:(rank + 1) * n]
        if name.endswith(("wo.weight", "w2.weight")):
            n = f.shape[1] // n_sh
            return f[:, rank * n:(rank + 1) * n]
        return f

    worst = worst_ratio = 0.0
    worst_name = ""
    for name, p in model.named_parameters():
        want = shard(name, og[name].float())
        single = shard(name, fg[name].float())
        denom = want.norm() + 1e-12
        rel_tp = ((p.grad.float() - want).norm() / denom).item()           # tensor-parallel bf16 vs fp32
        rel_1 = ((single - want).norm() / denom).item()                    # single-GPU bf16 vs fp32
        out.setdefault("rel", {})[name] = [rel_tp, rel_1]
        worst = max(worst, rel_tp)
        ratio = rel_tp / max(rel_1, 1e-3)                                   # floor: tensors whose bf16 error is tiny
        if ratio > worst_ratio:
            worst_ratio, worst_name = ratio, name
    out["worst_rel"], out["worst_ratio"], out["worst_tensor"] = worst, worst_ratio, worst_name
    heap.barrier()
    torch.cuda.synchronize()
    heap.check_guards()           # no store of any rank ran past the end of a symmetric block of this rank
    out["guards_ok"] = True
    res = [None] * world
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
