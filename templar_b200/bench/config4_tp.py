"""Tensor-parallel training window of the 72B-class layer shapes truncated to 16 layers (about 18B parameters).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
        -m templar_b200.bench.config4_tp --steps 3 --warmup 3

One process per GPU, TP = world size.  Every rank holds its shard of the weights in bf16 plus fp32
master / AdamW / snapshot / error-feedback state for that shard (about 26 bytes per local parameter, so
the 18B model needs 58 GB per GPU at TP=8 and no further parameter sharding).  A window is ``--accum``
micro-batches of ``--micro-batch`` x ``--seq-len`` uniform-random tokens (forward + backward through the
fused all-gather->GEMM and GEMM->reduce-scatter kernels), the all-reduce of the replicated norm
gradients, fused AdamW, and the compress (chunk-64 DCT, top-32, error feedback) + outer step over the
local shards.  Timed with CUDA events, max over ranks; prints one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="18B-tp")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0: preset)")
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--accum", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--activation-checkpointing", action="store_true")
    a = ap.parse_args()

    import dataclasses

    from ..models.llama import PRESETS
    from ..models.llama_tp import TPLlamaModel
    from ..ops import functional as OF, native
    from ..parallel.symmetric import SymmetricHeap
    from ..parallel.tensor_parallel import TensorParallel
    from ..parallel.window_engine import EngineConfig, WindowEngine

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    heap = SymmetricHeap.create(dev, rank, world, timeout_s=30.0)
    args = PRESETS[a.model]
    if a.layers:
        args = dataclasses.replace(args, n_layers=a.layers)
    B, S, A = a.micro_batch, a.seq_len, a.accum
    with torch.device(dev):
        model = TPLlamaModel(args, rank, world).to(torch.bfloat16)
    model.init_weights(seed=1 + rank, buffer_device=dev)
    model.attach(TensorParallel(heap, rows=B * S, width=args.dim))
    model.activation_checkpointing = a.activation_checkpointing
    eng = WindowEngine(model, EngineConfig(topk=a.topk, use_dct=True, max_peers=1), device=dev)
    g = torch.Generator().manual_seed(77)                       # every TP rank sees the same tokens
    toks = [torch.randint(0, args.vocab_size, (B, S + 1), generator=g).to(dev) for _ in range(A)]

    def window():
        eng.snapshot()
        losses = []
        for m in range(A):
            t = toks[m]
            losses.append(eng.micro_step(t[:, :-1], t[:, 1:], 1.0 / A))
        model.reduce_replicated_grads()
        eng.optimizer_step()
        eng.compress()
        eng.outer_step(1)
        return torch.stack(losses).mean()

    for _ in range(a.warmup):
        loss = window()
    dist.barrier()
    torch.cuda.synchronize()
    l0 = native.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = window()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    model.tp.check()
    status = eng.check_status() | int(OF.status_word(dev).item())
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    if rank == 0:
        ms = float(t.item()) / a.steps
        tokens = B * S * A
        n_local = sum(p.numel() for p in model.parameters())
        print(json.dumps({
            "case": "config4_tp_window", "model": a.model, "layers": args.n_layers, "tp": world, "ms_per_window": ms,
            "tokens_per_s": tokens / ms * 1e3, "tokens_per_window": tokens, "local_params": n_local,
            "model_tflops_per_gpu": tokens / ms * 1e3 * args.flops_per_token(S) / world / 1e12,
            "loss": float(loss), "peak_mem_gib": mem, "own_kernel_launches": native.launch_count - l0,
            "kernel_status": status, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"micro_batch": B, "seq_len": S, "accum": A, "topk": a.topk, "peers": 1,
                       "activation_checkpointing": bool(a.activation_checkpointing)}}))
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
