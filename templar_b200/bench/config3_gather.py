"""Compressed-gradient gather microbenchmark: compress, all-peer gather, decode, mean, sign update.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
        -m templar_b200.bench.config3_gather --model 1B --topk 16 32 64

Every rank is one peer and holds fp32 momentum-like tensors with the parameter shapes of ``--model``
(seeded N(0, 1e-3)).  Timed per k (CUDA events, max over ranks, median of ``--iters``):

  ours       ``compress`` (EF + chunk-64 DCT + top-k + 12-bit pack, one kernel) writing the payload into
             this rank's slot of the symmetric heap, one heap barrier, then ``outer_step`` in sign mode:
             ONE kernel per rank pulls every peer's packed payload over NVLink for the chunks this rank
             owns, unpacks, clips, means, inverse-DCTs and updates, and the bf16 result is pushed to all
             ranks.  No intermediate all-gather buffer exists.
  reference  the UNMODIFIED reference on the same box (``--reference``; baseline/reference_config3.py): its own
             ``ChunkingTransformer.encode`` + ``TopKCompressor.compress`` per tensor, NCCL ``all_gather`` of the packed
             tensors, and its own ``outer_step`` (rank 0 clips, batch-decompresses and inverse-transforms, broadcasts
             the dense gradient, every rank applies SGD).  Slow: about a second per round.

Reports ms, payload GB/s over NVLink, and the fraction of the roofline max(HBM bytes / measured copy
bandwidth, NVLink bytes / 770 GB/s).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1B")
    ap.add_argument("--topk", type=int, nargs="+", default=[16, 32, 64])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--reference", action="store_true")
    a = ap.parse_args()

    from ..models.llama import PRESETS, build_model
    from ..ops.microbench import peaks
    from ..parallel.symmetric import SymmetricHeap
    from ..parallel.window_engine import EngineConfig, WindowEngine

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    heap = SymmetricHeap.create(dev, rank, world, timeout_s=30.0) if world > 1 else None
    pk = peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    for k in a.topk:
        model = build_model(PRESETS[a.model], device=dev, dtype=torch.bfloat16, seed=0)
        eng = WindowEngine(model, EngineConfig(topk=k, use_dct=True, outer_update="sign", max_peers=world),
                           device=dev, rank=rank, world_size=world, heap=heap)
        n = eng.layout.total
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        eng.snapshot()
        # momentum-like delta: theta0 - theta = N(0, 1e-3) on this rank's shard
        eng.store.master_shard.sub_(torch.randn(eng.store.master_shard.shape, device=dev, generator=gen) * 1e-3)

        def step():
            own = None
            if heap is not None:
                own = (heap.peer_ptr(eng.own_idx, 0), heap.peer_ptr(eng.own_val, 0))
            eng.compress(own_slot_ptrs=own)
            if world > 1:
                eng._barrier()
            eng.outer_step(world, include_own=True)

        def timed(fn):
            ts = []
            for i in range(a.iters + 2):
                flush.add_(1.0)
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                if i >= 2:
                    ts.append(float(t.item()))
            return _median(ts)

        ms = timed(step)
        chunks = n // 4096
        payload = chunks * (k // 2 * 3 + 4 * k)                       # bytes of one peer's full payload
        shard = n / world
        hbm = shard * 16 + shard * 10 + world * payload / world        # compress r/w, apply r/w, payload reads of own chunks
        link = (world - 1) * payload / world                           # peers' payload bytes for the chunks this rank owns
        roof = max(hbm / (pk["hbm_gbs"] * 1e9), link / 770e9) * 1e3
        rec = {"case": "config3_gather", "model": a.model, "world": world, "topk": k, "ours_ms": ms,
               "payload_bytes_per_peer": payload, "nvlink_gbs": link / ms / 1e6, "roofline_ms": roof,
               "frac_of_roofline": roof / ms, "kernel_status": eng.check_status(), "peaks": pk["source"]}
        del eng, model
        torch.cuda.empty_cache()
        if a.reference:
            ref_step = _reference_step(a.model, k, world, rank, dev)
            rec["reference_ms"] = timed(ref_step)
            rec["reference"] = "unmodified reference install (tplr.compress + tplr.neurons.outer_step + NCCL all_gather)"
            rec["speedup"] = rec["reference_ms"] / ms
            del ref_step
            torch.cuda.empty_cache()
        if rank == 0:
            print(json.dumps(rec))
    if heap is not None:
        heap.close()
    dist.destroy_process_group()


def _reference_step(model_name, k, world, rank, dev):
    """One round of the UNMODIFIED reference (its ``ChunkingTransformer`` / ``TopKCompressor`` / ``outer_step`` with
    NCCL ``all_gather`` of the payloads), built by ``baseline/reference_config3.py`` from the install under
    ``baseline/_ref``; nothing of this package is on that path."""
    import importlib
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parents[2])
    if root not in sys.path:
        sys.path.insert(0, root)
    step, _ = importlib.import_module("baseline.reference_config3").make_step(model_name, k, world, rank, dev)
    return step


if __name__ == "__main__":
    main()
