"""Reference arm of the validator-scoring benchmark: the UNMODIFIED reference's own evaluation step.

For each of ``--peers`` synthetic peer payloads (the reference's wire format: 12-bit packed indices, uint8 value
codes, per-tensor lookup) the reference's ``Validator`` methods are called in the order of its scoring loop
(neurons/validator.py:1974-2179):

    Trainer.evaluate_model            loss on the batch with the current weights   (neurons/trainer.py:424-492)
    Validator.update_model_with_gradient   dequantise, clip to the median norm, decompress, inverse DCT, apply
                                                                                 (neurons/validator.py:3563-3738)
    Trainer.evaluate_model            loss after the apply
    Validator._restore_model_state    back to the saved weights                   (neurons/validator.py:290-302)

with ``compute_peer_val_norms`` (:3740-3770) and ``_save_model_state`` (:274-288) once before the loop.  The model is
the reference's FSDP2 torchtitan LLaMA built by its ``model_factory``; nothing of this repository's engine, models
or kernels runs.  Launch like ``bench.py --impl reference`` (torchrun for several GPUs).

    python -m baseline.reference_config5 --peers 8 --iters 2
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import sys
import time
from pathlib import Path
from types import SimpleNamespace

import torch

ROOT = Path(__file__).resolve().parents[1]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1B")
    ap.add_argument("--peers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--iters", type=int, default=2)
    a = ap.parse_args()
    a.micro_batch, a.accum = a.batch, 1
    sys.path.insert(0, str(ROOT))
    from baseline import ref_env
    from baseline.reference_bench import _hparams

    ref_env.prepare()
    import torch.distributed as dist
    import tplr
    from neurons.validator import Validator
    from tplr.distributed import dist_helper

    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0"), ("MASTER_ADDR", "127.0.0.1"),
                 ("MASTER_PORT", str(29400 + os.getpid() % 500))):
        os.environ.setdefault(k, v)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    if world > 1:
        dist_helper.init_process_group("nccl" if cuda else "gloo", timeout_minutes=30)
    vocab = 32000 if a.model != "tiny" else 512
    v = object.__new__(Validator)
    v.hparams = _hparams(a, vocab, world, os.environ.get("TPLR_REF_COMPILE", "1") == "1")
    v.hparams.eval_lr_factor = 0.2
    v.rank, v.world_size, v.local_rank, v.is_master = rank, world, local, rank == 0
    v.device, v.uid, v.current_window, v.sync_window, v.global_step = dev, 0, 100, 99, 0
    v.config = SimpleNamespace(device=str(dev), local=True)
    v.init_model(validator=False, meta=False)            # same sharding as the training benchmark: dp_shard = world
    v.tokenizer = v.hparams.tokenizer
    v.lr = float(v.hparams.outer_learning_rate)
    v.transformer = tplr.compress.ChunkingTransformer(v.model, target_chunk=v.hparams.target_chunk)
    v.compressor = tplr.compress.TopKCompressor(use_quantization=True, quantization_bins=256, quantization_range=6)
    v.xshapes, v.totalks = {}, {}
    for n, p in v.model.named_parameters():
        enc = v.transformer.encode(torch.empty(p.shape, dtype=torch.float16, device=dev), use_dct=False)
        _, _, xshape, totalk, _ = v.compressor.compress(enc, a.topk)
        v.xshapes[n], v.totalks[n] = xshape, totalk
    # the same seeded synthetic payloads as the other arm, re-keyed to the reference's dict format
    from templar_b200.parallel.flat import FlatLayout
    from templar_b200.utils.synthetic import synthetic_payload

    shapes = [(n, tuple(p.shape)) for n, p in v.model.named_parameters()]
    layout = FlatLayout(shapes, 64, a.topk, 1)
    peers = []
    for j in range(a.peers):
        idx, val = synthetic_payload(layout, 500 + j, device=dev)
        entry = {}
        for n, _ in shapes:
            i_view, v_view = layout.payload_views(idx, val, n)
            q, qp = v.compressor._quantize_values(v_view)
            entry[n + "idxs"], entry[n + "vals"], entry[n + "quant_params"] = i_view.clone(), q, qp
        peers.append(entry)
    gathered = SimpleNamespace(state_dict=SimpleNamespace(**{k: [p[k] for p in peers] for k in peers[0]}))
    g = torch.Generator().manual_seed(5 + rank)
    loader = [torch.randint(0, vocab, (a.batch, a.seq_len), generator=g)]

    async def score_all():
        clip = v.compute_peer_val_norms(gathered)
        saved = v._save_model_state()
        deltas = []
        for j in range(a.peers):
            before, nb = await v.evaluate_model(v.model, loader)
            v.update_model_with_gradient(v.model, j, peers[j], clip)
            after, na = await v.evaluate_model(v.model, loader)
            v._restore_model_state(saved)
            deltas.append(before / max(nb, 1) - after / max(na, 1))
        return deltas

    asyncio.run(score_all())                       # warm-up (compilation, allocator)
    times = []
    for _ in range(a.iters):
        if world > 1:
            dist.barrier()
        sync()
        t0 = time.perf_counter()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        deltas = asyncio.run(score_all())
        if cuda:
            e1.record()
        sync()
        ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    times.sort()
    ms = times[len(times) // 2]
    if rank == 0:
        print(json.dumps({"case": "config5_validator_scoring", "impl": "reference", "reference_version": tplr.__version__,
                          "model": a.model, "world": world, "peers": a.peers, "ms_per_peer": ms / a.peers,
                          "peers_per_s": a.peers / ms * 1e3, "tokens_per_eval_per_gpu": a.batch * a.seq_len,
                          "loss_delta_first_peer": float(deltas[0]), "dtype": "bf16",
                          "data": "synthetic uniform-random tokens, random-init weights, seeded synthetic peer payloads"}))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
