"""Reference arm of the compressed-gradient gather microbenchmark: the UNMODIFIED reference's own
``ChunkingTransformer`` / ``TopKCompressor`` (src/tplr/compress.py) and ``tplr.neurons.outer_step``
(src/tplr/neurons.py:224-476) with NCCL ``all_gather`` of the packed payloads, every rank acting as one peer.

Per round and rank, exactly what the reference's miner and outer step execute per parameter:
``encode(use_dct=True)`` -> ``compress(top-k, 12-bit pack)`` -> all_gather of indices and values -> a gather result
with one list entry per peer -> ``outer_step`` (rank 0 clips, batch-decompresses and inverse-transforms each
parameter and broadcasts the dense gradient; every rank applies SGD).  None of this repository's kernels, models
or engine is on that path: the parameter shapes are the benchmark model's, held in a plain module.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
        -m baseline.reference_config3 --topk 16 32 64
"""

from __future__ import annotations

import argparse
import json
import os
from types import SimpleNamespace

import torch
import torch.distributed as dist

# tensors of the 1B benchmark model: (name, shape) in named_parameters() order
def model_shapes(name: str = "1B") -> list[tuple[str, tuple]]:
    d, L, f, v = {"1B": (2048, 16, 8192, 32000), "150M": (768, 12, 3072, 32000), "tiny": (128, 2, 256, 512)}[name]
    out = [("tok_embeddings.weight", (v, d))]
    for i in range(L):
        p = f"layers.{i}."
        out += [(p + "attention.wq.weight", (d, d)), (p + "attention.wk.weight", (d, d)), (p + "attention.wv.weight", (d, d)),
                (p + "attention.wo.weight", (d, d)), (p + "feed_forward.w1.weight", (f, d)),
                (p + "feed_forward.w2.weight", (d, f)), (p + "feed_forward.w3.weight", (f, d)),
                (p + "attention_norm.weight", (d,)), (p + "ffn_norm.weight", (d,))]
    return out + [("norm.weight", (d,)), ("output.weight", (v, d))]


class ShapeModel(torch.nn.Module):
    """Parameters with the benchmark model's shapes under their usual names (no forward pass is needed)."""

    def __init__(self, shapes, device, dtype):
        super().__init__()
        self._names = []
        for name, shape in shapes:
            key = name.replace(".", "__")
            self.register_parameter(key, torch.nn.Parameter(torch.zeros(shape, device=device, dtype=dtype)))
            self._names.append(key)


def make_step(model_name: str, k: int, world: int, rank: int, dev):
    """Returns ``step()``: one reference round on this rank.  Imports the reference (``tplr``) on first use."""
    from baseline import ref_env

    ref_env.prepare()
    import tplr

    # FSDP2 keeps fp32 parameters (bf16 only inside the forward pass), so the DCT basis and the momentum are fp32
    model = ShapeModel(model_shapes(model_name), dev, torch.float32)
    transformer = tplr.compress.ChunkingTransformer(model, 64)
    compressor = tplr.compress.TopKCompressor(use_quantization=False)
    optimizer = torch.optim.SGD(model.parameters(), lr=0.4)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    momentum = {n: torch.randn(p.shape, device=dev, generator=gen) * 1e-3 for n, p in model.named_parameters()}

    def step():
        sd, xshapes, totalks = {}, {}, {}
        for n, m in momentum.items():
            enc = transformer.encode(m, use_dct=True)
            idx, val, xshape, totalk = compressor.compress(enc, k)
            xshapes[n], totalks[n] = xshape, totalk
            if world > 1:
                gi = [torch.empty_like(idx) for _ in range(world)]
                gv = [torch.empty_like(val) for _ in range(world)]
                dist.all_gather(gi, idx)
                dist.all_gather(gv, val)
            else:
                gi, gv = [idx], [val]
            sd[n + "idxs"], sd[n + "vals"], sd[n + "quant_params"] = gi, gv, [None] * world
        gather = SimpleNamespace(state_dict=SimpleNamespace(**sd), uids=list(range(world)), skipped_uids=[], success_rate=1.0)
        tplr.neurons.outer_step(model, optimizer, gather_result=gather, transformer=transformer, compressor=compressor,
                                xshapes=xshapes, totalks=totalks, device=str(dev), is_master=rank == 0, world_size=world,
                                use_dct=True)

    return step, tplr.__version__


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1B")
    ap.add_argument("--topk", type=int, nargs="+", default=[16, 32, 64])
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo")
    for k in a.topk:
        step, version = make_step(a.model, k, world, rank, dev)
        ts = []
        for i in range(a.iters + 1):
            if world > 1:
                dist.barrier()
            if cuda:
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1)
            else:
                import time
                t0 = time.perf_counter()
                step()
                ms = (time.perf_counter() - t0) * 1e3
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if i >= 1:
                ts.append(float(t.item()))
        if rank == 0:
            print(json.dumps({"case": "config3_gather", "impl": "reference", "reference_version": version, "model": a.model,
                              "world": world, "topk": k, "reference_ms": sorted(ts)[len(ts) // 2]}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
