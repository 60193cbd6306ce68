"""Reference arm of the tensor-parallel benchmark (``templar_b200.bench.config4_tp``): the UNMODIFIED reference's model
factory with ``tp_degree = world_size`` and its own inner loop.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
        -m baseline.reference_config4 --steps 3 --warmup 2

What runs, all of it the reference's code (src/tplr/model_factory.py:215-332 and torchtitan's ``apply_tp``; neurons/
trainer.py:752-1036): ``initialize_torchtitan_model`` builds the torchtitan LLaMA of the 18B shapes with the
tensor-parallel + sequence-parallel plan over all ranks, ``init_optimizers_schedulers`` its AdamW, and every timed window
is one call of ``Trainer.inner_steps`` on ``--accum`` micro-batches of ``--micro-batch`` x ``--seq-len`` tokens (the
same batches on every rank, as tensor parallelism needs): forward, backward, clip, optimizer step.

The reference has no compress / gather / outer-step path for a tensor-parallel model (its error-feedback buffers and
its gather validation assume whole tensors, neurons/miner.py:239, src/tplr/comms.py:1892-1917), so its window ends
there.  The other arm's window also compresses its shards and applies an outer step; its inner part is reported
separately by ``config4_tp --breakdown``-less timing of the same call sequence.  Prints one JSON line on rank 0, or an
``unavailable`` line when the reference's tensor-parallel path does not run on the installed torchtitan.
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

SHAPES = {
    "18B-tp": dict(hidden_size=8192, num_hidden_layers=16, num_attention_heads=64, num_key_value_heads=8,
                   intermediate_size=28672, vocab=128256, rope_theta=500000.0),
    "tiny": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                 intermediate_size=512, vocab=512, rope_theta=10000.0),
}


def _unavailable(why: str) -> None:
    print(json.dumps({"case": "config4_tp_window", "impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="18B-tp", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--accum", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    sys.path.insert(0, str(ROOT))
    try:
        from baseline import ref_env

        ref_env.prepare()
        import torch.distributed as dist
        import tplr
        from neurons.trainer import Trainer
        from tplr.distributed import dist_helper
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference import failed offline: {type(e).__name__}: {e}")
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0"), ("MASTER_ADDR", "127.0.0.1"),
                 ("MASTER_PORT", str(29400 + os.getpid() % 500))):
        os.environ.setdefault(k, v)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    if not torch.cuda.is_available():
        return _unavailable("the reference's device mesh needs CUDA")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist_helper.init_process_group("nccl", timeout_minutes=30)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    sh = dict(SHAPES[a.model])
    vocab, theta = sh.pop("vocab"), sh.pop("rope_theta")
    if a.layers:
        sh["num_hidden_layers"] = a.layers
    B, S, A = a.micro_batch, a.seq_len, a.accum
    compile_blocks = os.environ.get("TPLR_REF_COMPILE", "1") == "1"
    tok = SimpleNamespace(vocab_size=vocab, pad_token_id=vocab + 7, eos_token_id=2, pad_token="</s>", eos_token="</s>")
    hp = SimpleNamespace(
        model_size=f"bench-{a.model}", sequence_length=S, micro_batch_size=B, batch_size=B * A, target_batch_size=B * A,
        inner_steps=1, outer_learning_rate=0.4, momentum_decay=0.95, topk_compression=32, target_chunk=64, use_dct=True,
        quantization_bins=256, quantization_range=6, weight_decay=0.1, learning_rate=1e-3, blocks_per_window=10,
        anneal_mode={"enabled": False},
        optimizer={"type": "adamw", "adamw": {"betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1, "learning_rate": 1.17e-4,
                                              "scheduler": {"warmup_steps": 1500, "warmup_inner_steps": 0, "t_max": 140000,
                                                            "eta_min_factor": 0.1, "flatten_start_step": None,
                                                            "flatten_duration": 0}}},
        tokenizer=tok, model_config=SimpleNamespace(vocab_size=vocab, rms_norm_eps=1e-5, rope_theta=theta, **sh),
        torchtitan=SimpleNamespace(tp_degree=world, pp_degree=1, cp_degree=1, dp_replicate=1, dp_shard=1,
                                   compile=compile_blocks, enable_cpu_offload=False, mixed_precision_param="bfloat16",
                                   mixed_precision_reduce="float32", enable_async_tensor_parallel=False,
                                   disable_loss_parallel=True, fsdp_reshard_after_forward="default",
                                   enable_compiled_autograd=False, float8_recipe_name=None, tie_embeddings=False,
                                   activation_checkpoint={"mode": "none", "option": "op"}))

    class Node(Trainer):
        pass

    node = Node()
    node.hparams = hp
    node.rank, node.world_size, node.local_rank, node.is_master = rank, world, local, rank == 0
    node.device, node.uid, node.current_window, node.global_step = dev, 1, 100, 0
    node.config = SimpleNamespace(device=str(dev), local=True)
    node.stop_event = asyncio.Event()
    node.amp_dtype = torch.bfloat16
    node.scaler = torch.amp.GradScaler("cuda", enabled=False)
    node.wandb = None
    node.offload_optimizer = False
    try:
        node.init_model(validator=False, meta=False)
        node.init_optimizers_schedulers()
    except Exception as e:  # noqa: BLE001
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
        return _unavailable(f"reference model_factory with tp_degree={world} failed on the installed torchtitan: "
                            f"{type(e).__name__}: {e}")
    node.sampler = SimpleNamespace(grad_accum_steps=A)
    g = torch.Generator().manual_seed(77)                      # the same batches on every tensor-parallel rank
    batches = [torch.randint(0, vocab, (B, S), generator=g) for _ in range(A * 2)]

    async def window(w: int):
        node.current_window = 100 + w
        loader = [batches[(w * A + m) % len(batches)] for m in range(A)]
        return await node.inner_steps(loader=loader, step_window=node.current_window, null_round=False)

    async def timed():
        for w in range(a.warmup):
            await window(w)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        res = None
        for w in range(a.steps):
            res = await window(a.warmup + w)
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([e0.elapsed_time(e1), wall], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1]), res

    import threading

    limit = float(os.environ.get("TPLR_REF_TIMEOUT", "420"))

    def _expired():
        if rank == 0:
            _unavailable(f"reference tensor-parallel window did not finish within {limit:.0f} s at world_size={world}")
        os._exit(0)

    watchdog = threading.Timer(limit, _expired)
    watchdog.daemon = True
    watchdog.start()
    try:
        ms, wall, res = asyncio.run(timed())
        watchdog.cancel()
    except Exception as e:  # noqa: BLE001
        watchdog.cancel()
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
        return _unavailable(f"reference tensor-parallel window failed: {type(e).__name__}: {e}")
    free_b, total_b = torch.cuda.mem_get_info(dev)
    if rank == 0:
        n_params = sum(p.numel() for p in node.model.parameters())          # DTensor.numel() is the logical size
        print(json.dumps({"case": "config4_tp_window", "impl": "reference", "reference_version": tplr.__version__,
                          "model": a.model, "layers": sh["num_hidden_layers"], "world": world, "parallelism": f"tp{world}",
                          "window": "inner step only: forward + backward of the micro-batches, clip, AdamW "
                                    "(the reference has no compress / outer step for a tensor-parallel model)",
                          "micro_batch": B, "seq_len": S, "accum": A, "ms_per_window": ms / a.steps,
                          "wall_ms_per_window": wall / a.steps, "tokens_per_s": B * S * A * a.steps / (ms / 1e3),
                          "parameters": n_params, "compile": compile_blocks,
                          "micro_batches_last_window_summed_over_ranks": int(res["batch_count"]) if isinstance(res, dict) else None,
                          "device_memory_in_use_gib": round((total_b - free_b) / 2 ** 30, 2), "dtype": "bf16 autocast",
                          "data": "synthetic uniform-random tokens, random-init weights"}), flush=True)
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
