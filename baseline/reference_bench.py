"""Reference arm of ``bench.py``: the same window, run by the UNMODIFIED reference.

The node object below is a ``neurons.trainer.Trainer`` (the reference's own mixin) given the
attributes its methods read; every step of the timed window is a call into the reference:

    tplr.model_factory.initialize_torchtitan_model      FSDP2 (dp_shard = world) torchtitan LLaMA
    Trainer.init_optimizers_schedulers                  outer SGD, fused AdamW, LR schedule
    tplr.distributed.dist_helper.get_offloaded_params   window-start snapshot (pinned host)
    Trainer.inner_steps                                 micro-batches, clip, AdamW (its DataLoader/MinerSampler)
    dist_helper.restore_offloaded_params                pseudo-gradient into p.grad, restore
    tplr.prepare_gradient_dict                          error feedback, chunk DCT, top-k, 12-bit pack
    dist_helper.gather_object + merge                   as neurons/miner.py:629-668
    Trainer.outer_step -> tplr.neurons.outer_step       8 peers: clip, decompress, iDCT, scatter, SGD

Peers 1..7 are the same seeded synthetic payloads the other arm uses, held in pinned host memory
and moved to the device each window (what ``Comms.gather(device=...)`` does with downloads).
Storage, chain and telemetry are not part of the timed window in either arm.
"""

from __future__ import annotations

import asyncio
import json
import os
import sys
import time
from pathlib import Path
from types import SimpleNamespace

import torch

ROOT = Path(__file__).resolve().parents[1]


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))


def _hparams(a, vocab: int, world: int, compile_blocks: bool):
    sizes = {"1B": dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=16, num_key_value_heads=16,
                        intermediate_size=8192),
             "150M": dict(hidden_size=768, num_hidden_layers=12, num_attention_heads=12, num_key_value_heads=12,
                          intermediate_size=3072),
             "tiny": dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                          intermediate_size=256)}[a.model]
    tok = SimpleNamespace(vocab_size=vocab, pad_token_id=vocab + 7, eos_token_id=2, pad_token="</s>", eos_token="</s>")
    hp = SimpleNamespace(
        model_size=f"bench-{a.model}", sequence_length=a.seq_len, micro_batch_size=a.micro_batch,
        batch_size=a.micro_batch * a.accum * world, target_batch_size=a.micro_batch * a.accum * world,
        inner_steps=1, outer_learning_rate=0.4, momentum_decay=0.95, topk_compression=a.topk, target_chunk=64,
        use_dct=True, quantization_bins=256, quantization_range=6, weight_decay=0.1, learning_rate=1e-3, blocks_per_window=10, anneal_mode={"enabled": False},
        optimizer={"type": "adamw", "adamw": {"betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1,
                                              "learning_rate": 1.17e-4,
                                              "scheduler": {"warmup_steps": 1500, "warmup_inner_steps": 0, "t_max": 140000,
                                                            "eta_min_factor": 0.1, "flatten_start_step": None,
                                                            "flatten_duration": 0}}},
        tokenizer=tok, model_config=SimpleNamespace(vocab_size=vocab, rms_norm_eps=1e-5, rope_theta=10000.0, **sizes),
        torchtitan=SimpleNamespace(tp_degree=1, pp_degree=1, cp_degree=1, dp_replicate=1, dp_shard=world,
                                   compile=compile_blocks, enable_cpu_offload=False, mixed_precision_param="bfloat16",
                                   mixed_precision_reduce="float32", enable_async_tensor_parallel=False,
                                   disable_loss_parallel=True, fsdp_reshard_after_forward="default",
                                   enable_compiled_autograd=False, float8_recipe_name=None, tie_embeddings=False,
                                   activation_checkpoint={"mode": "none", "option": "op"}),
    )
    return hp


class _TokenDataset(torch.utils.data.Dataset):
    """Uniform-random token rows materialised once in host memory (same shape as a shard dataset)."""

    def __init__(self, n: int, seq: int, vocab: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        self.tokens = torch.randint(0, vocab, (n, seq), generator=g, dtype=torch.int64)

    def __len__(self):
        return self.tokens.shape[0]

    def __getitem__(self, i):
        return self.tokens[i]

    def sample_id(self, i):
        return int(i)


def main(a) -> None:
    try:
        from baseline import ref_env
        from bench import ClockSampler, config_labels

        report = ref_env.prepare()
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference environment could not be prepared: {e}")
    try:
        import torch.distributed as dist
        import tplr
        from neurons.trainer import Trainer
        from tplr.distributed import dist_helper
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference import failed offline: {type(e).__name__}: {e}")

    # single-process launch: give the device-mesh code the rendezvous variables torchrun would set
    # (the reference's scripts/local_miner_test.py:87-90 does the same)
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0"), ("MASTER_ADDR", "127.0.0.1"),
                 ("MASTER_PORT", str(29400 + os.getpid() % 500))):
        os.environ.setdefault(k, v)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    has_cuda = torch.cuda.is_available()
    if has_cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if has_cuda else torch.device("cpu")   # CPU only for harness debugging
    pin = (lambda t: t.pin_memory()) if has_cuda else (lambda t: t)
    sync = torch.cuda.synchronize if has_cuda else (lambda: None)
    if world > 1:
        dist_helper.init_process_group("nccl" if has_cuda else "gloo", timeout_minutes=30)
    torch.backends.cuda.matmul.allow_tf32 = True      # neurons/miner.py:54-55
    torch.backends.cudnn.allow_tf32 = True
    vocab = 32000 if a.model != "tiny" else 512
    compile_blocks = os.environ.get("TPLR_REF_COMPILE", "1") == "1"

    class Node(Trainer):
        pass

    node = Node()
    node.hparams = _hparams(a, vocab, world, compile_blocks)
    node.rank, node.world_size, node.local_rank, node.is_master = rank, world, local, rank == 0
    node.device, node.uid, node.current_window, node.global_step = dev, 1, 100, 0
    node.config = SimpleNamespace(device=str(dev), local=True)
    node.stop_event = asyncio.Event()
    node.amp_dtype = torch.bfloat16
    node.scaler = torch.amp.GradScaler(dev.type, enabled=False)
    node.wandb = None
    try:
        node.init_model(validator=False, meta=False)
    except Exception as e:  # noqa: BLE001
        if world > 1:
            dist.destroy_process_group()
        return _unavailable(f"reference model_factory failed on the installed torchtitan: {type(e).__name__}: {e}")
    node.transformer = tplr.compress.ChunkingTransformer(node.model, target_chunk=node.hparams.target_chunk)
    # neurons/miner.py:214-221: the reference always quantises payload values to 8 bit
    node.compressor = tplr.compress.TopKCompressor(use_quantization=True, quantization_bins=node.hparams.quantization_bins,
                                                   quantization_range=node.hparams.quantization_range)
    node.init_optimizers_schedulers()
    node.offload_optimizer = False
    node.error_feedback, node.error_feedback_cpu_buffers, node.owned_params = {}, {}, set()
    node.xshapes, node.totalks = {}, {}
    for idx, (n, p) in enumerate(node.model.named_parameters()):       # neurons/miner.py:235-254
        if idx % world == rank:
            node.owned_params.add(n)
            node.error_feedback[n] = None
            node.error_feedback_cpu_buffers[n] = torch.empty(p.shape, device="cpu", pin_memory=has_cuda)
        # shape dry-run as in neurons/miner.py:245-254; without the DCT (fp16 dummy x fp32 basis would
        # not multiply) — the chunk grid does not depend on the transform
        enc = node.transformer.encode(torch.empty(p.shape, dtype=torch.float16, device=dev), use_dct=False)
        _, _, xshape, totalk, _ = node.compressor.compress(enc, node.hparams.topk_compression)
        node.xshapes[n], node.totalks[n] = xshape, totalk
    # data: the reference's own sampler + DataLoader over a host-resident synthetic dataset
    B, S, A = a.micro_batch, a.seq_len, a.accum
    n_rows = max(B * A * world * 8, 64)
    node.dataset_manager = SimpleNamespace(active_dataset=_TokenDataset(n_rows, S, vocab, 1234))
    node.set_dataloader(validator=False)
    # synthetic peers in this framework's layout order are re-keyed to the reference's dict format
    sys.path.insert(0, str(ROOT))
    from templar_b200.parallel.flat import FlatLayout
    from templar_b200.utils.synthetic import synthetic_payload

    shapes = [(n, tuple(p.shape)) for n, p in node.model.named_parameters()]
    layout = FlatLayout(shapes, 64, a.topk, 1)
    peers_host = []
    for j in range(1, a.peers):
        idx, val = synthetic_payload(layout, 99 + j, device=dev)
        idx, val = pin(idx.cpu()), pin(val.cpu())
        entry = {}
        for n, _ in shapes:
            i_view, v_view = layout.payload_views(idx, val, n)
            q, qp = node.compressor._quantize_values(v_view.to(dev))     # the reference's own wire format
            entry[n] = (pin(i_view.cpu().clone()), pin(q.cpu()), (qp[0].cpu(), qp[1], qp[2], qp[3].cpu(), qp[4]))
        peers_host.append(entry)
    h2d_bytes = sum(i.numel() + v.numel() for d in peers_host for i, v, _ in d.values())

    def has_dstate(model):
        return hasattr(node, "offload_inner_optimizer_states")

    async def window(w: int) -> float:
        node.current_window = 100 + w
        node.sampler.set_window_uid(node.uid, node.current_window)
        saved, specs = dist_helper.get_offloaded_params(node.model)
        res = await node.inner_steps(loader=node.loader, step_window=node.current_window, null_round=False)
        dist_helper.restore_offloaded_params(node.model, saved, specs)
        shard, _, _ = tplr.prepare_gradient_dict(node, node.current_window, False)
        gathered = dist_helper.gather_object(shard, object_list=[None] * world if node.is_master else None, dst=0)
        gather_result = None
        if node.is_master:
            own = {}
            for part in gathered:
                own.update({k: v for k, v in part.items() if k != "metadata"})
            sd = {}
            for n, _ in shapes:
                idxs = [own[n + "idxs"].to(dev, non_blocking=True)]
                vals = [own[n + "vals"].to(dev, non_blocking=True)]
                # shards gathered from other ranks arrive with their tensors on the sender's GPU; the
                # reference reads payloads back through its object store with map_location = its device
                qps = [tuple(x.to(dev) if torch.is_tensor(x) else x for x in own[n + "quant_params"])]
                for d in peers_host:
                    i, v, qp = d[n]
                    idxs.append(i.to(dev, non_blocking=True))
                    vals.append(v.to(dev, non_blocking=True))
                    qps.append(qp)
                sd[n + "idxs"], sd[n + "vals"], sd[n + "quant_params"] = idxs, vals, qps
            gather_result = SimpleNamespace(state_dict=SimpleNamespace(**sd), uids=list(range(a.peers)),
                                            skipped_uids=[], success_rate=1.0)
        node.outer_step(gather_result)
        node.global_step += 1
        return float(res["total_loss"]) / max(int(res["batch_count"]), 1)

    async def timed(steps: int, warmup: int):
        for w in range(warmup):
            await window(w)
        if world > 1:
            dist.barrier()
        sync()
        sampler = ClockSampler(local)
        sampler.start()
        t0 = time.perf_counter()
        if has_cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        loss = 0.0
        for w in range(steps):
            loss = await window(warmup + w)
        if has_cuda:
            e1.record()
        sync()
        if world > 1:
            dist.barrier()
        wall = time.perf_counter() - t0
        clocks = sampler.stop()
        t = torch.tensor([e0.elapsed_time(e1) if has_cuda else wall * 1e3, wall * 1e3], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1]), clocks, loss

    # Watchdog: a collective of the reference path that never completes must not hold the GPUs.  After
    # TPLR_REF_TIMEOUT seconds (default 600) rank 0 prints the `unavailable` line and every rank leaves.
    import faulthandler
    import threading

    limit = float(os.environ.get("TPLR_REF_TIMEOUT", "600"))
    if os.environ.get("TPLR_REF_DEBUG_DUMP"):
        faulthandler.dump_traceback_later(float(os.environ["TPLR_REF_DEBUG_DUMP"]), exit=False)

    def _expired():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              f"reference window did not finish within {limit:.0f} s at world_size={world}: "
                              "a collective of its prepare_gradient_dict/outer_step path never completed"}), flush=True)
        os._exit(0)

    watchdog = threading.Timer(limit, _expired)
    watchdog.daemon = True
    watchdog.start()
    try:
        ms, wall_ms, clocks, loss = asyncio.run(timed(a.steps, a.warmup))
        watchdog.cancel()
    except Exception as e:  # noqa: BLE001
        watchdog.cancel()
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
        return _unavailable(f"reference window failed: {type(e).__name__}: {e}")
    tokens = B * S * A * world * a.steps
    if rank == 0:
        print(json.dumps({
            "metric": "1B tokens/s (device-timed, max over ranks); window = inner step + compress + gather + outer step",
            "impl": "reference", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights, seeded synthetic peer payloads",
            "clocks": clocks, "last_loss": loss,
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(A * B * S * 8 + h2d_bytes), "d2h_bytes_per_step": 8 * A},
            "gpu_launches": 0,
            "impl_detail": {"model_code": "torchtitan llama", "sharding": f"fsdp2 dp_shard={world}", "compile": compile_blocks,
                            "payload_values": "uint8 (256 bins) + per-tensor lookup, the reference's stock format",
                            "reference_version": tplr.__version__, "stubbed_packages": report["stubbed"]},
            "config": config_labels(a, world)}))
    if dist.is_initialized():
        dist.destroy_process_group()
