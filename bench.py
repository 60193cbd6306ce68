#!/usr/bin/env python
"""Headline benchmark: 1B-config training tokens/s over full windows (inner steps + compress +
gather + outer step), device-timed, max over ranks.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched through torchrun)
    python bench.py --impl reference ...                      (the unmodified reference, same window)

One *step* is one window of the benchmark configuration: ``accum`` micro-batches of
``micro_batch x seq_len`` uniform-random tokens per GPU (forward + backward, fp32 gradient
accumulation), one clipped AdamW inner step, the pseudo-gradient compression (error feedback,
chunk-64 DCT, top-32, 12-bit packing), the gather of 8 peers' payloads and the fused
unpack/clip/mean/inverse-DCT/outer update.  Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="1B")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--accum", type=int, default=4)
    ap.add_argument("--peers", type=int, default=8)
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--outer-update", default="sgd", choices=["sgd", "sign"])
    ap.add_argument("--values", default="uint8", choices=["fp32", "uint8"],
                    help="wire format of this node's payload values: fp32, or the reference miner's 8-bit codes "
                         "(256 bins, 6 sigma) with the quantisation error kept in the error feedback")
    ap.add_argument("--shard-params", action="store_true",
                    help="hold bf16 weights and fp32 gradients as shards too (the FSDP role): weights gathered per block "
                         "over NVLink ahead of their use, weight gradients reduce-added into the owners' shards by the "
                         "GEMM epilogue; the model is initialised tensor by tensor and never exists whole on a GPU")
    ap.add_argument("--gather-buffers", type=int, default=0,
                    help="with --shard-params: block buffers in rotation (>= the number of blocks keeps all gathered; "
                         "0 = all blocks when the bf16 weights are at most 8 GiB, else 2)")
    ap.add_argument("--replicas", type=int, default=1,
                    help="copies of the sharded state (the reference's dp_replicate): the ranks form this many groups of "
                         "world/replicas consecutive ranks, state sharded inside a group, gradient shards all-reduced "
                         "across the groups once per inner step; replicas == world is plain data parallelism")
    ap.add_argument("--gather-engine", default=None, choices=[None, "sm", "dma"],
                    help="with --shard-params: weight gathers by the copy kernel (sm) or by the copy engines (dma)")
    ap.add_argument("--checkpoint-blocks", action="store_true", help="recompute every block in the backward pass")
    ap.add_argument("--gemm", default=None, choices=[None, "tcgen05", "tcgen05_2sm", "cublas"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--breakdown", action="store_true",
                    help="also print per-phase device times of one extra window (stderr; not part of the timed region)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="also run one extra window under torch.profiler and print the summed duration of every kernel at "
                         "in-window clocks plus the total of the gaps between kernels (stderr; diagnostic, not a timing)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    return ap.parse_args()


MODEL_DIMS = {   # the benchmark shapes, as label text shared by both arms
    "tiny": "d128 L2 H4 F256 V512", "150M": "d768 L12 H12 F3072 V32000", "1B": "d2048 L16 H16 F8192 V32000",
    "8B": "d4096 L32 H32 KV8 F14336 V128256", "18B-tp": "d8192 L16 H64 KV8 F28672 V128256",
    "34B": "d8192 L32 H64 KV8 F28672 V128256",
}


def config_labels(a, world: int) -> dict:
    """The ``config`` object of the JSON line.  It names the workload only (model shapes, batch, window definition), so
    the two arms of the benchmark print the same object for the same arguments; what differs between the arms
    (kernels, sharding mechanics, compilation) is reported under ``impl_detail``."""
    return {"model": f"llama-{a.model} ({MODEL_DIMS.get(a.model, a.model)})",
            "global_batch": a.micro_batch * a.accum * world, "micro_batch": a.micro_batch, "accum": a.accum,
            "seq_len": a.seq_len, "parallelism": f"dp{world}: sharded data parallel over {world} ranks of one node"
            if world > 1 else "single GPU",
            "peers": a.peers, "topk": a.topk, "use_dct": True, "outer_update": a.outer_update, "payload_values": "uint8",
            "l2": "inputs larger than L2 (2.4 GB bf16 weights, 134 MB activations per layer)"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while timing."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def run_ours(a):
    import torch.distributed as dist
    from templar_b200.models.llama import PRESETS, build_model
    from templar_b200.ops import functional as OF, native
    from templar_b200.parallel.window_engine import EngineConfig, WindowEngine
    from templar_b200.parallel import symmetric

    rank = int(os.environ.get("RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    heap = None
    srank, sworld = rank, world                   # this rank's place inside its copy of the sharded state
    shard_group = replicate_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        if a.replicas > 1:
            if world % a.replicas:
                raise SystemExit(f"--replicas {a.replicas} does not divide {world} ranks")
            per = world // a.replicas
            sgs = [dist.new_group(list(range(r * per, (r + 1) * per))) for r in range(a.replicas)]
            rgs = [dist.new_group(list(range(s, world, per))) for s in range(per)]
            shard_group, replicate_group = (sgs[rank // per] if per > 1 else None), rgs[rank % per]
            srank, sworld = rank % per, per
        if sworld > 1:
            heap = symmetric.SymmetricHeap.create(dev, srank, sworld, group=shard_group)
    if a.gemm:
        OF.set_gemm_backend(a.gemm)
    args = PRESETS[a.model]
    cfg = EngineConfig(topk=a.topk, use_dct=True, outer_update=a.outer_update, max_peers=a.peers,
                       quantize=a.values == "uint8", quant_bins=256, quant_range=6.0, shard_params=a.shard_params,
                       gather_buffers=a.gather_buffers)
    if a.gather_engine:
        os.environ["TPLR_GATHER_ENGINE"] = a.gather_engine
    if a.shard_params:
        from templar_b200.models.llama import LlamaModel
        with torch.device("meta"):
            model = LlamaModel(args)
        model.freqs_cis = model._freqs_cis().to(dev)
        eng = WindowEngine(model, cfg, device=dev, rank=srank, world_size=sworld, heap=heap, group=shard_group,
                           replicate_group=replicate_group, replicate_size=a.replicas if replicate_group is not None else 1,
                           materialize=lambda name: model.materialize_param(name, dev, torch.bfloat16, seed=0))
    else:
        model = build_model(args, device=dev, dtype=torch.bfloat16, seed=0)
        eng = WindowEngine(model, cfg, device=dev, rank=srank, world_size=sworld, heap=heap, group=shard_group,
                           replicate_group=replicate_group, replicate_size=a.replicas if replicate_group is not None else 1)
    model.activation_checkpointing = a.checkpoint_blocks
    L = eng.layout
    B, S, A = a.micro_batch, a.seq_len, a.accum
    g = torch.Generator().manual_seed(1234 + rank)
    # synthetic data: a pool of pinned host batches (uniform-random token ids)
    n_pool = A * 2
    host_tokens = [torch.randint(0, args.vocab_size, (B, S + 1), generator=g).pin_memory() for _ in range(n_pool)]
    dev_tokens = [t.to(dev) for t in host_tokens]
    # synthetic peers 1..P-1: seeded payloads in pinned host memory (flat wire format of this layout)
    hosted = [j for j in range(1, a.peers) if j % sworld == srank]      # every copy of the state stages all peers
    host_payload = {}
    from templar_b200.utils.synthetic import synthetic_payload
    for j in hosted:
        idx, val = synthetic_payload(L, 99 + j, device=dev)
        if a.values == "uint8":                  # peers send 8-bit codes with per-tensor tables, decoded on the device
            codes, table = eng.encode_values(val)
            host_payload[j] = (idx.cpu().pin_memory(), codes.cpu().pin_memory(), table.cpu().pin_memory())
        else:
            host_payload[j] = (idx.cpu().pin_memory(), val.cpu().pin_memory())
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def window(e2e: bool, w: int):
        eng.snapshot()
        losses = []
        for m in range(A):
            if e2e:
                tok = host_tokens[(w * A + m) % n_pool].to(dev, non_blocking=True)
            else:
                tok = dev_tokens[(w * A + m) % n_pool]
            losses.append(eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0 / A))
        eng.optimizer_step()
        own_ptrs = None
        if heap is not None:
            own_ptrs = (heap.peer_ptr(eng.own_idx, 0), heap.peer_ptr(eng.own_val, 0))
        eng.compress(own_slot_ptrs=own_ptrs)
        # peers' payloads: pinned host memory -> device slots on a side stream, beside this node's own compress
        eng.load_peer_payloads_async([(j // sworld, host_payload[j]) for j in hosted])
        if sworld > 1:
            eng._barrier()
        eng.outer_step(a.peers)
        loss = torch.stack(losses).mean()
        if e2e:
            loss_host.copy_(loss.reshape(1), non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(loss_host[0])
        return loss

    def timed(e2e: bool, steps: int, warmup: int):
        for w in range(warmup):
            window(e2e, w)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local); sampler.start()
        l0 = native.launch_count
        t0w = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if a.profiler_range:
            torch.cuda.profiler.start()
        e0.record()
        for w in range(steps):
            window(e2e, warmup + w)
        e1.record()
        torch.cuda.synchronize()
        if a.profiler_range:
            torch.cuda.profiler.stop()
        if world > 1:
            dist.barrier()
        wall = time.perf_counter() - t0w
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms if not e2e else wall * 1e3], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), native.launch_count - l0, clocks

    def breakdown():
        """One extra window with a CUDA event at every phase boundary (and inside the optimizer, compress and outer
        steps); per phase the MAX over ranks, since a rank's barrier wait is another rank's work."""
        eng.start_trace()
        eng.snapshot()
        for m in range(A):
            tok = dev_tokens[m % n_pool]
            eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0 / A)
        eng.optimizer_step()
        own_ptrs = None
        if heap is not None:
            own_ptrs = (heap.peer_ptr(eng.own_idx, 0), heap.peer_ptr(eng.own_val, 0))
        eng.compress(own_slot_ptrs=own_ptrs)
        # peers' payloads: pinned host memory -> device slots on a side stream, beside this node's own compress
        eng.load_peer_payloads_async([(j // sworld, host_payload[j]) for j in hosted])
        eng._mark("peer_payload_h2d")
        if sworld > 1:
            eng._barrier()
            eng._mark("outer.barrier_payloads_staged")
        eng.outer_step(a.peers)
        ms = eng.trace_ms()
        names = sorted(ms)
        if world > 1:
            all_names = [None] * world
            dist.all_gather_object(all_names, names)
            names = sorted(set().union(*all_names))
        t = torch.tensor([ms.get(n, 0.0) for n in names], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return {n: round(float(v), 3) for n, v in zip(names, t.tolist())}

    def kernel_times():
        """One window under torch.profiler (CUPTI): where the device time of a window goes at the clocks the window
        really runs at, and how much of it is idle between kernels.  Diagnostic only: nothing here is a reported timing."""
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            window(False, a.warmup + a.steps + 1)
            torch.cuda.synchronize()
        evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
        if not evs:
            return {}
        by = {}
        for e in evs:
            name = e.name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
            name = name.split("(")[0].replace("void ", "")[:60]
            d = by.setdefault(name, [0, 0.0])
            d[0] += 1
            d[1] += (e.time_range.end - e.time_range.start) / 1e3
        gaps = sum(max(0, b_.time_range.start - a_.time_range.end) for a_, b_ in zip(evs, evs[1:])) / 1e3
        top = sorted(by.items(), key=lambda kv: -kv[1][1])[:24]
        return {"kernels": len(evs), "kernel_ms_sum": round(sum(v[1] for v in by.values()), 2),
                "span_ms": round((evs[-1].time_range.end - evs[0].time_range.start) / 1e3, 2), "gap_ms_sum": round(gaps, 2),
                "by_kernel_ms": {k: [v[0], round(v[1], 2)] for k, v in top}}

    ms_total, launches, clocks = timed(False, a.steps, a.warmup)
    if a.kernel_times:
        kt = kernel_times()
        if rank == 0:
            print("kernel_times " + json.dumps(kt), file=sys.stderr)
    if a.breakdown:
        bd = breakdown()
        if rank == 0:
            print("breakdown_ms " + json.dumps(bd), file=sys.stderr)
    tokens_per_step = B * S * A * world
    value = tokens_per_step * a.steps / (ms_total / 1e3)
    e2e = None
    if not a.no_e2e:
        ms_e2e, _, _ = timed(True, a.steps, 1)
        # bytes of the whole job, like the value: every rank copies its token batches and the payloads of the
        # peers it hosts from pinned host memory and reads its loss back
        io = torch.tensor([A * B * (S + 1) * 8 + sum(t.numel() * t.element_size() for pl in host_payload.values() for t in pl),
                           4], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(io)
        e2e = {"value": tokens_per_step * a.steps / (ms_e2e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(io[0]), "d2h_bytes_per_step": int(io[1])}
    status = eng.check_status()
    sharding_label = ("bf16 weights, fp32 gradients and all optimizer state sharded; weights gathered per block, "
                      f"{eng.store.gather.n_buffers} block buffers, gathers by {eng.store.gather.engine}" if a.shard_params else
                      "single GPU" if world == 1 else
                      "whole state on every rank" if sworld == 1 else
                      "optimizer state, master weights, snapshot and error feedback sharded; bf16 weights and fp32 "
                      "gradients whole on every rank")
    if eng.replicate_size > 1:
        sharding_label += f"; {eng.replicate_size} copies of {sworld} ranks, gradient shards all-reduced across the copies (NCCL)"
    free_b, total_b = torch.cuda.mem_get_info(dev)       # includes the symmetric heap, which torch's allocator does not see
    peak = torch.tensor([torch.cuda.max_memory_allocated(dev) / 2 ** 30, (total_b - free_b) / 2 ** 30],
                        dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        mfu = value / world * args.flops_per_token(S) / 1e12
        out = {"metric": "1B tokens/s (device-timed, max over ranks); window = inner step + compress + gather + outer step",
               "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
               "ms_per_step": ms_total / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
               "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights, seeded synthetic peer payloads",
               "impl": "ours", "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
               "model_tflops_per_gpu": mfu, "kernel_status": status, "gemm_backend": OF.gemm_backend(),
               "library_gemm_fallbacks": OF.library_gemm_fallbacks,
               "impl_detail": {"payload_values": a.values, "sharding": sharding_label,
                               "peak_torch_allocated_gib_max_over_ranks": round(float(peak[0]), 2),
                               "device_memory_in_use_gib_max_over_ranks": round(float(peak[1]), 2),
                               "weight_gathers": eng.store.gather.gathers if a.shard_params else 0},
               "config": config_labels(a, world)}
        if a.values != "uint8":
            out["config"]["payload_values"] = a.values
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_reference(a):
    try:
        from baseline import reference_bench
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"baseline harness import failed: {e}"[:300]}))
        return
    reference_bench.main(a)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
