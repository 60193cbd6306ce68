"""Miner: trains for a window, publishes a compressed pseudo-gradient, gathers its peers'
gradients and applies the outer step.

    torchrun --standalone --nproc-per-node 8 neurons/miner.py --device cuda [--offline]

Window flow (reference: neurons/miner.py:366-984):
update peers → snapshot parameters → inner steps → pseudo-gradient + error feedback + compression
→ upload → gather peers (with reserve tier, upload-time window) → outer step → debug slice,
metrics → next window.  With the window engine the snapshot stays in HBM and the restore is fused
into the compress / outer-step kernels; every rank compresses and applies its own shard.
"""

from __future__ import annotations

import argparse
import asyncio
import gc
import hashlib
import os
import sys
import time
from datetime import datetime, timedelta, timezone
from types import SimpleNamespace

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from neurons.base_node import BaseNode  # noqa: E402
from neurons.trainer import Trainer  # noqa: E402
from templar_b200.backends.chain import StaticWallet, make_subtensor  # noqa: E402
from templar_b200.distributed import dist_helper  # noqa: E402
from templar_b200.metrics import MetricsLogger  # noqa: E402
from templar_b200.wandb_ops import initialize_wandb  # noqa: E402


def common_args(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--netuid", type=int, default=268)
    parser.add_argument("--project", type=str, default="templar")
    parser.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    parser.add_argument("--amp-dtype", choices=["bf16", "fp16"], default="bf16")
    parser.add_argument("--local_rank", type=int, default=int(os.getenv("LOCAL_RANK", 0)))
    parser.add_argument("--debug", action="store_true")
    parser.add_argument("--trace", action="store_true")
    parser.add_argument("--store-gathers", action="store_true")
    parser.add_argument("--test", action="store_true", help="use every uid of the metagraph as a peer")
    # "--offline" is the same switch under a name that torch.distributed.run's own parser does not claim: behind
    # torchrun, "--local" is rejected as an ambiguous prefix of its --local-addr / --local-ranks-filter options
    parser.add_argument("--local", "--offline", dest="local", action="store_true", help="toy model / local storage run")
    parser.add_argument("--profile-iters", type=int, default=0)
    parser.add_argument("--profile-dir", type=str, default="./log/profiler")
    parser.add_argument("--hparams-dir", type=str, default=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hparams"))
    parser.add_argument("--hparams-file", type=str, default=None, help="JSON file merged over the loaded hparams")
    parser.add_argument("--peers", type=int, nargs="*", default=None, help="fixed peer uids (skips peer-list discovery)")
    parser.add_argument("--use_wandb", action="store_true")
    parser.add_argument("--log_to_private_wandb", action="store_true")
    parser.add_argument("--network", type=str, default="static", help="'static' (offline) or a bittensor network name")
    parser.add_argument("--static-n", type=int, default=8, help="metagraph size of the static chain")
    parser.add_argument("--block-time", type=float, default=12.0)
    parser.add_argument("--uid", type=int, default=None, help="uid on the static chain")
    parser.add_argument("--wallet-hotkey", type=str, default=None)
    parser.add_argument("--max-windows", type=int, default=0, help="stop after this many windows (0 = run forever)")
    parser.add_argument("--colocated", action="store_true",
                        help="the ranks of this launch are independent nodes (uid = --uid + rank) that share one box: "
                             "they read each other's gradients from GPU peer memory instead of the object store")


def finish_config(ns: argparse.Namespace) -> SimpleNamespace:
    cfg = SimpleNamespace(**vars(ns))
    cfg.static_chain = {"n": ns.static_n, "block_time": ns.block_time,
                        "state_file": os.environ.get("TPLR_STATIC_CHAIN_STATE", "/tmp/tplr_static_chain.json"),
                        "genesis": float(os.environ.get("TPLR_STATIC_CHAIN_GENESIS", 0.0)) or None}
    if ns.debug:
        tplr.debug()
    if ns.trace:
        tplr.trace_on()
    return cfg


def load_node_hparams(cfg) -> SimpleNamespace:
    """hparams directory (+ local-run overrides with --local) with an optional JSON file merged on top."""
    hp = tplr.load_hparams(cfg.hparams_dir, use_local_run_hparams=cfg.local)
    if cfg.hparams_file:
        import json

        with open(cfg.hparams_file) as f:
            extra = json.load(f)
        for k, v in extra.items():
            setattr(hp, k, SimpleNamespace(**v) if k == "torchtitan" and isinstance(v, dict) else v)
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                  "num_key_value_heads", "max_position_embeddings", "vocab_size"):
            if k in extra:
                setattr(hp.model_config, k, extra[k])
    return hp


class Miner(BaseNode, Trainer):
    @staticmethod
    def miner_config(argv=None) -> SimpleNamespace:
        p = argparse.ArgumentParser(description="Miner script")
        p.add_argument("--actual-batch-size", type=int, default=None)
        common_args(p)
        return finish_config(p.parse_args(argv))

    def __init__(self, config=None, hparams=None, store=None, subtensor=None):
        BaseNode.__init__(self)
        Trainer.__init__(self)
        self.config = config or Miner.miner_config()
        dist_helper.init_process_group(backend="nccl" if str(self.config.device).startswith("cuda") else "gloo",
                                       timeout_minutes=45)
        # --colocated: every rank of the launch is a whole miner of its own; the group only carries peer memory
        self.group_rank, self.group_world = 0, 1
        if getattr(self.config, "colocated", False) and dist_helper.world_size > 1:
            self.group_rank, self.group_world = dist_helper.solo()
            if self.config.uid is not None:
                self.config.uid = int(self.config.uid) + self.group_rank
        self.rank, self.world_size = dist_helper.rank, dist_helper.world_size
        self.local_rank, self.is_master = dist_helper.local_rank, dist_helper.is_master
        self.device = torch.device(self.config.device if not str(self.config.device).startswith("cuda")
                                   else f"cuda:{self.local_rank}")
        self.config.device = str(self.device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
        self.amp_dtype = torch.bfloat16 if self.config.amp_dtype == "bf16" else torch.float16
        self.hparams = hparams or load_node_hparams(self.config)
        if getattr(self.config, "actual_batch_size", None):
            self.hparams.batch_size = self.config.actual_batch_size
        # chain identity
        self.subtensor = subtensor or make_subtensor(self.config)
        self.metagraph = self.subtensor.metagraph(self.config.netuid)
        hotkey = self.config.wallet_hotkey or (self.metagraph.hotkeys[self.config.uid] if self.config.uid is not None
                                               else self.metagraph.hotkeys[-1])
        self.wallet = StaticWallet(hotkey)
        if hotkey not in self.metagraph.hotkeys:
            raise SystemExit(f"The wallet {hotkey} is not registered on subnet {self.config.netuid}")
        self.uid = self.metagraph.hotkeys.index(hotkey)
        # model + engine + compression geometry
        self.init_model(meta=False)
        self.model_initialized = True
        heap = None
        if self.world_size > 1:
            heap = self.make_heap()
        elif self.group_world > 1 and self.device.type == "cuda":
            from templar_b200.parallel.symmetric import SymmetricHeap

            # co-located nodes wait for each other once per window: the bound is a window, not a kernel
            heap = SymmetricHeap.create(self.device, self.group_rank, self.group_world, timeout_s=1800.0)
        self.attach_engine(heap=heap)
        self.peer_group = None
        if self.group_world > 1:
            from templar_b200.backends.store import PeerMemoryStore
            from templar_b200.comms import default_store
            from templar_b200.parallel.peer_group import LocalPeerGroup

            self.peer_group = LocalPeerGroup(self.uid, rank=self.group_rank, world_size=self.group_world, heap=heap,
                                             device=self.device)
            self.peer_group.attach(self.engine)
            store = PeerMemoryStore(store or default_store(), self.peer_group)
        self.transformer = tplr.compress.ChunkingTransformer(self.model, target_chunk=self.hparams.target_chunk)
        self.compressor = tplr.compress.TopKCompressor(use_quantization=False)
        self.init_optimizers_schedulers()
        L = self.engine.layout
        self.xshapes = {s.name: L.xshape(s.name) for s in L.specs}
        self.totalks = {s.name: s.totalk for s in L.specs}
        self.owned_params = {n for n, _ in self.model.named_parameters()}     # every rank owns its shard of all tensors
        self.error_feedback, self.error_feedback_cpu_buffers = {}, {}
        self.bootstrap_version = getattr(self.hparams, "checkpoint_init_version", None)
        # storage, checkpoints, telemetry
        self.comms = tplr.Comms(wallet=self.wallet, save_location="/tmp", key_prefix="model", config=self.config,
                                hparams=self.hparams, uid=self.uid, store=store, subtensor=self.subtensor)
        self.ckpt = tplr.DCPCheckpointer(self.comms, uid=self.uid, version=tplr.__version__, repo_root=".")
        if self.is_master:
            self.comms.try_commit(self.wallet, self.comms.bucket)
        dist_helper.safe_barrier("post_commit", self.local_rank)
        self.start_window = 0
        self.global_step = 0
        self.window_step = 0
        self.total_tokens_processed = 0
        self.next_peers, self.next_reserve_peers, self.peers_update_window = None, None, -1
        self.comms.peers, self.comms.reserve_peers = [], []
        self.wandb = initialize_wandb("M", self.uid, self.config, "miner", "mining") if self.is_master else None
        self.metrics_logger = MetricsLogger(prefix="M", uid=self.uid, config=self.config, role="miner", group="miner",
                                            job_type="mining") if self.is_master else None
        self.dataset_manager = self._dataset_manager()
        self.gather_timeout = 90

    def _dataset_manager(self):
        hp = self.hparams
        if os.environ.get("DATASET_BINS_PATH") and os.path.isdir(os.environ["DATASET_BINS_PATH"]) and \
                os.listdir(os.environ["DATASET_BINS_PATH"]):
            anneal = (getattr(hp, "anneal_mode", {}) or {})
            return tplr.ShardedDatasetManager(hp.sequence_length, self.rank, self.world_size, self.comms,
                                              file_prefix=anneal.get("file_prefix", "train") if anneal.get("enabled") else "train",
                                              anneal_mode=bool(anneal.get("enabled", False)))
        n = max(hp.inner_steps * hp.target_batch_size * 4, 1024)
        ds = tplr.SyntheticDataset(n, hp.sequence_length, self.hparams.model_config.vocab_size, seed=1234)
        return SimpleNamespace(active_dataset=ds, initialize_datasets=_noop_async, swap_datasets=_noop_async, shard_index=0)

    # ------------------------------------------------------------------------------------ #
    async def run(self):
        self.loop = asyncio.get_running_loop()
        self.comms.start_commitment_fetcher()
        self.comms.commitments = await self.comms.get_commitments()
        self.comms.current_window = self.current_window
        if self.config.peers is not None:
            self.comms.peers = [u for u in self.config.peers]
        elif self.is_master:
            await tplr.neurons.update_peers(instance=self, window=self.current_window, peer_start=tplr.T())
        # start window (validator-published); offline default: now
        sw = await self.comms.get_start_window(retries=2, retry_delay=0.5) if self.is_master else None
        t = torch.tensor([sw if sw is not None else self.current_window], dtype=torch.long, device=self.device)
        dist_helper.broadcast(t, src=0)
        self.start_window = int(t.item())
        ok, win, step, boot = await tplr.neurons.load_checkpoint_with_fallback(self)
        if ok or self.current_window > self.start_window:
            await tplr.neurons.handle_checkpoint_catchup(self, ok, win, step, boot)
        await self.init_shard_schedule()
        if self.is_master:
            # an (empty) object under this window's gradient key marks the miner as active for the validators
            await self.comms.put(state_dict={"metadata": {"window": self.current_window, "dummy": True}}, uid=str(self.uid),
                                 window=self.current_window, key="gradient", local=False)
        windows_done = 0
        while not self.stop_event.is_set():
            step_window = self.current_window
            self.global_step = max(self.global_step, 0)
            await self.run_window(step_window)
            windows_done += 1
            if self.config.max_windows and windows_done >= self.config.max_windows:
                self.stop_event.set()
                break
            await self.wait_until_window(step_window + 1)

    async def run_window(self, step_window: int) -> dict:
        """One full window; returns its timing / loss summary."""
        hp = self.hparams
        t_win = tplr.T()
        if self.is_master and self.config.peers is None:
            # every window, as the reference does (neurons/miner.py:484-489): the first list a validator publishes has
            # to be found by a miner that has none yet
            await tplr.neurons.update_peers(instance=self, window=step_window, peer_start=tplr.T())
        await self.maybe_switch_shard(step_window)
        self.sampler.set_window_uid(self.uid, step_window)
        saved, specs = dist_helper.get_offloaded_params(self.model)
        # null rounds (reference neurons/miner.py:542-568): no training signal is sent while the validators have
        # not published a peer list for this miner yet (the first validator_offset + peer_list_window_margin
        # windows after the start window) or while there is nobody to gather from; local runs start at once
        warmup = 0 if (self.config.local or self.config.test) else (
            getattr(hp, "validator_offset", 1) + getattr(hp, "peer_list_window_margin", 2))
        warmup_null = step_window - (self.start_window or step_window) < warmup
        no_peers_null = len(self.comms.peers) == 0 and not self.config.test
        null_round = dist_helper.all_agree(warmup_null or no_peers_null, self.device, "null_round")
        if null_round:
            tplr.logger.info("null round: " + ("warm-up" if warmup_null else "no gather peers" if no_peers_null
                                               else "requested by another rank"))
        t0 = tplr.T()
        res = await self.inner_steps(loader=self.loader, step_window=step_window, null_round=null_round)
        train_time = tplr.T() - t0
        dist_helper.restore_offloaded_params(self.model, saved, specs)
        self.offload_inner_optimizer_states()
        dist_helper.safe_barrier("pre_gather", self.local_rank)
        t0 = tplr.T()
        gradient, _, _ = tplr.prepare_gradient_dict(self, step_window, null_round)
        compress_time = tplr.T() - t0
        if self.peer_group is not None:
            self.peer_group.publish(step_window)      # the payload in this rank's buffers is this window's
        put_time = 0.0
        # The gradient of a window is uploaded once the window is over: validators and peers accept an upload only
        # between the first block of the next window and `time_window_delta_seconds` after it, so a miner that
        # finishes early waits for the chain (reference neurons/miner.py:685-701).  Local runs have no clock.
        if not self.config.local and self.current_window == step_window:
            tplr.logger.info("Training complete; waiting for window to be exhausted...")
            await self.wait_until_window(step_window + 1)
        if self.is_master:
            gidx = self.sampler._global_indices()
            ids = self.sampler.ids_for_indices(gidx.tolist())
            h = hashlib.blake2b(digest_size=16)
            h.update(np.asarray(sorted(ids), dtype=np.uint64).tobytes())
            gradient["metadata"] = {"window": step_window, "sample_digest": h.hexdigest(), "sample_count": len(ids)}
            put_time = await self.comms.put(state_dict={k: (v.clone() if torch.is_tensor(v) else v) for k, v in gradient.items()},
                                            uid=str(self.uid), window=step_window, key="gradient",
                                            global_step=self.global_step, local=False, stale_retention=100)
        # upload-time acceptance window of the peers' gradients: it opens with the first block of the window the
        # chain is in now, a block that exists (reference neurons/miner.py:718-730)
        sync_block = (self.current_window if not self.config.local else step_window + 1) * hp.blocks_per_window
        ts = await self.loop.run_in_executor(None, self.query_block_timestamp, sync_block)
        if ts is None:
            tplr.logger.warning(f"Could not get timestamp for sync block {sync_block}. Using current time as fall back.")
        tmin = datetime.fromtimestamp(ts if ts is not None else time.time(), tz=timezone.utc)
        tmax = tmin + timedelta(seconds=getattr(hp, "time_window_delta_seconds", 70))
        if self.config.test:
            self.comms.peers = [u for u in range(len(self.comms.metagraph.S)) if u != self.uid]
        gather_result, gather_time = None, 0.0
        if self.peer_group is not None:
            self.peer_group.exchange()                # every co-located node's payload of this window is in place
        if self.is_master and self.comms.peers:
            t0 = tplr.T()
            gather_result = await self.comms.gather_with_reserve(
                my_uid=self.uid, gather_uids=list(self.comms.peers), reserve_uids=list(self.comms.reserve_peers),
                window=step_window, key="gradient", timeout=self.gather_wait_seconds(), device="cpu", local=False,
                stale_retention=100, totalks=self.totalks, xshapes=self.xshapes, compressor=self.compressor,
                time_min=None if self.config.local else tmin, time_max=None if self.config.local else tmax,
                expected_compressed_params=self.expected_compressed_params)
            gather_time = tplr.T() - t0
        should_update = dist_helper.all_ok(gather_result is not None if self.is_master else True, self.device, "gather_update")
        t0 = tplr.T()
        fingerprint = None
        if should_update:
            fingerprint = self.outer_step(gather_result)
            self.global_step += 1
        else:
            self.engine.restore()            # no update this window: back to the window-start weights
            self.engine.window_open = False
        update_time = tplr.T() - t0
        self.window_step += 1
        self.total_tokens_processed += res["batch_tokens"]
        summary = {"window": step_window, "loss": res["total_loss"] / max(res["batch_count"], 1),
                   "tokens": res["batch_tokens"], "tokens_per_sec": res["batch_tokens"] / train_time if train_time else 0.0,
                   "train_time": train_time, "compress_time": compress_time, "put_time": put_time,
                   "gather_time": gather_time, "update_time": update_time, "window_time": tplr.T() - t_win,
                   "gather_success_rate": getattr(gather_result, "success_rate", 0.0) if gather_result else 0.0,
                   "skipped_uids": getattr(gather_result, "skipped_uids", []) if gather_result else [],
                   "global_step": self.global_step, "fingerprint": fingerprint}
        if self.is_master:
            await self._publish_debug(step_window)
            self._log_window(summary, res)
        await self.cleanup_window()
        dist_helper.safe_barrier("end_window", self.local_rank)
        return summary

    # -- memory hygiene (reference neurons/miner.py:59-81, :986-1008) -------------------------------------- #
    def log_gpu_memory(self, stage: str) -> None:
        if self.device.type == "cuda":
            gib = 1024 ** 3
            tplr.logger.info(f"[GPU Memory - {stage}] Allocated: {torch.cuda.memory_allocated(self.device) / gib:.2f} GB, "
                             f"Reserved: {torch.cuda.memory_reserved(self.device) / gib:.2f} GB")

    def check_memory_threshold(self, threshold_gb: float = 0.5) -> bool:
        """Release the caching allocator's free blocks when less than ``threshold_gb`` is left; True if it did."""
        if self.device.type != "cuda":
            return False
        free, _total = torch.cuda.mem_get_info(self.device)
        if free / 1024 ** 3 >= threshold_gb:
            return False
        tplr.logger.warning(f"Low GPU memory: {free / 1024 ** 3:.2f} GB available")
        torch.cuda.empty_cache()
        torch.cuda.synchronize(self.device)
        self.log_gpu_memory("After emergency cleanup")
        return True

    async def cleanup_window(self) -> None:
        """Between windows: drop autograd leftovers of the module tree and host garbage.  The flat buffers of the
        engine (weights, gradients, optimizer state, error feedback, payload slots) are allocated once and stay."""
        for p in self.model.parameters():
            p.grad = None
        torch.clear_autocast_cache()
        gc.collect()
        self.check_memory_threshold()

    async def _publish_debug(self, window: int) -> None:
        """Two elements ([10:12]) of every parameter of the local view, used by validators to
        measure how far this miner is from the consensus weights."""
        dbg = {name + "_debug": v.float().cpu().tolist() for name, v in tplr.neurons.param_samples(self.model, 10, 12).items()}
        dbg["successful_peers"] = sorted(set(self.comms.peers))
        await self.comms.put(state_dict=dbg, uid=str(self.uid), window=window, key="debug", local=False)

    def _log_window(self, s: dict, res: dict) -> None:
        tplr.logger.info(f"{tplr.P(s['window'], s['window_time'])} loss={s['loss']:.4f} tok/s={s['tokens_per_sec']:.0f} "
                         f"train={s['train_time']:.2f}s compress={s['compress_time']:.3f}s gather={s['gather_time']:.2f}s "
                         f"update={s['update_time']:.3f}s")
        fields = {k: v for k, v in s.items() if isinstance(v, (int, float))}
        fields.update({"global_grad_norm": res.get("global_grad_norm", 0.0), "global_weight_norm": res.get("global_weight_norm", 0.0)})
        if self.metrics_logger is not None:
            self.metrics_logger.log("training_step_v2", tags={"window": s["window"], "global_step": s["global_step"]},
                                    fields=fields, with_system_metrics=True, with_gpu_metrics=True)
        if self.wandb is not None:
            self.wandb.log({f"miner/{k}": v for k, v in fields.items()}, step=s["global_step"])


async def _noop_async(*a, **k):
    return 0


def main():
    try:
        import uvloop

        uvloop.install()
    except Exception:  # noqa: BLE001
        pass
    asyncio.run(Miner().main())


if __name__ == "__main__":
    main()
