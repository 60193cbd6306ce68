"""Evaluator: follows the published checkpoints and reports perplexity / bits-per-byte and
(where a harness is installed) downstream-task scores.

    torchrun --standalone --nproc-per-node 2 neurons/evaluator.py --device cuda [--local]

Flow (reference: neurons/evaluator.py:1113-1222): read the start window → find the newest complete
checkpoint (``_LATEST.json`` pointer or listing, completeness gate) → load it (DCP reshards to this
topology) → convert to HF layout and cache it → custom evaluation (cross entropy → perplexity and
bits per byte) → ``lm_eval`` in a subprocess when available (rank 0 runs it, the other ranks wait
on a sentinel file) → metrics → sleep ``eval_interval``.  ``--backfill-start/-end`` walks a window
range instead of following the head.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import math
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path
from types import SimpleNamespace

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from neurons.base_node import BaseNode  # noqa: E402
from neurons.miner import common_args, finish_config, load_node_hparams  # noqa: E402
from neurons.trainer import Trainer  # noqa: E402
from templar_b200 import model_factory  # noqa: E402
from templar_b200.backends.chain import StaticWallet, make_subtensor  # noqa: E402
from templar_b200.distributed import dist_helper  # noqa: E402
from templar_b200.metrics import MetricsLogger  # noqa: E402

DEFAULT_TASKS = "arc_challenge,arc_easy,openbookqa,winogrande,piqa,hellaswag,mmlu"


def compute_bpb(total_nll_nats: float, total_bytes: int) -> float:
    """Bits per byte from a summed negative log-likelihood in nats."""
    return total_nll_nats / (math.log(2.0) * total_bytes) if total_bytes > 0 else float("inf")


class ModelCache:
    """Remembers which window's HF export sits in ``path`` so it is not rebuilt."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.meta = self.path / "cache_meta.json"

    def is_valid(self, window: int, version: str) -> bool:
        try:
            m = json.loads(self.meta.read_text())
            return m.get("window") == window and m.get("version") == version and (self.path / "config.json").exists()
        except Exception:  # noqa: BLE001
            return False

    def mark(self, window: int, version: str) -> None:
        self.path.mkdir(parents=True, exist_ok=True)
        self.meta.write_text(json.dumps({"window": window, "version": version, "time": time.time()}))

    def clear(self) -> None:
        shutil.rmtree(self.path, ignore_errors=True)


class Evaluator(BaseNode, Trainer):
    @staticmethod
    def evaluator_config(argv=None) -> SimpleNamespace:
        p = argparse.ArgumentParser(description="Evaluator script")
        common_args(p)
        # both spellings of every option: dashes, and the reference's underscores (neurons/evaluator.py:1234-1298)
        p.add_argument("--eval-interval", "--eval_interval", dest="eval_interval", type=int, default=600)
        p.add_argument("--tasks", type=str, default=DEFAULT_TASKS)
        p.add_argument("--batch-size", "--batch_size", dest="batch_size", type=int, default=4)
        p.add_argument("--custom-eval-path", "--custom_eval_path", dest="custom_eval_path", type=str, default=None,
                       help="directory of pre-tokenised shards (val_/eval_/test_/train_000000.npy) for the perplexity run")
        p.add_argument("--custom-eval-batches", type=int, default=16)
        p.add_argument("--skip-lm-eval", action="store_true")
        p.add_argument("--cache-dir", "--cache_dir", dest="cache_dir", type=str, default="./eval_model_cache")
        p.add_argument("--version", type=str, default=None, help="checkpoint version to follow (default: this build)")
        p.add_argument("--from-window", "--from_window", "--backfill-start", dest="backfill_start", type=int, default=None,
                       help="backfill: first window (inclusive); with only --to-window the network's start window is used")
        p.add_argument("--to-window", "--to_window", "--backfill-end", dest="backfill_end", type=int, default=None,
                       help="backfill: last window (inclusive); with only --from-window the newest complete checkpoint")
        p.add_argument("--no-follow", "--no_follow", dest="no_follow", action="store_true",
                       help="one shot: stop after the first evaluation / the backfill instead of following new checkpoints")
        p.add_argument("--force-reval", "--force_reval", dest="force_reval", action="store_true",
                       help="evaluate windows again even if this process has evaluated them")
        return finish_config(p.parse_args(argv))

    def __init__(self, config=None, hparams=None, store=None, subtensor=None):
        BaseNode.__init__(self)
        Trainer.__init__(self)
        self.config = config or Evaluator.evaluator_config()
        dist_helper.init_process_group(backend="nccl" if str(self.config.device).startswith("cuda") else "gloo",
                                       timeout_minutes=30)
        self.rank, self.world_size = dist_helper.rank, dist_helper.world_size
        self.local_rank, self.is_master = dist_helper.local_rank, dist_helper.is_master
        self.device = torch.device(self.config.device if not str(self.config.device).startswith("cuda")
                                   else f"cuda:{self.local_rank}")
        self.hparams = hparams or load_node_hparams(self.config)
        self.subtensor = subtensor or make_subtensor(self.config)
        self.metagraph = self.subtensor.metagraph(self.config.netuid)
        self.wallet = StaticWallet(self.config.wallet_hotkey or self.metagraph.hotkeys[-1])
        self.uid = self.metagraph.hotkeys.index(self.wallet.hotkey.ss58_address)
        self.version = self.config.version or tplr.__version__
        self.model = model_factory.initialize_torchtitan_model(self.hparams, role="evaluator", device=str(self.device),
                                                               world_size=self.world_size)
        self.tokenizer = self.hparams.tokenizer
        self.comms = tplr.Comms(wallet=self.wallet, config=self.config, hparams=self.hparams, uid=self.uid, store=store,
                                subtensor=self.subtensor)
        self.ckpt = tplr.DCPCheckpointer(self.comms, uid=self.uid, version=self.version, repo_root=".")
        self.cache = ModelCache(self.config.cache_dir)
        self.metrics_logger = MetricsLogger(prefix="E", uid=self.uid, config=self.config, role="evaluator",
                                            group="evaluator", job_type="eval") if self.is_master else None
        self.last_eval_window = -1
        self.eval_counter = 0

    # -- checkpoints --------------------------------------------------------------------------
    async def check_latest_checkpoint(self) -> int | None:
        """Newest window whose checkpoint is complete and not evaluated yet."""
        w = await self.ckpt._discover_latest(prefer_highest_staked=True)
        if w is None or w <= self.last_eval_window:
            return None
        return w if await self.ckpt.check_checkpoint_exists(window=w) else None

    async def load_window(self, window: int) -> tuple[int, int] | None:
        return await self.ckpt.download_and_load(model=self.model, window=window, shared_fs=True)

    def save_model_for_eval(self, window: int) -> Path | None:
        """HF export of the loaded weights (rank 0 writes; cached per window)."""
        if self.cache.is_valid(window, self.version):
            return self.cache.path
        if self.is_master:
            self.cache.clear()
        model_factory.convert_titan_to_hf(self.model, self.hparams, save_path=str(self.cache.path) if self.is_master else None,
                                          is_master=self.is_master)
        if self.is_master:
            self.cache.mark(window, self.version)
        dist_helper.safe_barrier("hf_export", self.local_rank)
        return self.cache.path

    # -- custom eval ---------------------------------------------------------------------------
    def _custom_eval_rows(self, n_batches: int):
        """(dataset, row indices of this rank, batch size, exact-bytes flag).  With ``--custom-eval-path`` the rows
        come from pre-tokenised shards (prefix val / eval / test / train, first shard, at most 1024 sequences split
        over the ranks, as the reference neurons/evaluator.py:697-745); otherwise seeded synthetic tokens."""
        hp = self.hparams
        path = getattr(self.config, "custom_eval_path", None)
        if path:
            prefix = next((p for p in ("val", "eval", "test") if (Path(path) / f"{p}_000000.npy").exists()), "train")
            ds = tplr.SharedShardedDataset(0, hp.sequence_length, self.rank, self.world_size, file_prefix=prefix,
                                           custom_path=path)
            total = min(1024, len(ds))
            per = total // self.world_size
            lo = self.rank * per
            hi = lo + per if self.rank < self.world_size - 1 else total
            return ds, list(range(lo, hi)), max(int(getattr(self.config, "batch_size", 4)), 1), True
        ds = tplr.SyntheticDataset(max(n_batches * hp.micro_batch_size * self.world_size, 8), hp.sequence_length,
                                   hp.model_config.vocab_size, seed=4242)
        rows = list(range(self.rank, len(ds), self.world_size))[: n_batches * hp.micro_batch_size]
        return ds, rows, hp.micro_batch_size, False

    def _decoded_bytes(self, ids: torch.Tensor) -> int | None:
        """UTF-8 bytes of the evaluated sequences (exact bits per byte), when the tokenizer can decode."""
        tok = getattr(self, "tokenizer", None)
        if tok is None or not hasattr(tok, "batch_decode"):
            return None
        try:
            texts = tok.batch_decode(ids.detach().cpu().tolist(), skip_special_tokens=True,
                                     clean_up_tokenization_spaces=False)
            return sum(len(t.encode("utf-8")) for t in texts)
        except Exception as e:  # noqa: BLE001
            tplr.logger.debug(f"[eval] decode for byte counts failed: {e}")
            return None

    async def run_custom_eval(self, n_batches: int | None = None) -> dict[str, float]:
        """Mean token cross entropy on held-out rows -> loss, perplexity and bits per byte.  Bytes are counted by
        decoding the evaluated sequences when a dataset path and a tokenizer are given, else taken as 4 per token."""
        n_batches = n_batches or self.config.custom_eval_batches
        ds, rows, bs, want_bytes = self._custom_eval_rows(n_batches)
        nll, toks, nbytes, exact = torch.zeros((), dtype=torch.float64, device=self.device), 0, 0, want_bytes
        self.model.eval()
        with torch.no_grad():
            for i in range(0, len(rows), bs):
                ids = torch.stack([torch.as_tensor(ds[r]) for r in rows[i:i + bs]]).to(self.device, dtype=torch.long)
                labels = self._labels(ids)
                loss = self.model.loss(ids, labels)
                n = int((labels != -100).sum())
                nll += loss.double() * n
                toks += n
                if exact:
                    got = self._decoded_bytes(ids)
                    exact = got is not None
                    nbytes += got or 0
                await asyncio.sleep(0)
        self.model.train()
        # fp32 on CUDA (NCCL has no fp64 sum on every build); the reduced tensor is the one that is read
        t = torch.tensor([float(nll), float(toks), float(nbytes), 1.0 if exact else 0.0],
                         dtype=torch.float32 if self.device.type == "cuda" else torch.float64, device=self.device)
        if dist_helper.is_distributed():
            torch.distributed.all_reduce(t)
        total_nll, total_tok, total_bytes = float(t[0]), max(float(t[1]), 1.0), float(t[2])
        all_exact = float(t[3]) >= (self.world_size if dist_helper.is_distributed() else 1) and total_bytes > 0
        loss = total_nll / total_tok
        return {"loss": loss, "perplexity": math.exp(min(loss, 50.0)),
                "bits_per_byte": compute_bpb(total_nll, int(total_bytes) if all_exact else int(total_tok * 4)),
                "tokens": total_tok, "bytes": total_bytes if all_exact else total_tok * 4.0,
                "bytes_exact": 1.0 if all_exact else 0.0}

    # -- lm_eval ---------------------------------------------------------------------------------
    def lm_eval_command(self, model_path: Path, tasks: list[str], output_dir: Path, num_fewshot: int = 0) -> list[str] | None:
        exe = shutil.which("lm_eval")
        if exe is None:
            return None
        args = f"pretrained={model_path},tensor_parallel_size={self.world_size},dtype=bfloat16,gpu_memory_utilization=0.8"
        cmd = [exe, "--model", "vllm", "--model_args", args, "--tasks", ",".join(tasks), "--batch_size", "auto",
               "--output_path", str(output_dir)]
        if num_fewshot > 0:
            cmd += ["--num_fewshot", str(num_fewshot)]
        return cmd

    def run_lm_eval(self, model_path: Path, tasks: list[str], window: int, global_step: int) -> dict[str, float]:
        """Rank 0 runs the harness in a clean (non-torchrun) environment; other ranks wait on a sentinel."""
        sentinel = Path(f"/tmp/tplr_lm_eval_done_{window}")
        if not self.is_master:
            while not sentinel.exists() and not self.stop_event.is_set():
                time.sleep(1.0)
            return {}
        out_dir = Path(f"/tmp/eval_{int(time.time())}")
        out_dir.mkdir(parents=True, exist_ok=True)
        cmd = self.lm_eval_command(model_path, tasks, out_dir)
        results: dict[str, float] = {}
        try:
            if cmd is None:
                tplr.logger.warning("lm_eval is not installed; downstream tasks skipped")
            else:
                env = {k: v for k, v in os.environ.items()
                       if not k.startswith(("TORCHELASTIC", "NCCL_")) and k not in
                       ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_NAME",
                        "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS")}
                env["VLLM_WORKER_MULTIPROC_METHOD"] = "spawn"
                rc = subprocess.Popen(cmd, env=env).wait()
                if rc in (0, 134):
                    results = self.parse_lm_eval_results(out_dir)
        finally:
            sentinel.write_text("done")
            shutil.rmtree(out_dir, ignore_errors=True)
        return results

    @staticmethod
    def parse_lm_eval_results(output_dir: Path) -> dict[str, float]:
        """``{task: score}`` from the newest ``results*.json`` (acc_norm preferred over acc)."""
        files = sorted(Path(output_dir).rglob("results*.json"), key=lambda p: p.stat().st_mtime)
        if not files:
            return {}
        data = json.loads(files[-1].read_text())
        out = {}
        for task, res in (data.get("results") or {}).items():
            for key in ("acc_norm,none", "acc,none", "acc_norm", "acc"):
                if key in res:
                    out[task] = float(res[key])
                    break
        return out

    # -- main -------------------------------------------------------------------------------------
    async def evaluate_window(self, window: int) -> dict | None:
        res = await self.load_window(window)
        if res is None:
            return None
        sync_window, global_step = res
        custom = await self.run_custom_eval()
        tasks = {}
        if not self.config.skip_lm_eval:
            path = self.save_model_for_eval(window)
            tasks = self.run_lm_eval(path, self.config.tasks.split(","), window, global_step)
        self.last_eval_window = window
        self.eval_counter += 1
        if self.metrics_logger is not None:
            self.metrics_logger.log("custom_evaluation", tags={"window": window, "global_step": global_step}, fields=custom)
            for task, score in tasks.items():
                self.metrics_logger.log("benchmark_task", tags={"window": window, "task": task}, fields={"score": score})
            if tasks:
                self.metrics_logger.log("benchmark_summary", tags={"window": window},
                                        fields={"num_tasks": len(tasks), "mean_score": sum(tasks.values()) / len(tasks)})
        tplr.logger.info(f"[eval] window {window} step {global_step}: loss={custom['loss']:.4f} ppl={custom['perplexity']:.2f} "
                         f"bpb={custom['bits_per_byte']:.4f} tasks={tasks}")
        return {"window": window, "global_step": global_step, **custom, "tasks": tasks}

    async def _backfill_range(self) -> tuple[int, int] | None:
        """Window range of a backfill run; an open end is resolved from the network (start window / newest
        complete checkpoint)."""
        lo, hi = self.config.backfill_start, self.config.backfill_end
        if lo is None and hi is None:
            return None
        if lo is None:
            lo = await self.comms.get_start_window()
        if hi is None:
            hi = await self.ckpt._discover_latest(prefer_highest_staked=True)
        if lo is None or hi is None:
            tplr.logger.warning("[eval] backfill range could not be resolved")
            return None
        return int(lo), int(hi)

    async def run(self):
        self.loop = asyncio.get_running_loop()
        self.comms.commitments = await self.comms.get_commitments()
        done: set[int] = set()
        rng = await self._backfill_range()
        if rng is not None:
            for w in range(rng[0], rng[1] + 1):
                if self.stop_event.is_set():
                    break
                if (w in done and not self.config.force_reval) or not await self.ckpt.check_checkpoint_exists(window=w):
                    continue
                if await self.evaluate_window(w) is not None:
                    done.add(w)
            if self.config.no_follow or (self.config.backfill_start is not None and self.config.backfill_end is not None):
                return
        while not self.stop_event.is_set():
            w = await self.check_latest_checkpoint() if self.is_master else None
            t = torch.tensor([w if w is not None else -1], dtype=torch.long, device=self.device)
            dist_helper.broadcast(t, src=0)
            w = int(t.item())
            if w >= 0 and (w not in done or self.config.force_reval):
                if await self.evaluate_window(w) is not None:
                    done.add(w)
            if self.config.no_follow or (self.config.max_windows and self.eval_counter >= self.config.max_windows):
                break
            try:
                await asyncio.wait_for(self.stop_event.wait(), timeout=self.config.eval_interval)
            except asyncio.TimeoutError:
                pass


def main():
    asyncio.run(Evaluator().main())


if __name__ == "__main__":
    main()
