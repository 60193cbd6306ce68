"""Evaluator: follows the published checkpoints and reports perplexity / bits-per-byte and
(where a harness is installed) downstream-task scores.

    torchrun --standalone --nproc-per-node 2 neurons/evaluator.py --device cuda [--offline]

Flow (reference: neurons/evaluator.py:1113-1222): read the start window → find the newest complete
checkpoint (``_LATEST.json`` pointer or listing, completeness gate; rank 0 decides, the others follow) →
load it (DCP reshards to this topology) → custom evaluation (cross entropy → perplexity and bits per
byte) → convert to HF layout into a per-window cache → ``lm_eval`` in a subprocess when available (the
model leaves the GPU first; rank 0 runs the child, the other ranks wait on a sentinel file) → metrics →
old exports and local checkpoints pruned → sleep ``eval_interval``.  With nothing published and no
bootstrap version the untrained weights are evaluated once as the baseline.  ``--from-window/--to-window``
walk a window range first.
"""

from __future__ import annotations

import argparse
import asyncio
import contextlib
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
from templar_b200.metrics import MetricsLogger, NullMetricsLogger  # noqa: E402,F401
from templar_b200.wandb_ops import NullRun, initialize_wandb  # noqa: E402

DEFAULT_TASKS = "arc_challenge,arc_easy,openbookqa,winogrande,piqa,hellaswag,mmlu"


def compute_bpb(total_nll_nats: float, total_bytes: float) -> float:
    """Bits per byte from a summed negative log-likelihood in nats."""
    return total_nll_nats / (math.log(2.0) * total_bytes) if total_bytes > 0 else float("inf")


def loss_to_bpb(total_loss_nats: float, total_tokens: int, *, total_bytes: int | None = None,
                bytes_per_token: float | None = None) -> float:
    """Bits per byte from a summed cross entropy in nats: exact with the byte count of the evaluated text, estimated
    with an average number of bytes per token (reference neurons/evaluator.py:120-141)."""
    if total_tokens <= 0:
        return float("inf")
    if total_bytes is not None and total_bytes > 0:
        return compute_bpb(total_loss_nats, total_bytes)
    if bytes_per_token is not None and bytes_per_token > 0:
        return compute_bpb(total_loss_nats, total_tokens * bytes_per_token)
    raise ValueError("Provide total_bytes or bytes_per_token to compute bpb.")


_loss_to_bpb = loss_to_bpb


class ModelCache:
    """HF exports of evaluated windows, one directory per window under ``base_dir/<version>`` (the same window
    number can exist under several versions; reference: neurons/evaluator.py:144-210)."""

    WEIGHT_FILES = ("model.safetensors", "pytorch_model.bin")

    def __init__(self, base_dir: str | Path = Path("models/cache"), namespace: str | None = None):
        self.base_dir = Path(base_dir) / namespace if namespace else Path(base_dir)
        self.base_dir.mkdir(parents=True, exist_ok=True)

    def get_path(self, window: int) -> Path:
        return self.base_dir / f"window_{window}"

    def exists(self, window: int) -> bool:
        """A usable export: the config and a weight file (whole or sharded), as the reference's cache checks."""
        p = self.get_path(window)
        has_weights = any((p / f).exists() for f in self.WEIGHT_FILES) or any(p.glob("model-*.safetensors"))
        return (p / "config.json").exists() and has_weights

    def mark(self, window: int) -> None:
        p = self.get_path(window)
        p.mkdir(parents=True, exist_ok=True)
        (p / "cache_meta.json").write_text(json.dumps({"window": window, "time": time.time()}))

    def clear(self, window: int) -> None:
        shutil.rmtree(self.get_path(window), ignore_errors=True)

    def windows(self) -> list[int]:
        out = []
        if self.base_dir.is_dir():
            for d in self.base_dir.iterdir():
                tail = d.name[len("window_"):] if d.is_dir() and d.name.startswith("window_") else ""
                if tail.isdigit():
                    out.append(int(tail))
        return sorted(out)

    def cleanup(self, keep_latest: int = 2) -> list[int]:
        """Remove all but the ``keep_latest`` highest windows; returns the removed ones."""
        ws = self.windows()
        drop = ws[:-keep_latest] if keep_latest > 0 else ws
        for w in drop:
            self.clear(w)
        return drop


@contextlib.contextmanager
def pause_ddp_for_lm_eval(tag: str, stop=None):
    """The hand-over of a node's GPUs to a child process that only rank 0 starts.  All ranks arrive at a barrier;
    inside the block rank 0 runs the child and touches the sentinel file the block yields when it is done; on the
    way out the other ranks wait for that file (or for ``stop``, the node's shutdown event), all ranks meet at a
    second barrier and rank 0 removes the file: the sentinel of one evaluation is never seen by the next
    (reference: neurons/evaluator.py:76-106)."""
    if dist_helper.is_distributed():
        dist_helper.safe_barrier(f"pause_ddp_enter_{tag}", dist_helper.local_rank)
    sentinel = Path(f"/tmp/tplr_eval_done_{tag}")
    try:
        yield sentinel
    finally:
        if not dist_helper.is_master:
            while not sentinel.exists() and not (stop is not None and stop.is_set()):
                time.sleep(0.25)
        if dist_helper.is_distributed():
            dist_helper.safe_barrier(f"pause_ddp_exit_{tag}", dist_helper.local_rank)
        if dist_helper.is_master:
            sentinel.unlink(missing_ok=True)


def release_device_memory(label: str = "") -> None:
    """Collect garbage and give cached device memory back to the driver, so that a child process (the task
    harness with its own inference engine) finds the GPU empty."""
    import gc

    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        torch.cuda.ipc_collect()
        free, total = torch.cuda.mem_get_info()
        tplr.logger.debug(f"[eval] {label}: {free / 2**30:.1f} of {total / 2**30:.1f} GiB free")


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
        self._initialize_or_load_model()
        self.tokenizer = self.hparams.tokenizer
        self.comms = tplr.Comms(wallet=self.wallet, config=self.config, hparams=self.hparams, uid=self.uid, store=store,
                                subtensor=self.subtensor)
        self.ckpt = tplr.DCPCheckpointer(self.comms, uid=self.uid, version=self.version, repo_root=".")
        self.model_cache = ModelCache(self.config.cache_dir, namespace=self.version)
        self.metrics_logger = MetricsLogger(prefix="E", uid=self.uid, config=self.config, role="evaluator",
                                            group="evaluator", job_type="eval") if self.is_master else None
        self.wandb = initialize_wandb("E", self.uid, self.config, "evaluator", "eval") if self.is_master else NullRun()
        self.tasks = [t.strip() for t in str(self.config.tasks or "").split(",") if t.strip()]
        # the options that steer the loop, as attributes (a driver or a test may change them on a live node)
        self.from_window, self.to_window = self.config.backfill_start, self.config.backfill_end
        self.no_follow, self.force_reval = bool(self.config.no_follow), bool(self.config.force_reval)
        self.eval_interval = self.config.eval_interval
        self.eval_counter = 0
        self.evaluated_windows: set[int] = set()
        self.last_discovered_window: int | None = None
        self.baseline_evaluated = False
        self.start_window: int | None = None

    def _initialize_or_load_model(self) -> None:
        """The model with fresh weights on this node's device (a checkpoint is loaded into it per evaluated window)."""
        self.model = model_factory.initialize_torchtitan_model(hparams=self.hparams, role="evaluator", device=str(self.device),
                                                               world_size=self.world_size)

    @property
    def cache(self) -> ModelCache:
        return self.model_cache

    @property
    def last_eval_window(self) -> int:
        return max(self.evaluated_windows, default=-1)

    # -- checkpoints --------------------------------------------------------------------------
    async def check_latest_checkpoint(self) -> int | None:
        """Newest window whose checkpoint is complete and not evaluated yet."""
        w = await self.ckpt._discover_latest(prefer_highest_staked=True)
        if w is None:
            return None
        self.last_discovered_window = w
        if w in self.evaluated_windows and not self.force_reval:
            return None
        return w if await self.ckpt.check_checkpoint_exists(window=w) else None

    async def load_window(self, window: int) -> tuple[int, int] | None:
        return await self.ckpt.download_and_load(model=self.model, window=window, shared_fs=True)

    def save_model_for_eval(self, window: int) -> Path | None:
        """HF export of the loaded weights into this window's cache directory (rank 0 writes; an export that is
        already complete is reused).  None when the export failed."""
        path = self.cache.get_path(window)
        if not self.cache.exists(window):
            if self.is_master:
                self.cache.clear(window)
            try:
                model_factory.convert_titan_to_hf(self.model, self.hparams, save_path=str(path) if self.is_master else None,
                                                  is_master=self.is_master)
                if self.is_master:
                    self.cache.mark(window)
            except Exception as e:  # noqa: BLE001
                tplr.logger.error(f"[eval] export of window {window} failed: {e}")
                path = None
        dist_helper.safe_barrier("hf_export", self.local_rank)
        return path

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
        with pause_ddp_for_lm_eval(f"{getattr(self, 'uid', 0)}_{window}", stop=getattr(self, "stop_event", None)) as sentinel:
            if not self.is_master:
                return {}
            return self._run_lm_eval_master(model_path, tasks, window, global_step, sentinel)

    run_lm_eval_multi_gpu = run_lm_eval              # the reference's name (one child drives all GPUs of the node)

    def _run_lm_eval_master(self, model_path: Path, tasks: list[str], window: int, global_step: int,
                            sentinel: Path) -> dict[str, float]:
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
                if torch.cuda.is_available():
                    env["CUDA_VISIBLE_DEVICES"] = ",".join(str(i) for i in range(torch.cuda.device_count()))
                t0 = time.perf_counter()
                rc = subprocess.Popen(cmd, env=env).wait()
                # the inference engine of the harness may abort on exit (134) after it has written its results
                if rc in (0, 134):
                    scored = self.parse_lm_eval_results(out_dir, with_metric=True)
                    results = {t: v for t, (m, v) in scored.items()}
                    self._log_task_scores(scored, window, global_step)
                tplr.logger.info(f"[eval] lm_eval exit code {rc} after {time.perf_counter() - t0:.1f} s, "
                                 f"{len(results)} task results")
        finally:
            sentinel.write_text("done")
            if results or cmd is None:
                shutil.rmtree(out_dir, ignore_errors=True)
            else:
                tplr.logger.warning(f"[eval] no task results; {out_dir} kept for inspection")
        return results

    def _log_task_scores(self, scored: dict[str, tuple[str, float]], window: int, global_step: int) -> None:
        """``benchmark_task`` per task and one ``benchmark_summary`` (reference: neurons/evaluator.py:640-690)."""
        if self.metrics_logger is not None:
            for task, (metric, value) in scored.items():
                self.metrics_logger.log("benchmark_task", tags={"task": task, "metric": metric, "global_step": global_step,
                                                                "window": window}, fields={"score": float(value)})
            self.metrics_logger.log("benchmark_summary", tags={"global_step": global_step, "window": window},
                                    fields={"num_tasks": len(scored), "global_step": global_step,
                                            "mean_score": sum(v for _, v in scored.values()) / max(len(scored), 1)})
        self.wandb.log({**{f"evaluator/benchmark/{t}/{m}": v for t, (m, v) in scored.items()},
                        "evaluator/benchmark/num_tasks": len(scored)}, step=global_step)

    @staticmethod
    def parse_lm_eval_results(output_dir: Path, with_metric: bool = False) -> dict:
        """``{task: score}`` (``{task: (metric, score)}`` with ``with_metric``) from the newest JSON file under
        ``output_dir`` - the harness writes into a sub-directory named after the model - with the normalised
        accuracy preferred over the plain one (reference: neurons/evaluator.py:573-695)."""
        files = [f for f in Path(output_dir).rglob("*.json") if f.is_file()]
        if not files:
            return {}
        try:
            data = json.loads(max(files, key=lambda f: f.stat().st_mtime).read_text())
        except (OSError, ValueError) as e:
            tplr.logger.error(f"[eval] unreadable result file under {output_dir}: {e}")
            return {}
        out = {}
        for task, res in (data.get("results") or {}).items():
            for key in ("acc_norm,none", "acc,none", "acc_norm", "acc"):
                if isinstance(res, dict) and res.get(key) is not None:
                    out[task] = (key, float(res[key])) if with_metric else float(res[key])
                    break
            else:
                tplr.logger.warning(f"[eval] {task}: no accuracy metric in the results")
        return out

    # -- main -------------------------------------------------------------------------------------
    async def evaluate_window(self, window: int, is_baseline: bool = False) -> dict | None:
        """Evaluate the checkpoint of ``window`` (or, as the baseline, the freshly initialised weights).  The global
        step comes from the checkpoint's sidecar; an older checkpoint without one gets ``window - start_window``
        (reference: neurons/evaluator.py:871-985).  None when the checkpoint could not be loaded."""
        if window in self.evaluated_windows and not self.force_reval:
            tplr.logger.info(f"[eval] window {window} already evaluated")
            return {"window": window, "skipped": True}
        global_step = 0
        if not is_baseline and window > 0:
            try:
                res = await self.load_window(window)
            except Exception as e:  # noqa: BLE001
                tplr.logger.error(f"[eval] loading the checkpoint of window {window} failed: {e}")
                return None
            if res is None:
                return None
            loaded_window, global_step = res
            if loaded_window != window:
                tplr.logger.error(f"[eval] asked for window {window}, the checkpoint is of window {loaded_window}")
                return None
            if global_step is None or global_step < 0:
                global_step = window - (self.start_window if self.start_window is not None else window)
        global_step = max(int(global_step), 0)           # backfill before the start window: no negative steps
        custom = await self.run_custom_eval()
        tasks: dict[str, float] = {}
        if self.tasks and not self.config.skip_lm_eval:
            path = self.save_model_for_eval(window)
            if path is None:
                return None
            # the harness loads the export into an inference engine of its own: hand it an empty GPU
            on_gpu = self.device.type == "cuda" and shutil.which("lm_eval") is not None
            if on_gpu:
                self.model.to("cpu")
                release_device_memory("before lm_eval")
            try:
                tasks = self.run_lm_eval(path, self.tasks, window, global_step)
            finally:
                if on_gpu:
                    self.model.to(self.device)
        self.evaluated_windows.add(window)
        self.eval_counter = getattr(self, "eval_counter", 0) + 1
        if self.metrics_logger is not None:
            self.metrics_logger.log("custom_evaluation", tags={"window": window, "global_step": global_step,
                                                               "baseline": int(is_baseline)}, fields=custom)
        self.wandb.log({f"evaluator/custom/{k}": custom[k] for k in ("loss", "perplexity", "bits_per_byte")}, step=global_step)
        tplr.logger.info(f"[eval] window {window} step {global_step}{' (baseline)' if is_baseline else ''}: "
                         f"loss={custom['loss']:.4f} ppl={custom['perplexity']:.2f} bpb={custom['bits_per_byte']:.4f} tasks={tasks}")
        if self.is_master:                                # one export and one local checkpoint stay on disk
            self.cache.cleanup(keep_latest=1)
            self.ckpt.cleanup_local_checkpoints(keep_latest=1)
        return {"window": window, "global_step": global_step, "baseline": is_baseline, **custom, "tasks": tasks}

    def _from_master(self, *values: int | None) -> list[int | None]:
        """Rank 0's values on every rank (None travels as -1): what the object store shows can differ between
        two ranks that look a moment apart, and the ranks have to take the same branch."""
        t = torch.tensor([-1 if v is None else int(v) for v in values], dtype=torch.long, device=self.device)
        dist_helper.broadcast(t, src=0)
        return [None if v < 0 else v for v in t.tolist()]

    def _stopping(self) -> bool:
        ev = getattr(self, "stop_event", None)
        return ev is not None and ev.is_set()

    async def _resolve_to_window(self) -> int | None:
        """Upper end of a backfill that was given none: the newest complete checkpoint, as rank 0 sees it."""
        latest = None
        if self.is_master:
            try:
                w = await self.ckpt._discover_latest(prefer_highest_staked=True)
                if w is not None and await self.ckpt.check_checkpoint_exists(window=w):
                    latest = w
            except Exception as e:  # noqa: BLE001
                tplr.logger.error(f"[eval] resolving the newest checkpoint failed: {e}")
        return self._from_master(latest)[0]

    async def _backfill_range(self) -> tuple[int, int] | None:
        """Window range of a backfill run; an open end is resolved from the network (start window / newest
        complete checkpoint) by rank 0.  A reversed range is put in order."""
        lo, hi = self.from_window, self.to_window
        if lo is None and hi is None:
            return None
        if self.is_master:
            if lo is None:
                lo = self.start_window if self.start_window is not None else await self.comms.get_start_window()
        if hi is None:
            hi = await self._resolve_to_window()           # every rank takes part in its broadcast
        lo, hi = self._from_master(lo, hi)
        if lo is None or hi is None:
            tplr.logger.warning("[eval] backfill range could not be resolved")
            return None
        return (int(lo), int(hi)) if lo <= hi else (int(hi), int(lo))

    async def backfill_range(self) -> list[int]:
        """Evaluate every complete checkpoint of the range; returns the evaluated windows."""
        rng = await self._backfill_range()
        out: list[int] = []
        if rng is None:
            return out
        tplr.logger.info(f"[eval] backfilling windows {rng[0]}..{rng[1]} of version {self.version}")
        for w in range(rng[0], rng[1] + 1):
            if self._stopping():
                break
            ready = (await self.ckpt.check_checkpoint_exists(window=w)) if self.is_master else None
            if not self._from_master(int(bool(ready)))[0]:
                continue
            rep = await self.evaluate_window(w)
            if rep and not (isinstance(rep, dict) and rep.get("skipped")):
                out.append(w)
            dist_helper.safe_barrier(f"backfill_win_{w}", self.local_rank)
        return out

    async def run(self):
        """Start window -> newest checkpoint (or, when the network has published none and no bootstrap version is
        configured, the freshly initialised weights as the baseline) -> backfill range if one was asked for ->
        follow new checkpoints every ``eval_interval`` seconds (reference: neurons/evaluator.py:1113-1222)."""
        self.loop = asyncio.get_running_loop()
        self.comms.commitments = await self.comms.get_commitments()
        sw = None
        if self.is_master:
            # on a network the start window always appears (the validators publish it) and the evaluator waits for it;
            # an offline run may have no validator at all and then counts its steps from the window it starts in
            offline = bool(getattr(self.config, "local", False))
            sw = await self.comms.get_start_window(version=self.version, retries=3 if offline else -1,
                                                   retry_delay=0.5 if offline else 10.0)
            if sw is None:
                sw = int(self.current_window)
                tplr.logger.warning(f"[eval] no start window published; counting steps from window {sw}")
        self.start_window = self._from_master(sw)[0]
        backfill = self.from_window is not None or self.to_window is not None
        first = True
        while not self._stopping():
            if not first:
                self.comms.commitments = await self.comms.get_commitments()
            w = self._from_master((await self.check_latest_checkpoint()) if self.is_master else None)[0]
            if w is not None:
                await self.evaluate_window(w)
                dist_helper.safe_barrier("eval_complete", self.local_rank)
            elif (first and not backfill and not self.baseline_evaluated and self.start_window is not None
                  and not getattr(self.hparams, "checkpoint_init_version", None)):
                # nothing published yet and no bootstrap version: the untrained weights give the curve its origin
                if await self.evaluate_window(self.start_window, is_baseline=True) is not None:
                    self.baseline_evaluated = True
            if first and backfill:
                await self.backfill_range()
            first = False
            limit = getattr(self.config, "max_windows", 0)
            if self.no_follow or (isinstance(limit, int) and limit > 0 and getattr(self, "eval_counter", 0) >= limit):
                break
            if backfill and self.from_window is not None and self.to_window is not None:
                break                                     # a closed range is a one-shot job
            ev = getattr(self, "stop_event", None)
            if ev is None:
                await asyncio.sleep(self.eval_interval)
                continue
            try:
                await asyncio.wait_for(ev.wait(), timeout=self.eval_interval)
            except asyncio.TimeoutError:
                pass

    def cleanup(self) -> None:
        """Release the model's device memory and the loggers at shutdown."""
        if getattr(self, "model", None) is not None:
            self.model.to("cpu")
            release_device_memory("shutdown")
        ml = getattr(self, "metrics_logger", None)
        if ml is not None and hasattr(ml, "close"):
            ml.close()
        wb = getattr(self, "wandb", None)
        if wb is not None:
            wb.finish()


get_config = Evaluator.evaluator_config


def main():
    node = Evaluator()
    try:
        asyncio.run(node.main())
    finally:
        node.cleanup()


if __name__ == "__main__":
    main()
