"""Validator: keeps the consensus model in sync (gather + outer step), scores miners by the loss
change their individual gradients cause, maintains ratings / weights, publishes peer lists, the
start window, aggregated gradients, debug slices and DCP checkpoints.

    torchrun --standalone --nproc-per-node 4 neurons/validator.py --device cuda [--offline]

Behavioural parity with the reference's neurons/validator.py (state tensors of length 256, OpenSkill
Plackett–Luce ratings, binary moving average, sync score, slashing ladders for missing / invalid
gradients, poor sync, index overlap, inactivity and repeated negative evaluations, the piece-wise
emission schedule with a burn share, evaluation bins).  Scoring of one peer on a B200 is
``apply_single_peer`` (one fused kernel: unpack, clip, inverse DCT, theta0 - lr*g) → forward-only
losses → ``restore``; the snapshot never leaves HBM.
"""

from __future__ import annotations

import argparse
import asyncio
import contextlib
import hashlib
import os
import random
import sys
import time
from collections import deque
from datetime import datetime, timedelta, timezone
from types import SimpleNamespace

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from neurons.base_node import BaseNode  # noqa: E402
from neurons.miner import _noop_async, common_args, finish_config, load_node_hparams  # noqa: E402
from neurons.trainer import Trainer  # noqa: E402
from templar_b200.backends.chain import StaticWallet, make_subtensor  # noqa: E402
from templar_b200.distributed import dist_helper  # noqa: E402
from templar_b200.metrics import MetricsLogger, NullMetricsLogger  # noqa: E402,F401
from templar_b200.parallel.window_engine import peer_slice  # noqa: E402
from templar_b200.utils.ranges import phase  # noqa: E402
from templar_b200.utils.rating import PlackettLuce  # noqa: E402
from templar_b200.utils.tree import map_tensors, tensor_bytes, to_pinned_cpu  # noqa: E402
from templar_b200.wandb_ops import initialize_wandb  # noqa: E402

N_UIDS = 256


def min_power_normalization(logits: torch.Tensor, power: float = 2.0, epsilon: float = 1e-8) -> torch.Tensor:
    """``x^power / sum(x^power)``; zeros when the sum is below ``epsilon``."""
    if logits.dim() == 0:
        logits = logits.unsqueeze(0)
    p = logits ** power
    s = p.sum()
    return p / s if s > epsilon else torch.zeros_like(p)


@contextlib.contextmanager
def timer(name: str, wandb_obj=None, step=None, metrics_logger=None):
    """Time a phase: debug line, ``validator/<name>`` on the wandb run and a ``timing`` measurement, the last two only
    with a step to file them under (reference neurons/validator.py:76-87)."""
    t0 = time.perf_counter()
    try:
        yield
    finally:
        dt = time.perf_counter() - t0
        tplr.logger.debug(f"{name} took {dt:.2f}s")
        if wandb_obj is not None and step is not None:
            wandb_obj.log({f"validator/{name}": dt}, step=step)
        if metrics_logger is not None and step is not None:
            metrics_logger.log(measurement="timing", tags={"window": step}, fields={name: dt})


class Validator(BaseNode, Trainer):
    @staticmethod
    def validator_config(argv=None) -> SimpleNamespace:
        p = argparse.ArgumentParser(description="Validator script")
        common_args(p)
        return finish_config(p.parse_args(argv))

    def __init__(self, config=None, hparams=None, store=None, subtensor=None):
        BaseNode.__init__(self)
        Trainer.__init__(self)
        self.config = config or Validator.validator_config()
        dist_helper.init_process_group(backend="nccl" if str(self.config.device).startswith("cuda") else "gloo",
                                       timeout_minutes=30)
        self.rank, self.world_size = dist_helper.rank, dist_helper.world_size
        self.local_rank, self.is_master = dist_helper.local_rank, dist_helper.is_master
        self.device = torch.device(self.config.device if not str(self.config.device).startswith("cuda")
                                   else f"cuda:{self.local_rank}")
        self.config.device = str(self.device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.hparams = hparams or load_node_hparams(self.config)
        self.subtensor = subtensor or make_subtensor(self.config)
        self.metagraph = self.subtensor.metagraph(self.config.netuid)
        hotkey = self.config.wallet_hotkey or (self.metagraph.hotkeys[self.config.uid] if self.config.uid is not None
                                               else self.metagraph.hotkeys[0])
        self.wallet = StaticWallet(hotkey)
        self.uid = self.metagraph.hotkeys.index(hotkey)
        self.init_model(validator=False, meta=False)
        self.model_initialized = True
        heap = self.make_heap(validator=True)
        # one payload slot more than the largest gather: the uid under evaluation is staged beside the gathered peers
        self.attach_engine(heap=heap, validator=True, max_peers=int(getattr(self.hparams, "gather_peer_count", 8))
                           + int(getattr(self.hparams, "reserve_peer_count", 0)) + 1)
        self.transformer = tplr.compress.ChunkingTransformer(self.model, target_chunk=self.hparams.target_chunk)
        self.compressor = tplr.compress.TopKCompressor(use_quantization=False)
        self.init_optimizers_schedulers(validator=True)
        L = self.engine.layout
        self.xshapes = {s.name: L.xshape(s.name) for s in L.specs}
        self.totalks = {s.name: s.totalk for s in L.specs}
        self.bootstrap_version = getattr(self.hparams, "checkpoint_init_version", None)
        self.comms = tplr.Comms(wallet=self.wallet, save_location="/tmp", key_prefix="model", config=self.config,
                                hparams=self.hparams, uid=self.uid, store=store, subtensor=self.subtensor)
        self.ckpt = tplr.DCPCheckpointer(self.comms, uid=self.uid, version=tplr.__version__, repo_root=".")
        if self.is_master:
            self.comms.try_commit(self.wallet, self.comms.bucket)
        dist_helper.safe_barrier("post_commit", self.local_rank)
        # ---- scoring state -----------------------------------------------------------------
        z = lambda: torch.zeros(N_UIDS, dtype=torch.float32)  # noqa: E731
        self.gradient_scores, self.sync_scores, self.binary_indicator_scores = z(), z(), z()
        self.final_scores, self.binary_moving_averages, self.weights = z(), z(), z()
        self.openskill_model = PlackettLuce(beta=getattr(self.hparams, "openskill_beta", 25.0 / 6.0),
                                            tau=getattr(self.hparams, "openskill_tau", 25.0 / 300.0))
        self.openskill_ratings: dict[int, object] = {}
        self.current_window_scores: dict[int, float] = {}
        self.evaluated_uids: set[int] = set()
        self.eval_peers = self.comms.eval_peers
        self.inactive_scores: dict[int, tuple[int, float]] = {}
        self.inactivity_slash_rate = 0.25
        self.missing_gradient_slash_rate = 0.75
        self.sync_score_slash_rate = 0.75
        self.score_zero_threshold = 1e-4
        self.idx_similarity_slashing_rate = tplr.neurons.instantiate_slashing_multiplier()
        self.naughty_peers: dict[int, int] = {}
        self.naughty_peer_timeout = 20           # windows a mega-slashed peer stays excluded (reference neurons/validator.py:510-511)
        _uids = self.metagraph.uids.tolist() if hasattr(self.metagraph.uids, "tolist") else list(self.metagraph.uids)
        self.current_hotkeys = {int(u): hk for u, hk in zip(_uids, self.metagraph.hotkeys)}      # who owns which slot
        self.peer_eval_history: dict[int, deque] = {}
        self.eval_history_limit = 20
        self.consecutive_negative_count: dict[int, int] = {}
        self.consecutive_missing_gradient_count: dict[int, int] = {}
        self.missing_gradient_history: dict[int, deque] = {}
        self.missing_gradient_history_limit = 10
        self.excluded_from_gather: set[int] = set()
        self.exclusion_start_window: dict[int, int] = {}
        self.peers_last_eval_window: dict[int, int] = {}
        self.param_avg_change: dict[str, torch.Tensor] = {}
        self.prev_param_state: dict[str, torch.Tensor] = {}
        self.param_change_alpha = 0.2
        self.burn_uid = 1
        self.last_peer_update_window = None
        self.next_peers, self.next_reserve_peers, self.peers_update_window = None, None, -1
        self.comms.peers, self.comms.reserve_peers = [], []
        self.start_window = 0
        self.sync_window = 0
        self.global_step = 0
        self.window_step = 0
        self.eval_count = 0
        self.state_path = f"validator-state-{tplr.__version__}.pt"
        self.wandb = initialize_wandb("V", self.uid, self.config, "validator", "validation") if self.is_master else tplr.wandb_ops.NullRun()
        self.metrics_logger = MetricsLogger(prefix="V", uid=self.uid, config=self.config, role="validator",
                                            group="validator", job_type="validation") if self.is_master else None
        self.dataset_manager = self._dataset_manager()
        self.load_state()

    def _dataset_manager(self):
        from neurons.miner import Miner

        return Miner._dataset_manager(self)

    # ------------------------------------------------------------------------------------ #
    # state
    # ------------------------------------------------------------------------------------ #
    def _state_dict(self) -> dict:
        return {"global_step": self.global_step, "gradient_scores": self.gradient_scores.cpu(),
                "sync_scores": self.sync_scores.cpu(), "binary_indicator_scores": self.binary_indicator_scores.cpu(),
                "final_scores": self.final_scores.cpu(), "binary_moving_averages": self.binary_moving_averages.cpu(),
                "weights": self.weights.cpu(),
                "openskill_ratings": {int(u): {"mu": float(r.mu), "sigma": float(r.sigma), "ordinal": float(r.ordinal())}
                                      for u, r in self.openskill_ratings.items()},
                "naughty_peers": dict(getattr(self, "naughty_peers", {}) or {}),
                "consecutive_negative_count": dict(getattr(self, "consecutive_negative_count", {}) or {})}

    async def save_state(self):
        """Scores, ratings and the step counter to ``state_path``: rank 0 only (the other ranks hold no scores of their
        own, reference neurons/validator.py:3795-3811), written beside the file and renamed, so that a restart
        never reads half a file."""
        if not getattr(self, "is_master", True):
            return
        tmp = f"{self.state_path}.tmp{os.getpid()}"
        try:
            await asyncio.to_thread(torch.save, self._state_dict(), tmp)
            os.replace(tmp, self.state_path)
        except Exception as e:  # noqa: BLE001
            tplr.logger.warning(f"Failed to save validator state: {e}")
            if os.path.exists(tmp):
                os.remove(tmp)

    def load_state(self):
        """Rank 0 only, like ``save_state``: the scores live there (reference neurons/validator.py:3813-3887)."""
        if not getattr(self, "is_master", True) or not os.path.exists(self.state_path):
            return
        try:
            st = torch.load(self.state_path, map_location="cpu", weights_only=True)    # tensors, numbers and dicts only
            if not isinstance(st, dict):
                raise TypeError(f"state file holds a {type(st).__name__}, not a dict")
        except Exception as e:  # noqa: BLE001
            tplr.logger.warning(f"Failed to load validator state: {e}")
            return
        self.global_step = int(st.get("global_step", self.global_step))
        for name in ("gradient_scores", "sync_scores", "binary_indicator_scores", "final_scores",
                     "binary_moving_averages", "weights"):
            t = st.get(name)
            if torch.is_tensor(t) and t.shape == getattr(self, name).shape:
                setattr(self, name, t.float().clone())
        try:
            self.openskill_ratings = {int(u): self.openskill_model.rating(mu=float(d["mu"]), sigma=float(d["sigma"]), name=str(u))
                                      for u, d in st.get("openskill_ratings", {}).items()}
        except Exception as e:  # noqa: BLE001
            tplr.logger.warning(f"Failed to restore ratings: {e}")
        self.naughty_peers = {int(k): int(v) for k, v in st.get("naughty_peers", {}).items()}
        self.consecutive_negative_count = {int(k): int(v) for k, v in st.get("consecutive_negative_count", {}).items()}

    def reset_peer(self, uid: int) -> None:
        for t in (self.final_scores, self.weights, self.gradient_scores, self.binary_moving_averages,
                  self.binary_indicator_scores, self.sync_scores):
            t[uid] = 0.0
        for d in (self.openskill_ratings, self.eval_peers, self.inactive_scores, self.peer_eval_history,
                  self.consecutive_negative_count, self.consecutive_missing_gradient_count, self.missing_gradient_history,
                  self.exclusion_start_window):
            d.pop(uid, None)
        self.excluded_from_gather.discard(uid)

    # ------------------------------------------------------------------------------------ #
    # negative-evaluation bookkeeping
    # ------------------------------------------------------------------------------------ #
    def should_skip_negative_penalty(self) -> bool:
        """True when the 5th best score of the current window (or the worst, if fewer) is negative:
        the whole window went badly, so nobody is punished for it."""
        if not getattr(self, "current_window_scores", None):
            return False
        ranked = sorted(self.current_window_scores.values(), reverse=True)
        return ranked[min(4, len(ranked) - 1)] < 0

    def track_negative_evaluation(self, eval_uid: int) -> None:
        neg = bool(self.gradient_scores[eval_uid] < 0)
        if eval_uid not in self.peer_eval_history:
            self.peer_eval_history[eval_uid] = deque(maxlen=self.eval_history_limit)
            self.consecutive_negative_count[eval_uid] = 0
        self.peer_eval_history[eval_uid].append(neg)
        prev = self.consecutive_negative_count.get(eval_uid, 0)
        if neg:
            self.consecutive_negative_count[eval_uid] = prev + 1
        else:
            if prev > 0 and eval_uid in self.excluded_from_gather:
                self.excluded_from_gather.discard(eval_uid)
                self.exclusion_start_window.pop(eval_uid, None)
                tplr.logger.info(f"UID {eval_uid} re-included in gathering after a positive evaluation")
            self.consecutive_negative_count[eval_uid] = 0

    def apply_negative_evaluation_penalties(self) -> None:
        if not self.peer_eval_history:
            return
        skip = self.should_skip_negative_penalty()
        thr = getattr(self.hparams, "consecutive_negative_threshold", 3)
        for uid, hist in list(self.peer_eval_history.items()):
            if len(hist) >= 8 and sum(list(hist)[-8:]) / 8 > 0.5 and not skip and self.final_scores[uid] > 0:
                self.final_scores[uid] *= 0.25
                self.binary_moving_averages[uid] *= 0.25
                if self.final_scores[uid] < self.score_zero_threshold:
                    self.final_scores[uid] = 0.0
            if (getattr(self.hparams, "exclude_negative_peers", False) and self.consecutive_negative_count.get(uid, 0) >= thr
                    and uid not in self.excluded_from_gather and not skip):
                self.excluded_from_gather.add(uid)
                self.exclusion_start_window[uid] = self.sync_window
                tplr.logger.warning(f"UID {uid} excluded from gathering after repeated negative evaluations")

    def should_exclude_from_gather(self, uid: int) -> bool:
        if not getattr(self.hparams, "exclude_negative_peers", False):
            return False
        if self.consecutive_negative_count.get(uid, 0) < getattr(self.hparams, "consecutive_negative_threshold", 3):
            return False
        return not self.should_skip_negative_penalty()

    # ------------------------------------------------------------------------------------ #
    # ratings and weights
    # ------------------------------------------------------------------------------------ #
    def update_openskill_ratings(self) -> None:
        if len(self.current_window_scores) <= 1:
            return
        uids = list(self.current_window_scores)
        for u in uids:
            self.openskill_ratings.setdefault(u, self.openskill_model.rating(name=str(u)))
        rated = self.openskill_model.rate([[self.openskill_ratings[u]] for u in uids],
                                          scores=[self.current_window_scores[u] for u in uids])
        warm = getattr(self.hparams, "bma_warmup_windows", 10)
        thr = getattr(self.hparams, "bma_threshold", 0.10)
        for i, u in enumerate(uids):
            self.openskill_ratings[u] = rated[i][0]
            sync = float(self.sync_scores[u]) if u in self.evaluated_uids else 0.0
            bma = max(0.0, float(self.binary_moving_averages[u]))
            if self.current_window - self.start_window >= warm and bma < thr:
                bma = 0.0
            self.final_scores[u] = self.openskill_ratings[u].ordinal() * bma * sync
            if self.metrics_logger is not None:
                r = self.openskill_ratings[u]
                self.metrics_logger.log("validator_openskill", tags={"eval_uid": str(u), "window": int(self.sync_window)},
                                        fields={"mu": float(r.mu), "sigma": float(r.sigma), "ordinal": float(r.ordinal())})
        self.current_window_scores = {}

    def update_weights(self) -> None:
        """Emission schedule: the best ``gather_peer_count`` scores share ``gather_share`` of the
        non-burned weight on a linear ramp (first = ``gather_top_ratio`` x last), the next
        ``reserve_peer_count`` share the rest on a geometric decay, everybody else gets 0 and
        ``burn_rate`` goes to the burn uid."""
        hp = self.hparams
        self.weights.zero_()
        burn = max(0.0, min(1.0, getattr(hp, "burn_rate", 0.0)))
        share = getattr(hp, "gather_share", 0.75)
        g_n, r_n = getattr(hp, "gather_peer_count", 15), getattr(hp, "reserve_peer_count", 10)
        top, decay = getattr(hp, "gather_top_ratio", 2.0), getattr(hp, "reserve_decay_ratio", 0.75)
        ranked = sorted((u for u in self.evaluated_uids if self.final_scores[u] > 0),
                        key=lambda u: float(self.final_scores[u]), reverse=True)
        gather, reserve = ranked[:g_n], ranked[g_n:g_n + r_n]
        if gather:
            prof = torch.linspace(top, 1.0, len(gather))
            self.weights[gather] = (1.0 - burn) * share * prof / prof.sum()
        if reserve:
            prof = torch.tensor([decay ** i for i in range(len(reserve))])
            self.weights[reserve] = (1.0 - burn) * (1.0 - share) * prof / prof.sum()
        if gather and reserve:
            lo, hi = float(self.weights[gather].min()), float(self.weights[reserve].max())
            if hi > lo:
                self.weights[reserve] *= lo / hi * decay
        self.weights[self.burn_uid] = burn
        rest = float(self.weights.sum()) - burn
        if rest > 0:
            self.weights *= (1.0 - burn) / rest
            self.weights[self.burn_uid] = burn
        else:
            self.weights[self.burn_uid] = 1.0

    def update_and_log_evals(self) -> None:
        self.update_openskill_ratings()
        self.update_weights()
        rows = [(u, float(self.gradient_scores[u]), float(self.binary_moving_averages[u]), float(self.sync_scores[u]),
                 float(self.final_scores[u]), float(self.weights[u])) for u in sorted(self.evaluated_uids)]
        for u, g, b, s, f, w in rows:
            tplr.logger.info(f"UID {u:3d} grad={g:+.5f} bma={b:+.3f} sync={s:.3f} final={f:.4f} weight={w:.4f}")
            if self.metrics_logger is not None:
                self.metrics_logger.log("validator_scores", tags={"eval_uid": str(u), "window": int(self.sync_window)},
                                        fields={"gradient_score": g, "binary_moving_avg": b, "sync_score": s,
                                                "final_score": f, "weight": w})

    # ------------------------------------------------------------------------------------ #
    # slashing
    # ------------------------------------------------------------------------------------ #
    def _scale_score(self, uid: int, mult: float) -> None:
        if self.final_scores[uid] > 0:
            self.final_scores[uid] *= mult
            self.binary_moving_averages[uid] *= mult
            if self.final_scores[uid] < self.score_zero_threshold:
                self.final_scores[uid] = 0.0

    def record_missing_gradient_for_openskill(self, uid: int) -> None:
        self.openskill_ratings.setdefault(uid, self.openskill_model.rating(name=str(uid)))
        self.current_window_scores[uid] = float(getattr(self.hparams, "missing_gradient_penalty_score", -99.0))

    def slash_for_missing_gradient(self, eval_uid: int) -> None:
        if not self.is_master:
            return
        self._scale_score(eval_uid, self.missing_gradient_slash_rate)
        self.evaluated_uids.add(eval_uid)
        self.record_missing_gradient_for_openskill(eval_uid)

    def slash_for_invalid_gradient(self, eval_uid: int, error: Exception) -> None:
        if not self.is_master:
            return
        before = float(self.final_scores[eval_uid])
        if before > 0:
            self.final_scores[eval_uid] = 0.0
        self.evaluated_uids.add(eval_uid)
        self.record_missing_gradient_for_openskill(eval_uid)
        if self.metrics_logger is not None:
            self.metrics_logger.log("validator_slash", tags={"eval_uid": str(eval_uid), "reason_code": "invalid_gradient"},
                                    fields={"score_before": before, "score_after": float(self.final_scores[eval_uid]),
                                            "reason": str(error)[:255]})

    def slash_for_missing_gradients(self, skipped_uids: list[int], success_rate: float) -> None:
        """Escalating penalty for peers that were on the gather list but delivered nothing:
        x0.75, x0.5, then 0; 0 at once when the whole gather did badly; a peer missing in at least
        half of its last >= 8 gathers is reset and put on the naughty list."""
        for uid in skipped_uids:
            if not 0 <= uid < N_UIDS:
                continue
            hist = self.missing_gradient_history.setdefault(uid, deque(maxlen=self.missing_gradient_history_limit))
            hist.append(True)
            self.consecutive_missing_gradient_count[uid] = self.consecutive_missing_gradient_count.get(uid, 0) + 1
            n = self.consecutive_missing_gradient_count[uid]
            if len(hist) >= 8 and sum(hist) / len(hist) >= 0.5:
                self.naughty_peers[uid] = self.naughty_peer_timeout
                if self.final_scores[uid] > 0:
                    self.reset_peer(uid)
            else:
                if success_rate < getattr(self.hparams, "gather_peers_slash_threshold", 0.4):
                    mult = 0.0
                else:
                    mult = {1: 0.75, 2: 0.5}.get(n, 0.0)
                self._scale_score(uid, mult)
            self.evaluated_uids.add(uid)
            self.peers_last_eval_window[uid] = self.sync_window
            self.record_missing_gradient_for_openskill(uid)

    def note_delivered(self, uids: list[int]) -> None:
        for uid in uids:
            self.consecutive_missing_gradient_count[uid] = 0
            if uid in self.missing_gradient_history:
                self.missing_gradient_history[uid].append(False)

    def check_deregistered_uids(self, peers: dict) -> dict:
        """Drop from ``peers`` (uid -> overlap level, the repeat offenders included) every uid whose hotkey changed
        since the last look: the slot has a new owner, who must not inherit the old one's punishment - unless the new
        owner is itself caught copying outright ("mega").  Such a uid also leaves the list of repeat offenders
        (reference neurons/validator.py:4140-4170)."""
        mg = self.comms.metagraph
        uids = mg.uids.tolist() if hasattr(mg.uids, "tolist") else list(mg.uids)
        hotkeys = getattr(mg, "hotkeys", None) or [None] * len(uids)
        latest = {int(u): hk for u, hk in zip(uids, hotkeys)}
        known = getattr(self, "current_hotkeys", None)
        if known is None:
            known = latest                              # first look: nothing to compare with
        for uid in list(peers.keys()):
            if int(uid) not in latest:                  # not a slot of this subnet (any more): nothing to punish
                self.naughty_peers.pop(uid, None)
                peers.pop(uid, None)
            elif latest.get(uid) != known.get(uid) and peers.get(uid) != "mega":
                self.naughty_peers.pop(uid, None)
                peers.pop(uid, None)
        self.current_hotkeys = latest
        return peers

    def slash_from_overlap(self, idx_overlap: dict) -> None:
        peers = {uid: "max" for uid in self.naughty_peers}
        peers.update(idx_overlap.get("uids_over_thresh", {}))
        for uid, level in self.check_deregistered_uids(peers).items():
            before = float(self.final_scores[uid])
            mult = self.idx_similarity_slashing_rate.get(level, 0.5)
            if level in ("mega", "max"):
                self.reset_peer(uid)
                if level == "mega":
                    self.naughty_peers[uid] = self.naughty_peer_timeout
            if self.naughty_peers.get(uid):
                self.naughty_peers[uid] -= 1
                if self.naughty_peers[uid] <= 0:
                    self.naughty_peers.pop(uid)
            if before > 0:
                self.final_scores[uid] *= mult
                self.binary_moving_averages[uid] *= mult

    async def evaluate_miner_sync(self, eval_uid: int) -> dict:
        dbg = await self.comms.get(uid=str(eval_uid), window=self.sync_window - 1, key="debug", local=False, stale_retention=10)
        if not dbg.success or not isinstance(dbg.data, dict):
            return {"success": False, "error": "Failed to retrieve debug dictionary", "sync_score": 0.0}
        cmp = await tplr.neurons.compare_model_with_debug_dict(model=self.model, debug_dict=dbg.data, learning_rate=self.lr,
                                                               index_range=(10, 12), param_avg_change=self.param_avg_change)
        if not cmp["success"]:
            return {"success": False, "error": "Failed to compare model with debug dictionary", "sync_score": 0.0}
        x = min(cmp["avg_steps_behind"], 3.0)
        return {**cmp, "sync_score": max(0.0, (1.0 - x / 3.0) ** 2.5)}

    async def slash_for_poor_sync(self) -> None:
        res = await asyncio.gather(*(self.evaluate_miner_sync(u) for u in self.comms.peers))
        for info, uid in zip(res, self.comms.peers):
            if info.get("success", False) and self.metrics_logger is not None:
                self.metrics_logger.log("validator_sync_score",
                                        tags={"uid": str(uid), "window": int(self.sync_window), "global_step": int(self.global_step)},
                                        fields={k: float(info.get(k, 0.0)) for k in
                                                ("l2_norm", "avg_l2_norm", "avg_abs_diff", "max_diff", "avg_steps_behind",
                                                 "max_steps_behind", "sync_score")})
            if not info.get("success", False) or info.get("avg_steps_behind", 99.0) > self.hparams.sync_max_steps_behind:
                if self.final_scores[uid] > 0:
                    self.final_scores[uid] *= self.sync_score_slash_rate
                    self.binary_moving_averages[uid] *= self.sync_score_slash_rate

    def penalize_inactive_peers(self) -> None:
        """Peers that stopped uploading lose 25 % of their score per window and are reset after
        ``reset_inactivity_windows`` windows."""
        for uid in self.comms.inactive_peers:
            if uid not in self.inactive_scores:
                self.inactive_scores[uid] = (self.current_window, float(self.final_scores[uid]))
        for uid, (since, _) in list(self.inactive_scores.items()):
            if uid in self.eval_peers or uid in self.comms.active_peers:
                del self.inactive_scores[uid]
                continue
            if self.current_window - since > getattr(self.hparams, "reset_inactivity_windows", 3):
                self.reset_peer(uid)
                continue
            if self.final_scores[uid] > 0:
                before = float(self.final_scores[uid])
                self.final_scores[uid] *= (1.0 - self.inactivity_slash_rate)
                self.binary_moving_averages[uid] *= (1.0 - self.inactivity_slash_rate)
                if self.metrics_logger is not None:
                    self.metrics_logger.log("validator_inactivity",
                                            tags={"uid": str(uid), "window": int(self.current_window),
                                                  "global_step": int(self.global_step)},
                                            fields={"score_before": before, "score_after": float(self.final_scores[uid])},
                                            with_system_metrics=True, with_gpu_metrics=True)

    # ------------------------------------------------------------------------------------ #
    # peer lists and evaluation bins
    # ------------------------------------------------------------------------------------ #
    def select_initial_peers(self):
        hp = self.hparams
        need = hp.gather_peer_count + hp.reserve_peer_count
        inc = getattr(self.comms.metagraph, "I", None)
        inc = inc.tolist() if inc is not None else [0.0] * len(self.comms.metagraph.uids)
        ranked = [u for u, i in sorted(zip(self.comms.metagraph.uids.tolist(), inc), key=lambda x: -x[1])
                  if u in self.comms.active_peers and i > 0 and not self.should_exclude_from_gather(u)][:need]
        if len(ranked) < need:
            pool = [int(p) for p in self.comms.active_peers if p not in ranked and not self.should_exclude_from_gather(p)]
            ranked.extend(random.sample(pool, min(len(pool), need - len(ranked))))
        if len(ranked) < hp.minimum_peers:
            return None
        return ranked[:hp.gather_peer_count], ranked[hp.gather_peer_count:need]

    def select_next_peers(self):
        hp = self.hparams
        active, excluded = [], []
        for p in self.comms.active_peers:
            p = int(p)
            if p in self.naughty_peers:
                continue
            (excluded if self.should_exclude_from_gather(p) else active).append(p)
        if len(active) < hp.minimum_peers:
            excluded.sort(key=lambda u: self.consecutive_negative_count.get(u, 0))
            active.extend(excluded[: hp.minimum_peers - len(active)])
            if len(active) < hp.minimum_peers:
                return None
        active.sort(key=lambda u: float(self.weights[u]), reverse=True)
        need = hp.gather_peer_count + hp.reserve_peer_count
        return active[:hp.gather_peer_count], active[hp.gather_peer_count:need]

    async def create_and_post_peers(self) -> None:
        hp = self.hparams
        if self.last_peer_update_window is not None and self.sync_window - self.last_peer_update_window < hp.peer_replacement_frequency:
            return
        initial = self.last_peer_update_window is None
        sel = self.select_initial_peers() if initial else self.select_next_peers()
        if sel is None or not self.is_master:
            return
        self.last_peer_update_window = self.sync_window
        await self.comms.post_peer_list(peers=sel[0], reserve_peers=sel[1],
                                        first_effective_window=self.current_window + hp.peer_list_window_margin,
                                        sync_window=self.sync_window, initial_selection=initial)

    def bin_evaluation_peers(self, num_bins: int) -> dict[int, list[int]]:
        peers = list(self.eval_peers.keys())
        if len(peers) < num_bins * self.hparams.uids_per_window:
            return {0: peers}
        peers.sort(key=lambda u: float(self.openskill_ratings[u].ordinal()) if u in self.openskill_ratings else 0.0, reverse=True)
        per, rem = divmod(len(peers), num_bins)
        bins, start = {}, 0
        for i in range(num_bins):
            size = per + (1 if i < rem else 0)
            if start >= len(peers):
                break
            bins[i] = peers[start:start + size]
            start += size
        return bins

    def select_next_bin_for_evaluation(self, num_bins: int) -> int:
        return random.randint(0, num_bins - 1)

    def select_evaluation_uids_from_bin(self, bins: dict[int, list[int]], bin_idx: int) -> list[int]:
        peers = list(bins.get(bin_idx, bins.get(0, [])))
        k = min(self.hparams.uids_per_window, len(peers))
        return self.comms.weighted_random_sample_no_replacement(peers, [self.eval_peers[u] for u in peers], k)

    # ------------------------------------------------------------------------------------ #
    # gradients of a single peer
    # ------------------------------------------------------------------------------------ #
    def validate_gradient_data(self, uid: int, state_dict: dict) -> None:
        """Raises ``ValueError`` for malformed payloads (same checks as ``Comms.gather``)."""
        ok = self.comms.validate_payload(uid, {k: v for k, v in state_dict.items() if k != "metadata"}, self.totalks,
                                         self.xshapes, "cpu", set())
        if not ok:
            raise ValueError(f"UID {uid}: gradient failed validation")

    def _training_pool_digest(self, uid: int, window: int) -> tuple[str, int]:
        hp = self.hparams
        sampler = tplr.MinerSampler(self.dataset, uid, window, steps_per_window=hp.inner_steps, micro_bs=hp.micro_batch_size,
                                    batch_size=hp.batch_size, target_batch_size=hp.target_batch_size, rank=0, world_size=1)
        ids = sampler.ids_for_indices(sampler._global_indices().tolist())
        h = hashlib.blake2b(digest_size=16)
        h.update(np.asarray(sorted(ids), dtype=np.uint64).tobytes())
        return h.hexdigest(), len(ids)

    def log_digest_match(self, uid: int, meta: dict) -> bool:
        mine, n = self._training_pool_digest(uid, self.sync_window)
        ok = meta.get("sample_digest") == mine and meta.get("sample_count") == n
        if not ok:
            tplr.logger.warning(f"UID {uid}: sample digest mismatch (the miner did not train on its assigned data)")
        return ok

    def compute_peer_val_norms(self, gather_result):
        """Per-tensor median of the gathered peers' value norms: the clip reference for single-peer applies.
        With the number of peers staged in the engine: the engine's vector, one entry per tensor, computed on the
        device.  With a gather result: ``{"<name>vals": median norm}`` from its (dequantised) values, tensor by
        tensor (reference neurons/validator.py:3740-3770)."""
        if isinstance(gather_result, int):
            return self.engine.compute_peer_norms(gather_result).clone()
        state_dict = getattr(gather_result, "state_dict", None)
        if not state_dict:
            raise ValueError("Must have gather_result.state_dict to compute norms")
        out = {}
        for n, p in self.model.named_parameters():
            vals = getattr(state_dict, n + "vals", None)
            if vals is None:
                continue
            vals = self.compressor.maybe_dequantize_values(vals, getattr(state_dict, n + "quant_params", None), p.device)
            out[n + "vals"] = torch.median(torch.stack([torch.norm(v.float(), p=2) for v in vals]).to(p.device))
        return out

    async def upload_gather_results(self, gather_result) -> None:
        if not self.is_master or gather_result is None:
            return
        cpu = lambda o: o.cpu() if torch.is_tensor(o) else ([cpu(x) for x in o] if isinstance(o, (list, tuple)) else o)  # noqa: E731
        payload = {"state_dict": {k: cpu(v) for k, v in vars(gather_result.state_dict).items()},
                   "uids": list(gather_result.uids), "skipped_uids": list(gather_result.skipped_uids),
                   "success_rate": float(gather_result.success_rate)}
        await self.comms.put(state_dict=payload, window=self.sync_window, key="aggregator", global_step=self.global_step, local=False)

    # ------------------------------------------------------------------------------------ #
    # main loop
    # ------------------------------------------------------------------------------------ #
    async def run(self):
        self.loop = asyncio.get_running_loop()
        self.comms.start_commitment_fetcher()
        self.comms.commitments = await self.comms.get_commitments()
        self.comms.current_window = self.current_window
        if self.is_master:
            sw = await self.comms.get_start_window(retries=1, retry_delay=0.2)
            if sw is None:
                sw = self.current_window
                await self.comms.post_start_window(sw)
            self.start_window = sw
        t = torch.tensor([self.start_window], dtype=torch.long, device=self.device)
        dist_helper.broadcast(t, src=0)
        self.start_window = int(t.item())
        ok, win, step, boot = await tplr.neurons.load_checkpoint_with_fallback(self)
        if ok:
            await tplr.neurons.handle_checkpoint_catchup(self, ok, win, step, boot)
        await self.init_shard_schedule(validator=True)
        self.sync_window = self.current_window - 1
        done = 0
        while not self.stop_event.is_set():
            await self.wait_until_window(self.sync_window + getattr(self.hparams, "validator_offset", 1) + 1)
            self.sync_window += 1
            await self.run_window()
            done += 1
            if self.config.max_windows and done >= self.config.max_windows:
                self.stop_event.set()

    async def run_window(self) -> dict:
        """Gather, score a sample of peers, update ratings/weights, apply the outer step for ``sync_window``."""
        hp = self.hparams
        t_win = tplr.T()
        await self.save_state()
        await self.maybe_switch_shard(self.sync_window, validator=True)
        gather_result = None
        self._accept_window = (None, None)
        if self.is_master:
            await self.comms.refresh_active_peers()
            self.comms.update_peers_with_buckets()
            self.eval_peers = self.comms.eval_peers
            await self.create_and_post_peers()
            if self.config.peers is not None:
                self.comms.peers = list(self.config.peers)
            else:
                # the validator gathers from the list it (or a higher-staked validator) published, like the miners
                # (reference neurons/validator.py:1366-1373); until a first list is in effect: whoever is active
                await tplr.neurons.update_peers(instance=self, window=self.sync_window, peer_start=tplr.T())
                if not self.comms.peers:
                    self.comms.peers = sorted(int(u) for u in self.comms.active_peers
                                              if int(u) != self.uid)[:hp.gather_peer_count]
            self.penalize_inactive_peers()
            ts = await self.loop.run_in_executor(None, self.query_block_timestamp, (self.sync_window + 1) * hp.blocks_per_window)
            tmin = datetime.fromtimestamp(ts, tz=timezone.utc) if ts is not None else None
            tmax = tmin + timedelta(seconds=hp.time_window_delta_seconds) if tmin is not None else None
            if self.config.local:
                tmin = tmax = None
            self._accept_window = (tmin, tmax)
            if self.comms.peers:
                t_gather = tplr.T()
                gather_result = await self.comms.gather_with_reserve(
                    my_uid=self.uid, gather_uids=list(self.comms.peers), reserve_uids=list(self.comms.reserve_peers),
                    window=self.sync_window, key="gradient", timeout=self.gather_wait_seconds(), device="cpu",
                    local=False, totalks=self.totalks, xshapes=self.xshapes, compressor=self.compressor, time_min=tmin,
                    time_max=tmax, expected_compressed_params=self.expected_compressed_params)
                self.log_timing("gather", tplr.T() - t_gather)
        skip = torch.tensor([0 if (not self.is_master or gather_result is not None) else 1], dtype=torch.int32, device=self.device)
        dist_helper.broadcast(skip, src=0)
        for _ in range(hp.inner_steps):            # LR bookkeeping only
            if not self.should_skip_scheduler_step():
                self.inner_scheduler.step()
            self.inner_scheduler_step_count += 1
        scored = []
        if not bool(skip.item()):
            n_peers = self._stage_gather(gather_result)
            # every rank of a sharded engine counts the index overlap over its own chunks (a collective); the master
            # then judges the pairs
            self.overlap_matrix = None
            if self.engine.cuda and self.engine.world_size > 1 and n_peers >= 2:
                self.overlap_matrix = self.engine.index_overlap(n_peers)
            if self.is_master:
                asyncio.create_task(self.upload_gather_results(gather_result))
                overlap = await tplr.neurons.check_uid_index_overlap(self, gather_result, self.sync_window,
                                                                     overlap_threshold=getattr(hp, "idx_overlap_threshold", 0.9))
                if self.global_step > 20:
                    self.slash_from_overlap(overlap)
                await self.slash_for_poor_sync()
                self.slash_for_missing_gradients(list(gather_result.skipped_uids), float(gather_result.success_rate))
                self.note_delivered(list(gather_result.uids))
                self.offload_gather_results(gather_result, log=False)
            t_eval = tplr.T()
            scored = await self.score_peers(gather_result, n_peers, *self._accept_window)
            self.log_timing("evaluation", tplr.T() - t_eval)
            if self.is_master:
                self.apply_negative_evaluation_penalties()
                self.update_and_log_evals()
                if self.window_step % max(getattr(hp, "windows_per_weights", 1), 1) == 0:
                    pos = self.weights > 0
                    self.subtensor.set_weights(wallet=self.wallet, netuid=self.config.netuid,
                                               uids=torch.nonzero(pos).flatten().tolist(), weights=self.weights[pos].tolist())
            # consensus update for this window
            self.engine.window_open = True          # theta0 already holds the pre-update weights
            t_outer = tplr.T()
            with phase("Outer Step"):
                self.engine.outer_step(n_peers, lr=self.lr, include_own=False, base="theta0")
            self.log_timing("outer_step", tplr.T() - t_outer)
            self.engine.window_open = False
            self.global_step += 1
            if self.is_master:
                self._log_gradient_stats(n_peers)
                self._track_param_change()
                await self._publish_debug()
            if self.global_step % max(getattr(hp, "checkpoint_frequency", 10), 1) == 0:
                handle = await self.ckpt.save_local_async(model=self.model, window=self.sync_window,
                                                          sync_window=self.sync_window, global_step=self.global_step)
                await self.ckpt.upload(window=self.sync_window, background=True, wait_for=handle, initial_sleep_s=0.0,
                                       pointer_poll_interval_s=1.0, pointer_poll_timeout_s=60.0)
        self.window_step += 1
        out = {"sync_window": self.sync_window, "scored": scored, "global_step": self.global_step,
               "window_time": tplr.T() - t_win, "gathered": list(getattr(gather_result, "uids", []) or [])}
        if self.metrics_logger is not None:
            self.metrics_logger.log("validator_window_v2", tags={"window": int(self.sync_window)},
                                    fields={"window_time": out["window_time"], "n_scored": len(scored),
                                            "n_gathered": len(out["gathered"])}, with_system_metrics=True, with_gpu_metrics=True)
        dist_helper.safe_barrier("validator_end_window", self.local_rank)
        return out

    def offload_gather_results(self, gather_result, *, log: bool = True) -> None:
        """Move the gathered state dict to pinned host memory (reference neurons/validator.py:92-156).  The
        engine keeps its own packed copy of every staged peer in device slots, so after ``_stage_gather``
        the dict is only needed again for uploads and per-UID bookkeeping."""
        if gather_result is None or not getattr(self.hparams, "offload_gather_results", True):
            return
        state = getattr(gather_result, "state_dict", None)
        if state is None or getattr(gather_result, "_offloaded", None) == "cpu":
            return
        t0 = time.time()
        on_device = tensor_bytes(map_tensors(state, lambda t: t)) if log else 0
        map_tensors(state, to_pinned_cpu)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        gather_result._offloaded = "cpu"
        if log:
            tplr.logger.info(f"[GatherOffload] gathered payloads -> pinned host | {on_device / 1e6:.1f} MB "
                             f"in {time.time() - t0:.3f}s")

    def load_gather_results_to_device(self, gather_result, device, *, log: bool = True) -> None:
        """Inverse of :meth:`offload_gather_results` (reference neurons/validator.py:158-219)."""
        if gather_result is None or getattr(gather_result, "_offloaded", None) != "cpu":
            return
        state = getattr(gather_result, "state_dict", None)
        if state is None:
            return
        device, t0 = torch.device(device), time.time()
        map_tensors(state, lambda t: t if t.device == device else t.to(device, non_blocking=True))
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        gather_result._offloaded = None
        if log:
            tplr.logger.info(f"[GatherOffload] gathered payloads -> {device.type} | "
                             f"{tensor_bytes(state) / 1e6:.1f} MB in {time.time() - t0:.3f}s")

    def _stage_gather(self, gather_result) -> int:
        """Put the gathered payloads into the engine's device slots (all ranks); returns the peer count."""
        eng = self.engine
        sd = vars(gather_result.state_dict) if (self.is_master and gather_result is not None) else None
        n = (len(gather_result.uids) - len(getattr(gather_result, "local_ranks", None) or {})) if sd is not None else 0
        n = min(n, eng.cfg.max_peers - 1)          # the last slot is kept for the uid under evaluation
        t = torch.tensor([n], dtype=torch.int32, device=self.device)
        dist_helper.broadcast(t, src=0)
        n = int(t.item())
        if eng.world_size == 1:
            for j in range(n):
                eng.load_peer_payload(j, peer_slice(sd, j))
        else:
            eng.distribute_peer_payloads(sd, n)
        self.staged_peers = n                       # slot j holds uids[j]: the overlap check reads the slots
        return n

    # -- the reference's per-peer evaluation API on top of the engine ---------------------------------------- #
    def _save_model_state(self):
        """Remember the weights that the per-peer applies start from (reference neurons/validator.py:274-288: a copy
        of the local shards on the host).  Here the engine's window snapshot is that state and stays on the device."""
        self.engine.snapshot()
        return "engine-snapshot"

    def _restore_model_state(self, state=None) -> None:
        """Back to the saved weights (reference neurons/validator.py:290-302)."""
        self.engine.restore()

    def update_model_with_gradient(self, model, eval_uid: int, eval_state_dict: dict, clip_norm_dict=None) -> None:
        """Apply one peer's payload alone, scaled by ``lr * eval_lr_factor``, its values clipped per tensor to the
        median norm of the gathered peers (reference neurons/validator.py:3563-3738).  ``clip_norm_dict``: the
        per-tensor medians as a ``[n_params]`` tensor (:meth:`compute_peer_val_norms`) or the reference's
        ``{name + "vals": norm}`` dict.  Raises ``ValueError`` for a payload that does not decode to finite values."""
        eng = self.engine
        median = clip_norm_dict
        if isinstance(clip_norm_dict, dict):
            median = torch.full((eng.layout.n_params,), float("inf"), device=eng.device)
            for sp in eng.layout.specs:
                if sp.name + "vals" in clip_norm_dict:
                    median[sp.index] = float(clip_norm_dict[sp.name + "vals"])
        slot = eng.cfg.max_peers - 1
        eng.stage_single_peer(eval_state_dict if self.is_master else None, slot)
        eng.apply_single_peer(slot, self.lr * getattr(self.hparams, "eval_lr_factor", 1.0), median)
        bad = bool(eng.check_status() & 3)             # bad index / non-finite value met while decoding the payload
        bad = dist_helper.any_ok(bad, self.device, "eval_payload_bad")    # every rank decodes its own chunks: agree
        if bad:
            eng.restore()
            raise ValueError(f"Invalid gradient from peer {eval_uid}: payload did not decode to finite values")

    def log_sync_score(self, eval_uid: int, sync_result: dict) -> None:
        """``validator_sync_score`` measurement and the wandb series of one peer (reference neurons/validator.py:
        851-903)."""
        keys = ("l2_norm", "avg_l2_norm", "avg_abs_diff", "max_diff", "avg_steps_behind",
                "interquartile_mean_steps_behind", "max_steps_behind")
        vals = {k: float(sync_result.get(k, 99.0)) for k in keys}
        tplr.log_with_context(level="info", message=f"Sync average steps behind: {vals['avg_steps_behind']:.3f}, "
                              f"interquartile mean: {vals['interquartile_mean_steps_behind']:.3f}",
                              sync_window=self.sync_window, current_window=self.current_window, eval_uid=eval_uid)
        if not self.is_master:
            return
        if self.wandb is not None:
            names = {"max_diff": "sync_max_diff"}
            self.wandb.log({f"validator/sync/{names.get(k, k)}/{eval_uid}": v for k, v in vals.items()}, step=self.global_step)
        if self.metrics_logger is not None:
            self.metrics_logger.log("validator_sync_score",
                                    tags={"uid": str(eval_uid), "window": int(self.sync_window),
                                          "global_step": int(self.global_step)}, fields=vals)

    async def fetch_eval_gradient(self, uid: int, time_min, time_max) -> dict | None:
        """Master only: the upload of the uid that is about to be scored, fetched from the uid's own bucket with
        the window's acceptance times, checked like a gathered payload and against the data the uid was assigned.
        A missing, too early or too late upload is slashed as missing; a malformed one as invalid (reference
        neurons/validator.py:1912-1957).  A transport error is neither: the uid is only skipped.  Returns the
        payload, or ``None`` when the uid cannot be scored this window."""
        try:
            res = await self.comms.get(uid=str(uid), window=self.sync_window, key="gradient", local=False, stale_retention=10,
                                       time_min=time_min, time_max=time_max)
        except Exception as e:  # noqa: BLE001
            tplr.logger.warning(f"[validator] fetch gradient failed for {uid}: {e} - marking invalid")
            return None
        if res.status == "ERROR":
            tplr.logger.warning(f"[validator] fetch gradient failed for {uid} (transport) - marking invalid")
            return None
        if not res.success or not isinstance(res.data, dict):
            tplr.logger.info(f"UID {uid}: no acceptable gradient for window {self.sync_window} ({res.status}); slashing")
            self.slash_for_missing_gradient(uid)
            return None
        state = res.data
        if (state.get("metadata") or {}).get("dummy"):               # the liveness marker of a miner that has not trained yet
            self.slash_for_missing_gradient(uid)
            return None
        try:
            self.validate_gradient_data(uid, state)
            missing = self.expected_compressed_params - set(state)
            if missing:
                raise ValueError(f"UID {uid}: payload lacks {len(missing)} expected entries, e.g. {sorted(missing)[0]}")
            self.log_digest_match(uid, state.get("metadata", {}) or {})
        except Exception as e:  # noqa: BLE001
            tplr.logger.warning(f"UID {uid}: invalid gradient ({e}); slashing")
            self.slash_for_invalid_gradient(uid, e)
            return None
        return state

    async def score_peers(self, gather_result, n_peers: int, time_min=None, time_max=None) -> list[dict]:
        """For a sample of the *evaluation* peers (whether or not they are on the gather list): fetch the uid's own
        upload, check it, and measure the loss on the uid's assigned data and on random data before and after
        applying that gradient alone; update gradient / binary / sync scores.  The loop ends early when the chain
        moves to the next window (reference neurons/validator.py:1879-2318)."""
        hp, eng = self.hparams, self.engine
        if self.is_master:
            bins = self.bin_evaluation_peers(getattr(hp, "num_evaluation_bins", 5))
            uids = self.select_evaluation_uids_from_bin(bins, self.select_next_bin_for_evaluation(max(len(bins), 1)))
            if not uids:                                   # no eligible evaluation peer known yet: score who delivered
                uids = list(gather_result.uids)[: hp.uids_per_window]
            pad = uids[: N_UIDS] + [-1] * (N_UIDS - len(uids))
        else:
            pad = [-1] * N_UIDS
        t = torch.tensor(pad, dtype=torch.int32, device=self.device)
        dist_helper.broadcast(t, src=0)
        uids = [int(u) for u in t.tolist() if u >= 0]
        median = self.compute_peer_val_norms(n_peers)
        eval_slot = eng.cfg.max_peers - 1                  # spare slot: the gathered peers keep theirs for the outer step
        if n_peers > eval_slot:
            raise RuntimeError("the engine has no spare payload slot for the uid under evaluation")
        eng.snapshot()
        random_seed = random.randint(1000, 10_000_000) if self.is_master else 0
        rs = torch.tensor([random_seed], dtype=torch.long, device=self.device)
        dist_helper.broadcast(rs, src=0)
        random_seed = int(rs.item())
        self.sampler.set_window_uid(random_seed, self.sync_window)
        lb_rand_sum, lb_rand_n = await self.evaluate_model(self.model, self.loader)
        loss_before_random = lb_rand_sum / max(lb_rand_n, 1)
        out = []
        eval_window = self.current_window
        for uid in uids:
            t0 = time.time()
            state, stop = None, False
            if self.is_master:
                stop = (not self.config.local) and self.current_window != eval_window
                if stop:
                    tplr.logger.info(f"Window changed during evaluation (was {eval_window}, now {self.current_window}); "
                                     f"leaving the evaluation loop after {len(out)}/{len(uids)} uids")
                else:
                    self.peers_last_eval_window[uid] = self.sync_window
                    state = await self.fetch_eval_gradient(uid, time_min, time_max)
            flags = torch.tensor([int(state is not None), int(stop)], dtype=torch.int32, device=self.device)
            dist_helper.broadcast(flags, src=0)                       # every rank takes the master's view
            if bool(flags[1].item()):
                break
            if not bool(flags[0].item()):
                continue
            self.sampler.set_window_uid(uid, self.sync_window)
            s, n = await self.evaluate_model(self.model, self.loader)
            loss_before_own = s / max(n, 1)
            try:
                self.update_model_with_gradient(self.model, uid, state, median)
            except ValueError as e:                      # decoded to non-finite values: every rank sees the same status
                if self.is_master:
                    self.slash_for_invalid_gradient(uid, e)
                continue
            s, n = await self.evaluate_model(self.model, self.loader)
            loss_after_own = s / max(n, 1)
            self.sampler.set_window_uid(random_seed, self.sync_window)
            s, n = await self.evaluate_model(self.model, self.loader)
            loss_after_random = s / max(n, 1)
            eng.restore()
            self.eval_count += 1
            score = (loss_before_random - loss_after_random) / loss_before_random if loss_before_random > 0 else 0.0
            imp_own = (loss_before_own - loss_after_own) / loss_before_own if loss_before_own > 0 else 0.0
            self.gradient_scores[uid] = score
            if self.is_master:
                self.track_negative_evaluation(uid)
                self.openskill_ratings.setdefault(uid, self.openskill_model.rating(name=str(uid)))
                self.current_window_scores[uid] = float(score)
                self.binary_indicator_scores[uid] = 1.0 if imp_own > score else -1.0
                a = hp.binary_score_ma_alpha
                self.binary_moving_averages[uid] = (1 - a) * self.binary_moving_averages[uid] + a * self.binary_indicator_scores[uid]
                sync = await self.evaluate_miner_sync(uid)
                self.sync_scores[uid] = float(sync.get("sync_score", 0.0))
                self.log_sync_score(uid, sync)
            self.evaluated_uids.add(uid)
            self.peers_last_eval_window[uid] = self.sync_window
            out.append({"uid": uid, "gradient_score": float(score), "loss_before_own": loss_before_own,
                        "loss_after_own": loss_after_own, "loss_before_random": loss_before_random,
                        "loss_after_random": loss_after_random, "seconds": time.time() - t0})
        eng.window_open = False
        return out

    def _log_gradient_stats(self, n_peers: int) -> None:
        """``validator_gradient_stats`` (reference neurons/validator.py:2466-2545): statistics of the gathered
        peers' whole-payload norms, read from the per-(peer, tensor) norms the clip computation left on the
        device (one small read-back per window)."""
        if self.metrics_logger is None or n_peers <= 0:
            return
        eng = self.engine
        np_ = eng.layout.n_params
        per_peer = eng.peer_norms[: n_peers * np_].view(n_peers, np_).double().pow(2).sum(dim=1).sqrt().cpu()
        finite = per_peer[torch.isfinite(per_peer)]
        if finite.numel() == 0:
            return
        w = float(eng.store.master_shard.double().pow(2).sum().sqrt())
        mean = float(finite.mean())
        self.metrics_logger.log("validator_gradient_stats",
                                tags={"window": int(self.sync_window), "global_step": int(self.global_step)},
                                fields={"mean_grad_norm": mean, "max_grad_norm": float(finite.max()),
                                        "min_grad_norm": float(finite.min()), "median_grad_norm": float(finite.median()),
                                        "grad_norm_std": float(finite.std()) if finite.numel() > 1 else 0.0,
                                        "mean_weight_norm": w, "grad_to_weight_ratio": mean / w if w > 0 else 0.0})

    def log_timing(self, name: str, seconds: float) -> None:
        """``timing`` measurement for one phase of the window (reference neurons/validator.py:76-87)."""
        if self.metrics_logger is not None:
            self.metrics_logger.log("timing", tags={"window": int(self.sync_window)}, fields={name: float(seconds)})

    def _track_param_change(self) -> None:
        a = self.param_change_alpha
        for name, cur in tplr.neurons.param_samples(self.model, 10, 12).items():
            cur = cur.float().cpu()
            if name in self.prev_param_state:
                d = (cur - self.prev_param_state[name]).abs()
                self.param_avg_change[name] = d.clone() if name not in self.param_avg_change else \
                    self.param_avg_change[name] * (1 - a) + d * a
            self.prev_param_state[name] = cur

    async def _publish_debug(self) -> None:
        dbg = {name + "_debug": v.float().cpu().tolist() for name, v in tplr.neurons.param_samples(self.model, 0, 2).items()}
        await self.comms.put(state_dict=dbg, uid=str(self.uid), window=self.sync_window, key="debug", local=False)


def main():
    try:
        import uvloop

        uvloop.install()
    except Exception:  # noqa: BLE001
        pass
    asyncio.run(Validator().main())


if __name__ == "__main__":
    main()
