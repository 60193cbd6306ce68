"""Training mixin: model / optimizer / scheduler construction, the inner loop, evaluation,
the outer step and optimizer-state offload.

Parity: the reference's neurons/trainer.py:41-1115 (same method names and hparams keys: outer
``SGD(lr=outer_learning_rate)``, inner AdamW or Muon, ``LinearLR`` warm-up into cosine annealing or
the anneal-mode up/down ramp, the LR "flatten" window, per-restart warm-up scaling of the LR).

The inner loop is restructured for a B200: step boundaries come from the sampler's
``grad_accum_steps`` (no per-micro-batch flag all-reduce), losses stay on the device and are
read back once per inner step, and with a :class:`~templar_b200.parallel.window_engine.WindowEngine`
the optimizer step is the fused reduce / clip / AdamW / publish sequence on the rank's shard.
"""

from __future__ import annotations

import asyncio
import math
from contextlib import nullcontext

import torch
import torch.distributed as dist
from torch.optim import SGD
from torch.optim import lr_scheduler

import templar_b200 as tplr
from templar_b200 import model_factory
from templar_b200.distributed import dist_helper
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine
from templar_b200.utils.ranges import labelled, phase


def _opt_cfg(hparams) -> tuple[str, dict, dict]:
    oc = getattr(hparams, "optimizer", {}) or {}
    kind = oc.get("type", "adamw").lower()
    spec = oc.get(kind, {}) or {}
    return kind, spec, spec.get("scheduler", {}) or {}


class Trainer:
    def __init__(self):
        self.inner_scheduler_step_count = 0

    # ------------------------------------------------------------------------------------ #
    # data
    # ------------------------------------------------------------------------------------ #
    def set_dataloader(self, validator: bool = False) -> None:
        self.dataset = self.dataset_manager.active_dataset
        hp = self.hparams
        shared = dict(dataset=self.dataset, uid=self.uid, window=self.current_window, steps_per_window=hp.inner_steps,
                      micro_bs=hp.micro_batch_size, rank=self.rank, world_size=self.world_size)
        if validator:
            self.sampler = tplr.EvalSampler(**shared, batch_size=hp.target_batch_size,
                                            validation_bs=hp.validator_sample_micro_bs * hp.micro_batch_size)
        else:
            self.sampler = tplr.MinerSampler(**shared, batch_size=hp.batch_size, target_batch_size=hp.target_batch_size)
        self.loader = torch.utils.data.DataLoader(dataset=self.dataset, sampler=self.sampler,
                                                  batch_size=hp.micro_batch_size, pin_memory=torch.cuda.is_available())
        tplr.logger.info("[Run] dataset + sampler ready")

    async def init_shard_schedule(self, validator: bool = False) -> None:
        """Open the dataset shard that belongs to ``global_step`` and remember it (reference neurons/miner.py:
        425-456, neurons/validator.py:1261-1275)."""
        hp = self.hparams
        epoch, shard = tplr.compute_shard_state(self.global_step, getattr(hp, "outer_steps_per_shard", 455),
                                                getattr(hp, "shard_reset_outer_step", None))
        await self.dataset_manager.initialize_datasets(shard)
        dist_helper.safe_barrier("dataset_init_complete", getattr(self, "local_rank", 0))
        self.set_dataloader(validator=validator)
        self._shard_epoch, self._shard_index = epoch, shard

    async def maybe_switch_shard(self, window: int, validator: bool = False) -> bool:
        """At the start of a window: move to the next shard when ``global_step`` has crossed a shard boundary, or
        re-open the schedule when the reset step was passed (reference neurons/miner.py:497-527).  Anneal mode
        stays on its single shard.  Returns whether the dataset changed."""
        hp = self.hparams
        if (getattr(hp, "anneal_mode", {}) or {}).get("enabled", False):
            return False
        epoch, shard = tplr.compute_shard_state(self.global_step, getattr(hp, "outer_steps_per_shard", 455),
                                                getattr(hp, "shard_reset_outer_step", None))
        last_epoch, last_shard = getattr(self, "_shard_epoch", 0), getattr(self, "_shard_index", 0)
        if epoch != last_epoch:
            tplr.logger.info(f"Resetting shard schedule at outer_step {self.global_step} to shard {shard}")
            await self.dataset_manager.initialize_datasets(shard)
        elif shard > last_shard:
            tplr.logger.info(f"Swapping dataset after {self.global_step} outer steps at window {window}")
            await self.dataset_manager.swap_datasets()
        else:
            return False
        self.set_dataloader(validator=validator)
        dist_helper.safe_barrier("sync_shard_switch", getattr(self, "local_rank", 0))
        self._shard_epoch, self._shard_index = epoch, shard
        return True

    def get_expected_params(self) -> set[str]:
        out = set()
        for name, _ in self.model.named_parameters():
            out.update((name + "idxs", name + "vals", name + "quant_params"))
        return out

    # ------------------------------------------------------------------------------------ #
    # model / optimizers
    # ------------------------------------------------------------------------------------ #
    def init_model(self, validator: bool = False, meta: bool = False):
        role = "validator" if validator else "miner"
        if meta:
            self.model = model_factory.create_meta_model(hparams=self.hparams, role=role, world_size=self.world_size)
        else:
            self.model = model_factory.initialize_torchtitan_model(hparams=self.hparams, role=role, device=str(self.device),
                                                                   world_size=self.world_size)
        self.expected_compressed_params = self.get_expected_params()
        self.tokenizer = self.hparams.tokenizer

    def engine_topology(self, validator: bool = False) -> dict:
        """Which ranks share one copy of the sharded state and which ranks are replicas of each other.

        ``torchtitan.dp_replicate = R`` on a miner (the reference's DDP setting, src/tplr/model_factory.py:139-160,
        and with ``world_size / R > 1`` ranks per copy the hybrid layout torchtitan calls HSDP) cuts the node's
        ranks into R copies of ``world_size / R`` consecutive ranks: the state is sharded inside a copy (peer
        memory of that copy's symmetric heap) and the gradient shards are summed over the copies with one
        all-reduce per inner step.  Everything else, and every validator, is one copy over all ranks: on one
        NVSwitch box every peer is equally near, so a second copy of the state buys nothing there.
        Collective: every rank creates every group."""
        if getattr(self, "_engine_topology", None) is not None:
            return self._engine_topology
        tt = getattr(self.hparams, "torchtitan", None)
        replicas = int((tt.get("dp_replicate", 1) if isinstance(tt, dict) else getattr(tt, "dp_replicate", 1)) or 1)
        world = self.world_size
        topo = dict(shard_rank=self.rank, shard_world=world, shard_group=None, replicate_group=None, replicas=1)
        if not validator and replicas > 1 and world > 1:
            if world % replicas:
                raise ValueError(f"World size ({world}) must be divisible by torchtitan.dp_replicate ({replicas})")
            per = world // replicas
            shard_groups = [dist.new_group(list(range(r * per, (r + 1) * per))) for r in range(replicas)]
            replicate_groups = [dist.new_group(list(range(s, world, per))) for s in range(per)]
            topo = dict(shard_rank=self.rank % per, shard_world=per,
                        shard_group=shard_groups[self.rank // per] if per > 1 else None,
                        replicate_group=replicate_groups[self.rank % per], replicas=replicas)
        self._engine_topology = topo
        return topo

    def make_heap(self, validator: bool = False, timeout_s: float = 30.0):
        """The symmetric heap of this rank's copy of the sharded state (None on CPU or for a copy of one rank)."""
        topo = self.engine_topology(validator)
        if topo["shard_world"] <= 1 or torch.device(self.device).type != "cuda":
            return None
        from templar_b200.parallel.symmetric import SymmetricHeap

        return SymmetricHeap.create(self.device, topo["shard_rank"], topo["shard_world"], group=topo["shard_group"],
                                    timeout_s=timeout_s)

    def attach_engine(self, heap=None, max_peers: int | None = None, validator: bool = False) -> WindowEngine:
        """Put the (materialised) model on the flat store and the fused per-window kernels."""
        hp = self.hparams
        topo = self.engine_topology(validator)
        kind, spec, _ = _opt_cfg(hp)
        adam = (getattr(hp, "optimizer", {}) or {}).get("adamw", {}) or {}
        kw = dict(
            topk=getattr(hp, "topk_compression", 32), target_chunk=getattr(hp, "target_chunk", 64),
            use_dct=getattr(hp, "use_dct", False), momentum_decay=getattr(hp, "momentum_decay", 0.95),
            outer_lr=float(getattr(hp, "outer_learning_rate", 0.4)), outer_update=getattr(hp, "outer_update", "sgd"),
            outer_weight_decay=float(getattr(hp, "outer_weight_decay", 0.0)),
            inner_lr=float(adam.get("learning_rate", 2e-4)), betas=tuple(adam.get("betas", [0.9, 0.95])),
            eps=float(adam.get("eps", 1e-8)), weight_decay=float(adam.get("weight_decay", 0.1)), max_grad_norm=1.0,
            max_peers=max_peers or (getattr(hp, "gather_peer_count", 8) + getattr(hp, "reserve_peer_count", 0)),
            # 8-bit value codes on the wire (what the reference's miner always sends); the statistics are per
            # whole tensor, so a sharded CUDA engine needs the symmetric heap for it (the CPU path merges the
            # payload with a collective)
            quantize=bool(getattr(hp, "payload_quantization", False))
            and (topo["shard_world"] == 1 or heap is not None or torch.device(self.device).type == "cpu"),
            quant_bins=min(int(getattr(hp, "quantization_bins", 256)), 256),
            quant_range=float(getattr(hp, "quantization_range", 6)),
            # torchtitan.shard_params: bf16 weights and fp32 gradients held as shards too (what the reference's
            # dp_shard does with FSDP2, src/tplr/model_factory.py:215-332), for models whose whole weights and
            # gradients do not fit beside the activations; on CUDA with several ranks it needs the symmetric heap
            shard_params=self._shard_params(heap),
            gather_buffers=int((lambda tt: (tt.get("gather_buffers", 0) if isinstance(tt, dict)
                                            else getattr(tt, "gather_buffers", 0)) or 0)(getattr(hp, "torchtitan", None))))
        kw.update(self._muon_engine_args(kind, spec))
        cfg = EngineConfig(**kw)
        self.engine = WindowEngine(self.model, cfg, device=self.device, rank=topo["shard_rank"],
                                   world_size=topo["shard_world"], group=topo["shard_group"], heap=heap,
                                   replicate_group=topo["replicate_group"], replicate_size=topo["replicas"])
        return self.engine

    def _shard_params(self, heap) -> bool:
        tt = getattr(self.hparams, "torchtitan", None)
        want = bool(tt.get("shard_params", False) if isinstance(tt, dict) else getattr(tt, "shard_params", False))
        if not want:
            return False
        if torch.device(self.device).type == "cuda" and self.engine_topology()["shard_world"] > 1 and heap is None:
            raise ValueError("torchtitan.shard_params on several GPUs needs the symmetric heap")
        return True

    def _muon_engine_args(self, kind: str, spec: dict) -> dict:
        """Engine settings for ``optimizer.type == "muon"``: the same groups, LR scales and decays that
        :meth:`get_inner_optimizer` builds for the unfused path."""
        if kind != "muon":
            return {}
        return dict(inner_optimizer="muon", inner_lr=float(spec.get("learning_rate", 0.02)),
                    muon_momentum=float(spec.get("momentum", 0.95)), muon_weight_decay=float(spec.get("weight_decay", 0.01)),
                    muon_aux_lr_scale=(("head", float(spec.get("head_lr_scale", 0.5))),
                                       ("embed", float(spec.get("embed_lr_scale", 0.5))),
                                       ("scalar", float(spec.get("scalar_lr_scale", 0.2)))),
                    betas=(0.9, 0.95), eps=1e-8, weight_decay=float(getattr(self.hparams, "weight_decay", 0.1)))

    def init_optimizers_schedulers(self, validator: bool = False):
        self.lr = float(self.hparams.outer_learning_rate)
        self.outer_optimizer = SGD(self.model.parameters(), lr=self.lr)
        self.inner_optimizer = self.get_inner_optimizer(validator)
        self.inner_scheduler = self.get_inner_scheduler()
        self.inner_scheduler_step_count = 0
        _, _, sched = _opt_cfg(self.hparams)
        self.warmup_inner_steps = sched.get("warmup_inner_steps", 0)
        self.warmup_steps_taken = 0
        tplr.logger.info("[Init] optimizers & schedulers constructed")

    def get_inner_optimizer(self, validator: bool):
        kind, spec, _ = _opt_cfg(self.hparams)
        lr = spec.get("learning_rate", 2e-4 if kind == "adamw" else 0.02)
        if validator or getattr(self, "engine", None) is not None:
            # the engine owns the optimizer state (fused AdamW, or Muon with auxiliary Adam on the flat
            # buffers); this stand-in carries the LR for the scheduler
            dummy = torch.nn.Parameter(torch.zeros(1), requires_grad=False)
            return torch.optim.SGD([dummy], lr=lr)
        if kind == "adamw":
            fused = next(self.model.parameters()).is_cuda
            return torch.optim.AdamW(self.model.parameters(), lr=lr, weight_decay=spec.get("weight_decay", 0.1),
                                     betas=tuple(spec.get("betas", [0.9, 0.95])), eps=spec.get("eps", 1e-8), fused=fused)
        if kind == "muon":
            from templar_b200.muon import SingleDeviceMuonWithAuxAdam

            hidden, embed, scalar, head = [], [], [], []
            for name, p in self.model.named_parameters():
                if not p.requires_grad:
                    continue
                if p.ndim >= 2 and "embed" not in name and "lm_head" not in name and name != "output.weight":
                    hidden.append(p)
                elif "embed" in name:
                    embed.append(p)
                elif "lm_head" in name or name == "output.weight":
                    head.append(p)
                else:
                    scalar.append(p)
            if not hidden:
                raise ValueError("Model must have 2D weight matrices for Muon")
            wd = getattr(self.hparams, "weight_decay", 0.1)
            groups = []
            for ps, key, dflt in ((head, "head_lr_scale", 0.5), (embed, "embed_lr_scale", 0.5), (scalar, "scalar_lr_scale", 0.2)):
                if ps:
                    groups.append(dict(params=ps, lr=lr * spec.get(key, dflt), weight_decay=wd, betas=(0.9, 0.95),
                                       eps=1e-8, use_muon=False))
            groups.append(dict(params=hidden, lr=lr, momentum=spec.get("momentum", 0.95),
                               weight_decay=spec.get("weight_decay", 0.01), use_muon=True))
            return SingleDeviceMuonWithAuxAdam(groups)
        raise ValueError(f"Unknown optimizer type: {kind}. Supported: 'adamw', 'muon'")

    def get_inner_scheduler(self):
        kind, spec, sched = _opt_cfg(self.hparams)
        lr = spec.get("learning_rate", 2e-4 if kind == "adamw" else 0.02)
        anneal = getattr(self.hparams, "anneal_mode", {}) or {}
        opt = self.inner_optimizer
        if anneal.get("enabled", False):
            warm = anneal.get("warmup_inner_steps", 100)
            peak, floor = anneal.get("peak_lr_factor", 0.5), anneal.get("eta_min_factor", 0.0)
            total = anneal.get("decay_outer_steps", 550) * self.hparams.inner_steps
            up = lr_scheduler.LinearLR(opt, start_factor=1e-6, end_factor=peak, total_iters=warm)
            down = lr_scheduler.LinearLR(opt, start_factor=peak, end_factor=floor, total_iters=total)
            return lr_scheduler.SequentialLR(opt, schedulers=[up, down], milestones=[warm])
        warm = sched.get("warmup_steps", 750)
        up = lr_scheduler.LinearLR(opt, start_factor=1e-6, end_factor=1.0, total_iters=warm)
        cos = lr_scheduler.CosineAnnealingLR(opt, T_max=sched.get("t_max", 20000), eta_min=lr * sched.get("eta_min_factor", 0.1))
        return lr_scheduler.SequentialLR(opt, schedulers=[up, cos], milestones=[warm])

    def should_skip_scheduler_step(self) -> bool:
        """True inside the LR flatten window (``flatten_start_step`` / ``flatten_duration`` are in outer steps)."""
        _, _, sched = _opt_cfg(self.hparams)
        start, dur = sched.get("flatten_start_step"), sched.get("flatten_duration", 0)
        if start is None or start <= 0 or dur <= 0:
            return False
        n = self.hparams.inner_steps
        return start * n <= self.inner_scheduler_step_count < (start + dur) * n

    # ------------------------------------------------------------------------------------ #
    # evaluation
    # ------------------------------------------------------------------------------------ #
    def _labels(self, input_ids: torch.Tensor) -> torch.Tensor:
        pad = self.tokenizer.pad_token_id
        labels = torch.empty_like(input_ids)
        labels[:, :-1] = input_ids[:, 1:]
        labels[:, -1] = pad
        return torch.where(labels == pad, torch.full_like(labels, -100), labels)

    async def evaluate_model(self, model, loader) -> tuple[float, int]:
        """Forward-only mean loss over ``loader``: returns (sum of batch losses, number of batches).
        Losses are accumulated on the device and read back once."""
        device = self.device
        losses = []
        model.eval()
        with torch.no_grad():
            for batch in loader:
                if getattr(self, "stop_event", None) is not None and self.stop_event.is_set():
                    break
                ids = (batch if isinstance(batch, torch.Tensor) else torch.tensor(batch)).to(device, dtype=torch.long,
                                                                                         non_blocking=True)
                labels = self._labels(ids)
                if hasattr(model, "loss"):
                    losses.append(model.loss(ids, labels).float())
                else:
                    with torch.autocast(device_type=device.type, dtype=getattr(self, "amp_dtype", torch.bfloat16)):
                        out = model(ids, labels)
                    losses.append(torch.nn.functional.cross_entropy(out.float().flatten(0, 1), labels.flatten(), ignore_index=-100))
                await asyncio.sleep(0)
        model.train()
        if not losses:
            return 0.0, 0
        stacked = torch.stack(losses)
        finite = torch.isfinite(stacked)
        total = float(torch.where(finite, stacked, torch.zeros_like(stacked)).sum().item())
        return total, int(finite.sum().item())

    # ------------------------------------------------------------------------------------ #
    # inner loop
    # ------------------------------------------------------------------------------------ #
    def _lr_now(self) -> float:
        return float(self.inner_optimizer.param_groups[0]["lr"])

    def _warmup_scale(self) -> float:
        anneal = (getattr(self.hparams, "anneal_mode", {}) or {}).get("enabled", False)
        if not anneal and self.warmup_steps_taken < self.warmup_inner_steps:
            return (self.warmup_steps_taken + 1) / self.warmup_inner_steps
        return 1.0

    async def inner_steps(self, loader, step_window: int, null_round: bool = False) -> dict:
        """One window of inner optimisation.  Returns ``total_loss`` (sum over ranks and batches),
        ``window_entry_loss``, ``batch_count``, ``batch_tokens``, norms and Adam metrics."""
        engine = getattr(self, "engine", None)
        hp, dev = self.hparams, self.device
        accum = max(self.sampler.grad_accum_steps, 1)
        self.prefetch_inner_optimizer_states()
        prof_cfg = getattr(self, "_prof_config", None)
        prof = None
        if prof_cfg is not None:
            import torch.profiler as tp

            prof = tp.profile(**prof_cfg)
            prof.__enter__()
        if engine is None:
            self.inner_optimizer.zero_grad(set_to_none=True)
        step_losses, all_losses = [], []
        batch_count = batch_tokens = inner_step_count = 0
        entry_loss = None
        try:
            for batch in labelled(loader, "Data Loading"):
                # A rank never leaves the loop on its own view of the world: the stop request and the window
                # clock are rank-local, and the optimizer step below contains collectives.  Both are agreed on
                # at accumulation boundaries, which every rank reaches at the same batch count.
                if self.stop_event.is_set() and not (self.world_size > 1 and dist_helper.is_distributed()):
                    break
                with phase("Prepare Inputs"):
                    ids = (batch if isinstance(batch, torch.Tensor) else torch.tensor(batch)).to(
                        dev, dtype=torch.long, non_blocking=True)
                    labels = self._labels(ids)
                batch_tokens += ids.numel()
                if engine is not None:
                    with phase("Forward + Backward Pass"):
                        loss = engine.micro_step(ids, labels, 1.0 / accum)
                else:
                    ctx = (torch.autocast(device_type=dev.type, dtype=getattr(self, "amp_dtype", torch.bfloat16))
                           if dev.type == "cuda" else nullcontext())
                    with ctx:
                        if hasattr(self.model, "loss"):
                            loss_t = self.model.loss(ids, labels, 1.0 / accum)
                        else:
                            out = self.model(ids, labels)
                            loss_t = torch.nn.functional.cross_entropy(out.float().flatten(0, 1), labels.flatten(),
                                                                       ignore_index=-100) / accum
                    loss_t.backward()
                    loss = loss_t.detach() * (accum if not hasattr(self.model, "loss") else 1.0)
                step_losses.append(loss.float())
                batch_count += 1
                # The step boundary is a function of the batch count alone (the same on every rank).  The reference
                # instead agrees on `step_now` with a MAX all-reduce after every micro-batch
                # (neurons/trainer.py:903-918); here the window change and the stop request wait for the boundary
                # and are agreed on there with ONE reduce per inner step.
                step_now = batch_count % accum == 0
                if step_now:
                    leave = self.current_window != step_window or self.stop_event.is_set()
                    if self.world_size > 1 and dist_helper.is_distributed():
                        leave = bool(dist_helper.ddp_reduce(int(leave), op=dist.ReduceOp.MAX, device=dev))
                    window_changed = leave
                    if not null_round:
                        scale = self._warmup_scale()
                        if engine is not None:
                            with phase("Optimizer Step"):
                                engine.optimizer_step(lr=self._lr_now() * scale)
                        else:
                            torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
                            saved = [g["lr"] for g in self.inner_optimizer.param_groups]
                            for g in self.inner_optimizer.param_groups:
                                g["lr"] = g["lr"] * scale
                            self.inner_optimizer.step()
                            for g, v in zip(self.inner_optimizer.param_groups, saved):
                                g["lr"] = v
                        if scale < 1.0 or self.warmup_steps_taken < self.warmup_inner_steps:
                            self.warmup_steps_taken += 1
                        if not self.should_skip_scheduler_step():
                            self.inner_scheduler.step()
                        self.inner_scheduler_step_count += 1
                    if engine is not None:
                        if null_round:
                            engine.zero_grad()
                    else:
                        self.inner_optimizer.zero_grad(set_to_none=True)
                    inner_step_count += 1
                    stacked = torch.stack(step_losses)
                    all_losses.append(stacked)
                    if entry_loss is None:
                        entry_loss = stacked.mean()
                    step_losses = []
                    if prof is not None:
                        prof.step()
                    if self.is_master:
                        tplr.logger.info(f"Inner Step {inner_step_count}, Batch {batch_count}")
                    if window_changed or inner_step_count == hp.inner_steps:
                        if not null_round:
                            for _ in range(inner_step_count, hp.inner_steps):
                                if not self.should_skip_scheduler_step():
                                    self.inner_scheduler.step()
                                self.inner_scheduler_step_count += 1
                        break
                await asyncio.sleep(0)
        finally:
            if prof is not None:
                prof.__exit__(None, None, None)
        if step_losses:
            all_losses.append(torch.stack(step_losses))
        # single read-back for the whole window
        if all_losses:
            flat = torch.cat(all_losses)
            stats = torch.stack((flat.sum(), entry_loss if entry_loss is not None else flat.mean()))
        else:
            stats = torch.zeros(2, device=dev)
        counts = torch.tensor([batch_count, batch_tokens], device=dev, dtype=torch.float64)
        if self.world_size > 1 and dist_helper.is_distributed():
            pack = torch.cat((stats.double(), counts))
            dist.all_reduce(pack)
            pack[1] /= self.world_size
            stats, counts = pack[:2], pack[2:]
        total_loss, window_entry_loss = (float(x) for x in stats.tolist())
        g_batches, g_tokens = (int(x) for x in counts.tolist())
        return {"total_loss": total_loss, "window_entry_loss": window_entry_loss, "batch_count": g_batches,
                "batch_tokens": g_tokens, "inner_steps": inner_step_count, **self._norm_metrics(),
                "adam_metrics": self.compute_adam_metrics()}

    def _norm_metrics(self) -> dict:
        engine = getattr(self, "engine", None)
        dev = self.device
        if engine is not None:
            sq = torch.stack(((engine.store.master_shard.double() ** 2).sum(), engine.gnorm_sq.double().sum()))
        else:
            w = sum(((p.detach().double() ** 2).sum() for p in self.model.parameters() if p.requires_grad),
                    torch.zeros((), dtype=torch.float64, device=dev))
            g = sum(((p.grad.detach().double() ** 2).sum() for p in self.model.parameters() if p.grad is not None),
                    torch.zeros((), dtype=torch.float64, device=dev))
            sq = torch.stack((w, g))
        if self.world_size > 1 and dist_helper.is_distributed() and engine is not None:
            t = sq.float() if dev.type == "cuda" else sq
            dist.all_reduce(t[:1])
            sq = t.double()
        w, g = (float(x) for x in sq.tolist())
        return {"global_weight_norm": math.sqrt(max(w, 0.0)), "global_grad_norm": math.sqrt(max(g, 0.0))}

    def compute_adam_metrics(self) -> dict:
        """Mean |m|, mean v and the update-to-weight ratio of the Adam state (empty for other optimizers)."""
        engine = getattr(self, "engine", None)
        if engine is not None:
            if engine.adam_step == 0 or engine.cfg.inner_optimizer != "adamw":
                return {}                      # with Muon the first-moment buffer is its momentum and v is unused
            m, v, p = engine.exp_avg, engine.exp_avg_sq, engine.store.master_shard
            upd = m / (v.sqrt() + engine.cfg.eps)
            vals = torch.stack((m.abs().mean(), v.mean(), upd.norm() / (p.norm() + 1e-12))).tolist()
            return {"adam/exp_avg_abs_mean": vals[0], "adam/exp_avg_sq_mean": vals[1], "adam/update_to_weight": vals[2]}
        opt = getattr(self, "inner_optimizer", None)
        if not isinstance(opt, torch.optim.AdamW):
            return {}
        ms, vs = [], []
        for st in opt.state.values():
            if "exp_avg" in st:
                ms.append(st["exp_avg"].abs().mean())
                vs.append(st["exp_avg_sq"].mean())
        if not ms:
            return {}
        return {"adam/exp_avg_abs_mean": float(torch.stack(ms).mean()), "adam/exp_avg_sq_mean": float(torch.stack(vs).mean())}

    # ------------------------------------------------------------------------------------ #
    # outer step and optimizer-state offload
    # ------------------------------------------------------------------------------------ #
    def outer_step(self, gather_result, log_wandb: bool = False):
        return tplr.neurons.outer_step(
            self.model, self.outer_optimizer, gather_result=gather_result, transformer=self.transformer,
            compressor=self.compressor, xshapes=self.xshapes, totalks=self.totalks, device=str(self.device),
            is_master=self.is_master, world_size=self.world_size, use_dct=self.hparams.use_dct,
            wandb_run=self.wandb if self.is_master and log_wandb else None, global_step=self.global_step)

    def _optimizer_state_tensors(self):
        engine = getattr(self, "engine", None)
        if engine is not None:
            return [("exp_avg", engine, "exp_avg"), ("exp_avg_sq", engine, "exp_avg_sq")]
        out = []
        opt = getattr(self, "inner_optimizer", None)
        for st in (opt.state.values() if opt is not None else []):
            for k, v in st.items():
                if torch.is_tensor(v) and v.numel() > 1:
                    out.append((k, st, k))
        return out

    def offload_inner_optimizer_states(self) -> None:
        """Move the inner optimizer's moments to pinned host memory (frees HBM for the gather phase)."""
        if not getattr(self.hparams, "offload_optimizer_states", False):
            return
        for _, holder, key in self._optimizer_state_tensors():
            t = holder[key] if isinstance(holder, dict) else getattr(holder, key)
            if t.is_cuda:
                host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
                host.copy_(t, non_blocking=True)
                if isinstance(holder, dict):
                    holder[key] = host
                else:
                    setattr(holder, key, host)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    def prefetch_inner_optimizer_states(self) -> None:
        dev = getattr(self, "device", None)
        if dev is None or torch.device(dev).type != "cuda":
            return
        for _, holder, key in self._optimizer_state_tensors():
            t = holder[key] if isinstance(holder, dict) else getattr(holder, key)
            if not t.is_cuda:
                moved = t.to(dev, non_blocking=True)
                if isinstance(holder, dict):
                    holder[key] = moved
                else:
                    setattr(holder, key, moved)
