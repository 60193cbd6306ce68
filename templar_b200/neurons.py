"""Protocol logic shared by miners and validators: building the compressed pseudo-gradient,
applying gathered gradients, peer-list rotation, checkpoint fallback and catch-up, sync
metrics and the index-overlap (copy detection) check.

Function-level parity with the reference's src/tplr/neurons.py:47-1479.  Two execution paths:

* **engine path** — when the model is attached to a
  :class:`~templar_b200.parallel.window_engine.WindowEngine` (``model._window_engine``), the
  per-window work is a handful of fused sm_100a kernel launches over the flat parameter
  buffers (each rank handles its own chunk-aligned shard);
* **generic path** — tensor-by-tensor PyTorch with exactly the reference's semantics (DTensor
  aware, owner-rank compression, rank-0 decompression + scatter/broadcast).  It is what runs on
  CPU, with foreign models, and in the unit tests that drive these functions with dummy objects.
"""

from __future__ import annotations

import asyncio
import gc
import math
import typing
from collections import defaultdict
from datetime import datetime, timedelta, timezone
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.nn as nn

from .compress import unpack_12bit_indices
from .distributed import dist_helper
from .logging import P, T, logger
from .utils.ranges import phase

__all__ = ["prepare_gradient_dict", "outer_step", "update_peers", "load_checkpoint_with_fallback",
           "handle_checkpoint_catchup", "catchup_with_aggregation_server", "compare_model_with_debug_dict",
           "check_uid_index_overlap", "determine_slash_egregiousness", "instantiate_slashing_multiplier", "NeuronT"]

NeuronT = typing.TypeVar("NeuronT")            # a miner or a validator: what these functions take as ``instance``


def _engine_of(model):
    """The window engine attached to ``model`` (``model._window_engine``), or None.  Looked up in the instance
    dictionary: an object that answers every attribute (a mock standing in for a model) has no engine."""
    return getattr(model, "__dict__", {}).get("_window_engine")


try:
    from torch.distributed.tensor import DTensor as _DTensor
except Exception:  # noqa: BLE001  (a torch build without the distributed tensor package)
    _DTensor = None


def _is_dtensor(x) -> bool:
    return _DTensor is not None and isinstance(x, _DTensor)


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def _mesh_group(x):
    mesh = getattr(x, "device_mesh", None)
    if mesh is not None:
        try:
            return mesh.get_group()
        except Exception:  # noqa: BLE001
            pass
    return dist.group.WORLD if _dist_on() else None


def _named_parameters(model):
    inner = model.module if isinstance(model, torch.nn.parallel.DistributedDataParallel) else model
    return inner.named_parameters()


def _to_host_async(t):
    if not isinstance(t, torch.Tensor):
        return t
    if t.is_cuda:
        out = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        out.copy_(t, non_blocking=True)
        return out
    return t.cpu()


# --------------------------------------------------------------------------------------- #
# miner side
# --------------------------------------------------------------------------------------- #
def prepare_gradient_dict(miner, step_window: int, null_round: bool = False):
    """Returns ``(gradient, xshapes, totalks)``; ``gradient`` maps ``<name>idxs`` / ``<name>vals`` /
    ``<name>quant_params`` plus ``"metadata": {"window": step_window}``.

    Error feedback: ``e <- momentum_decay * e + grad`` (``e <- 0`` on a null round), the payload is
    ``compress(encode(e))`` and ``e <- e - decode(decompress(payload))``.
    """
    engine = _engine_of(miner.model)
    if engine is not None and getattr(miner, "use_engine", True):
        return _prepare_gradient_dict_engine(miner, engine, step_window, null_round)

    gradient, xshapes, totalks = {}, {}, {}
    use_dct = getattr(miner.hparams, "use_dct", False)
    topk = getattr(miner.hparams, "topk_compression", 32)
    params = dict(miner.model.named_parameters())
    for n in miner.owned_params:
        ef = miner.error_feedback.get(n)
        if ef is not None and not ef.is_cuda and n in params and params[n].is_cuda:
            miner.error_feedback[n] = ef.to(params[n].device, non_blocking=True)

    for n, p in _named_parameters(miner.model):
        g = getattr(p, "grad", None)
        if _is_dtensor(g):
            grp = _mesh_group(g)
            if _dist_on() and grp is not None:
                dist.barrier(group=grp)
            grad_full = g.full_tensor().to(p.device)
            if _dist_on() and grp is not None:
                dist.barrier(group=grp)
        else:
            if g is None and not _is_dtensor(p):
                continue
            assert g is not None, f"p.grad is None for {n}"
            grad_full = g.to(p.device)
        if n not in miner.owned_params:
            p.grad = None
            continue
        ef = miner.error_feedback[n]
        if ef is None:
            ef = torch.zeros_like(grad_full, device=p.device)
        elif ef.device != p.device:
            ef = ef.to(p.device)
        if null_round:
            ef.zero_()
        else:
            ef.mul_(miner.hparams.momentum_decay).add_(grad_full)
        encoded = miner.transformer.encode(ef, use_dct=use_dct)
        idxs, vals, xshape, totalk, quant_params = _compress5(miner.compressor, encoded, topk)
        del encoded
        dense = miner.compressor.decompress(p, idxs, vals, xshape, totalk, quant_params)
        ef.sub_(miner.transformer.decode(dense, use_dct=use_dct))
        del dense
        miner.error_feedback[n] = ef
        gradient[n + "idxs"] = _to_host_async(idxs)
        gradient[n + "vals"] = _to_host_async(vals)
        gradient[n + "quant_params"] = quant_params
        xshapes[n], totalks[n] = xshape, totalk
        p.grad = None

    bufs = getattr(miner, "error_feedback_cpu_buffers", None)
    if bufs is not None:
        for name, ef in miner.error_feedback.items():
            if ef is not None and ef.is_cuda and name in bufs:
                bufs[name].copy_(ef, non_blocking=True)
                miner.error_feedback[name] = bufs[name]
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    gradient["metadata"] = {"window": step_window}
    return gradient, xshapes, totalks


def _compress5(compressor, encoded, topk):
    out = compressor.compress(encoded, topk)
    return out if len(out) == 5 else (*out, None)


def _prepare_gradient_dict_engine(miner, engine, step_window: int, null_round: bool):
    """Fused path: one compress launch per basis group over the rank's shard; the payload stays in
    the engine's flat buffers and the returned dict holds pinned host copies of its tensors."""
    heap = engine.heap
    own = None
    if heap is not None and engine.world_size > 1:
        own = (heap.peer_ptr(engine.own_idx, 0), heap.peer_ptr(engine.own_val, 0))
    with phase("Compress"):
        engine.compress(null_round=null_round, own_slot_ptrs=own)
        if engine.world_size > 1:
            engine.merge_own_payload()              # no-op with a heap: the ranks wrote into rank 0's buffers
            engine._barrier()
    gradient, xshapes, totalks = {}, {}, {}
    L = engine.layout
    want_payload = engine.rank == 0 and engine.replica == 0        # the replicas hold the same payload
    quant = None
    if want_payload:
        idx_host = _to_host_async(engine.own_idx)
        if engine.cfg.quantize:                  # codes and tables were computed by engine.compress()
            quant = engine.own_payload()
            val_host = _to_host_async(engine._q_codes)
        else:
            val_host = _to_host_async(engine.own_val)
    for s in sorted(L.specs, key=lambda s: s.index):
        xshapes[s.name], totalks[s.name] = L.xshape(s.name), s.totalk
        if want_payload:
            idx, val = L.payload_views(idx_host, val_host, s.name)
            gradient[s.name + "idxs"], gradient[s.name + "vals"] = idx, val
            gradient[s.name + "quant_params"] = quant[s.name + "quant_params"] if quant is not None else None
    if engine.cuda:
        torch.cuda.current_stream().synchronize()
    gradient["metadata"] = {"window": step_window}
    return gradient, xshapes, totalks


# --------------------------------------------------------------------------------------- #
# outer step
# --------------------------------------------------------------------------------------- #
@torch.no_grad()
def outer_step(model: nn.Module, optimizer, *, gather_result, transformer, compressor, xshapes: dict, totalks: dict,
               device, is_master: bool, world_size: int, use_dct: bool = False, wandb_run=None,
               global_step: int | None = None) -> dict | None:
    """Aggregate the gathered payloads (median-norm clip, mean over contributors, inverse
    transform) and apply them parameter by parameter with ``optimizer`` (plain SGD in the
    reference).  Returns the gradient fingerprint on the source rank."""
    engine = _engine_of(model)
    if engine is not None and getattr(model, "_use_engine_outer_step", True):
        return _outer_step_engine(model, engine, optimizer, gather_result, is_master)

    model.train()
    optimizer.zero_grad(set_to_none=True)
    ddp = world_size > 1 and _dist_on()
    on_src = is_master or not ddp
    src_sd = None
    if on_src and gather_result is not None and getattr(gather_result, "state_dict", None) is not None:
        sd = gather_result.state_dict
        src_sd = vars(sd).copy() if isinstance(sd, SimpleNamespace) else dict(sd)
    fingerprint = {"param_norms": {}, "param_means": {}, "total_norm_sq": 0.0, "total_elements": 0} if on_src else None
    med_lo, med_hi = float("inf"), float("-inf")

    def bcast_flag(v: int) -> int:
        t = torch.tensor([v], device=device, dtype=torch.int32)
        if ddp:
            dist.broadcast(t, 0)
        return int(t.item())

    def to_dev(obj):
        if torch.is_tensor(obj):
            return obj.to(device=device, non_blocking=True)
        if isinstance(obj, (list, tuple)):
            return type(obj)(to_dev(x) for x in obj)
        return obj

    for name, p in model.named_parameters():
        payload = None
        if on_src and src_sd is not None:
            idxs, vals, qps = src_sd.get(name + "idxs"), src_sd.get(name + "vals"), src_sd.get(name + "quant_params")
            if idxs is not None and vals is not None:
                idxs = list(idxs) if isinstance(idxs, (list, tuple)) else [idxs]
                vals = list(vals) if isinstance(vals, (list, tuple)) else [vals]
                vals_f = compressor.maybe_dequantize_values(vals, qps, device)
                if vals_f:
                    payload = (to_dev(idxs), vals_f)
        if bcast_flag(1 if payload is not None else 0) == 0:
            continue
        grad_src = None
        if on_src:
            idxs_dev, vals_f = payload
            norms = torch.stack([torch.linalg.vector_norm(v.float()) for v in vals_f])
            med = float(torch.median(norms).item())
            med_lo, med_hi = min(med_lo, med), max(med_hi, med)
            ref = torch.empty_like(p, device=device, dtype=p.dtype) if not _is_dtensor(p) else \
                torch.empty(p.shape, device=device, dtype=p.dtype)
            dense = compressor.batch_decompress(ref, idxs_dev, vals_f, xshapes[name], totalks[name],
                                                quantize_params=None, block_norms=norms, normalise=False, clip_norm=True)
            grad_src = transformer.decode(dense, use_dct=use_dct).to(dtype=p.dtype, device=p.device)
            del dense, ref
            if fingerprint is not None:
                pn = float(torch.linalg.vector_norm(grad_src.float()).item())
                fingerprint["param_norms"][name] = pn
                fingerprint["total_norm_sq"] += pn * pn
                fingerprint["total_elements"] += grad_src.numel()
                fingerprint["param_means"][name] = float(grad_src.float().mean().item())
        if _is_dtensor(p):
            from torch.distributed.tensor import distribute_tensor

            src = grad_src if on_src else torch.empty(p.shape, device=p.device, dtype=p.dtype)
            new_grad = distribute_tensor(src, device_mesh=p.device_mesh, placements=p.placements, src_data_rank=0)
            if not torch.isfinite(new_grad.to_local()).all():
                continue
            p.grad = new_grad
        else:
            if ddp:
                if on_src:
                    dist.broadcast(grad_src, 0)
                    p.grad = grad_src
                else:
                    p.grad = torch.empty_like(p)
                    dist.broadcast(p.grad, 0)
            else:
                p.grad = grad_src
            if p.grad is not None and not torch.isfinite(p.grad).all():
                p.grad = None
                continue
        optimizer.step()
        p.grad = None

    if on_src and wandb_run is not None and global_step is not None and med_hi > float("-inf"):
        wandb_run.log({"compress/min_median_block_norm": med_lo, "compress/max_median_block_norm": med_hi},
                      step=global_step)
    optimizer.zero_grad(set_to_none=True)
    if on_src and fingerprint is not None:
        fingerprint["global_l2_norm"] = math.sqrt(fingerprint["total_norm_sq"])
        return fingerprint
    return None


def _outer_step_engine(model, engine, optimizer, gather_result, is_master: bool) -> dict | None:
    """Fused path.  The gathered payloads (host tensors on the master rank) are placed in the
    engine's device slots, spread round-robin over the ranks, and one aggregate launch per basis
    group applies the update to every rank's shard."""
    lr = float(optimizer.param_groups[0]["lr"]) if optimizer is not None else engine.cfg.outer_lr
    sd = None
    if gather_result is not None and getattr(gather_result, "state_dict", None) is not None:
        s = gather_result.state_dict
        sd = vars(s) if isinstance(s, SimpleNamespace) else dict(s)
    n_peers = 0
    if sd:
        first = next((v for k, v in sd.items() if k.endswith("vals")), None)
        n_peers = len(first) if isinstance(first, (list, tuple)) else (1 if first is not None else 0)
    n_peers = min(n_peers, engine.cfg.max_peers)
    # co-located peers (gather_result.local_ranks): read from the owners' GPU memory, nothing to stage
    local = sorted((getattr(gather_result, "local_ranks", None) or {}).values()) if gather_result is not None else []
    if engine.dp_size > 1:
        t = torch.tensor([n_peers], device=engine.device, dtype=torch.int32)
        dist.broadcast(t, 0)
        n_peers = int(t.item())
    if n_peers == 0 and not local:
        return None
    leader = engine.rank == 0                        # the rank of a copy of the state that stages the payloads
    if engine.replicate_size > 1 and leader:
        # the gathered payloads are on the master rank: hand them to the leader of every other copy
        box = [sd if engine.replica == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(engine.replicate_group, 0), group=engine.replicate_group)
        sd = box[0]
    if engine.world_size == 1:
        for j in range(n_peers):
            from .parallel.window_engine import peer_slice
            engine.load_peer_payload(j, peer_slice(sd, j))
    else:
        engine.distribute_peer_payloads(sd if leader else None, n_peers)
    if not engine.window_open:
        engine.snapshot()           # catch-up / validator flow: apply to the current weights
    with phase("Outer Step"):
        if local:
            engine.outer_step(peers=list(range(n_peers)) + [("rank", r) for r in local], lr=lr, include_own=False,
                              base="theta0")
        else:
            engine.outer_step(n_peers, lr=lr, include_own=False, base="theta0")
    engine.window_open = False
    # fingerprint: the applied update is (theta0 - theta) / lr on every shard
    d = engine.theta0 - engine.store.master_shard
    sq = (d.double() ** 2).sum().reshape(1)
    sm = d.double().sum().reshape(1)
    if engine.world_size > 1:
        t = torch.cat((sq, sm)).to(torch.float32 if engine.cuda else torch.float64)
        dist.all_reduce(t, group=engine.group)
        sq, sm = t[0:1].double(), t[1:2].double()
    if not is_master:
        return None
    lr_safe = lr if lr != 0 else 1.0
    n_el = engine.layout.total
    return {"param_norms": {}, "param_means": {}, "total_norm_sq": float(sq) / lr_safe ** 2, "total_elements": n_el,
            "global_l2_norm": math.sqrt(float(sq)) / abs(lr_safe), "global_mean": float(sm) / lr_safe / max(n_el, 1)}


# --------------------------------------------------------------------------------------- #
# peers
# --------------------------------------------------------------------------------------- #
async def update_peers(instance, window: int, peer_start: float) -> None:
    comms, hp = instance.comms, instance.hparams
    # on a network the list always appears (the validators publish it) and the node waits for it; an offline run may
    # have no validator at all and must not wait for ever
    kw = {"retries": 2, "retry_delay": 0.5} if getattr(getattr(instance, "config", None), "local", False) is True else {}
    if len(comms.peers) == 0:
        prev = await comms.get_peer_list(fetch_previous=True, **kw)
        if prev is not None:
            comms.peers, comms.reserve_peers = prev[0], prev[1]
            logger.info(f"Got previous peer list with {len(prev[0])} peers and update window {prev[2]}")
        else:
            logger.warning("Failed to fetch previous peer list, continuing with empty peers")
    due = (instance.next_peers is None and
           instance.peers_update_window + hp.peer_replacement_frequency - window <= hp.peer_list_window_margin)
    if due:
        res = await comms.get_peer_list(**kw)
        if res is None:
            logger.info("Unable to get peer list from bucket")
        else:
            nxt, reserve, upd = res
            if instance.peers_update_window is None or upd > instance.peers_update_window:
                instance.next_peers, instance.next_reserve_peers, instance.peers_update_window = nxt, reserve, upd
                logger.info(f"Got new peer list {nxt} effective at window {upd}")
    if instance.next_peers is not None and window >= instance.peers_update_window:
        comms.peers = instance.next_peers
        comms.reserve_peers = instance.next_reserve_peers if instance.next_reserve_peers is not None else []
        late = window - instance.peers_update_window
        logger.info(f"{P(window, T() - peer_start)} Updated peers {'on time' if late <= 0 else f'{late} windows late'} "
                    f"- gather:{len(comms.peers)}, reserve:{len(comms.reserve_peers)}")
        instance.next_peers = None
    else:
        logger.info("Not time to replace peers: " + ("next peers are not defined yet" if instance.next_peers is None
                    else f"sync window is {window} and peers update window is {instance.peers_update_window}"))


# --------------------------------------------------------------------------------------- #
# checkpoints and catch-up
# --------------------------------------------------------------------------------------- #
async def load_checkpoint_with_fallback(instance) -> tuple[bool, int, int, bool]:
    """Try the current version's newest checkpoint, then the configured bootstrap version.
    Returns ``(ok, sync_window, global_step, from_bootstrap)``."""
    from .dcp_checkpoint import DCPCheckpointer

    ok, win, step, boot = False, 0, 0, False
    latest = await instance.ckpt._discover_latest(prefer_highest_staked=True)
    if latest is not None:
        res = await instance.ckpt.download_and_load(model=instance.model, window=latest, shared_fs=True,
                                                    process_group=None, prefer_highest_staked=True)
        if res is not None:
            ok, (win, step) = True, res
            instance.model_initialized = True
            logger.info(f"Loaded current version checkpoint (window={win}, global_step={step})")
    if not ok and getattr(instance, "bootstrap_version", None):
        bwin = getattr(instance.hparams, "checkpoint_init_window", None)
        bck = DCPCheckpointer(instance.comms, uid=instance.uid, version=instance.bootstrap_version, repo_root=".")
        if bwin is None:
            bwin = await bck._discover_latest(prefer_highest_staked=True)
        if bwin is not None:
            res = await bck.download_and_load(model=instance.model, window=bwin, shared_fs=True, process_group=None,
                                              prefer_highest_staked=True)
            if res is not None:
                ok, boot, (win, step) = True, True, res
                instance.model_initialized = True
                logger.info(f"Loaded bootstrap checkpoint (version={instance.bootstrap_version}, window={win})")
    if ok and step == -1:
        if boot:
            bstart = await instance.comms.get_start_window(version=instance.bootstrap_version)
            step = win - bstart if bstart is not None else 0
        else:
            step = win - instance.start_window
    if ok:
        instance.global_step = step
    return ok, win, step, boot


def _scheduler_cfg(hparams) -> dict:
    opt = getattr(hparams, "optimizer", {}) or {}
    kind = opt.get("type", "adamw").lower()
    return (opt.get(kind, {}) or {}).get("scheduler", {}) or {}


async def handle_checkpoint_catchup(instance, ckpt_ok: bool, ckpt_sync_win: int, ckpt_global_step: int,
                                    from_bootstrap: bool, aggregator_device: str | None = None) -> None:
    """Decide where to replay from, run the replay, and fast-forward the inner LR scheduler."""
    hp = instance.hparams
    anneal = getattr(hp, "anneal_mode", {}) or {}

    async def replay_from_decision(allow_bootstrap_rule: bool):
        if not ckpt_ok:
            logger.info("No checkpoint found, will catch up from start_window")
            await catchup_with_aggregation_server(instance, instance.start_window, aggregator_device=aggregator_device)
        elif allow_bootstrap_rule and from_bootstrap:
            await catchup_with_aggregation_server(instance, instance.start_window, aggregator_device=aggregator_device)
        elif ckpt_sync_win < instance.current_window:
            await catchup_with_aggregation_server(instance, max(ckpt_sync_win, instance.start_window),
                                                  aggregator_device=aggregator_device)
        else:
            logger.info(f"Checkpoint at window {ckpt_sync_win} is up to date with current window {instance.current_window}")

    if anneal.get("enabled", False):
        warm = anneal.get("warmup_inner_steps", 100)
        n = max(0, ckpt_global_step - anneal.get("start_global_step", 0)) * hp.inner_steps
        instance.warmup_inner_steps = warm
        instance.warmup_steps_taken = min(n, warm)
        instance.inner_scheduler_step_count = 0
        sched = getattr(instance, "inner_scheduler", None)
        if n > 0 and sched is not None:
            for _ in range(n):
                sched.step()
                instance.inner_scheduler_step_count += 1
        await replay_from_decision(allow_bootstrap_rule=False)
        return

    sc = _scheduler_cfg(hp)
    default_warm = sc.get("warmup_inner_steps", getattr(instance, "warmup_inner_steps", 0))
    startup_warm = sc.get("initial_warmup_inner_steps", default_warm)
    if ckpt_global_step != 0:
        instance.warmup_inner_steps = startup_warm if from_bootstrap else default_warm
        instance.warmup_steps_taken = 0
    await replay_from_decision(allow_bootstrap_rule=True)
    total = ckpt_global_step * hp.inner_steps
    rewind = sc.get("replay_rewind_inner_steps", 0)
    if rewind > 0:
        total = max(total - rewind, 0)
    sched = getattr(instance, "inner_scheduler", None)
    if total > 0 and sched is not None:
        for _ in range(total):
            if not instance.should_skip_scheduler_step():
                sched.step()
            instance.inner_scheduler_step_count += 1
        logger.info(f"Replayed {total} scheduler steps")


async def catchup_with_aggregation_server(instance, checkpoint_current_window: int,
                                          aggregator_device: str | None = None) -> None:
    """Replay the lead validator's aggregated gradients window by window (live gather as the
    fallback for the last window only) until the model has caught up with the chain head."""
    assert instance.start_window is not None
    device = aggregator_device if aggregator_device is not None else instance.config.device
    leader = int(instance.comms.metagraph.S.argmax().item())
    start_w, target_w = checkpoint_current_window + 1, instance.current_window
    logger.info(f"Replaying windows {start_w} ... {target_w - 1}")

    if checkpoint_current_window > 0 and instance.is_master:
        dbg = await instance.comms.get(uid=str(leader), window=checkpoint_current_window, key="debug", local=False,
                                       stale_retention=10)
        if dbg.success and isinstance(dbg.data, dict):
            cmp = await compare_model_with_debug_dict(instance.model, dbg.data, param_avg_change={},
                                                      learning_rate=getattr(instance.hparams, "learning_rate", 1e-3))
            if cmp["success"] and cmp["l2_norm"] > 0.1:
                logger.warning(f"Large L2 difference to the leader at the checkpoint window: {cmp['l2_norm']:.4f}")

    prev_state: dict[str, torch.Tensor] = {}
    avg_change: dict[str, torch.Tensor] = {}
    alpha = 0.20
    while start_w < target_w:
        logger.info(f"  • window {start_w}")
        gather_ns = None
        if instance.is_master:
            fetch = await instance.comms.get(uid=str(leader), window=start_w, key="aggregator", timeout=60, local=False,
                                             stale_retention=10, map_location=device)
            if fetch.success and fetch.data is not None and "state_dict" in fetch.data:
                pl = fetch.data
                gather_ns = SimpleNamespace(state_dict=SimpleNamespace(**pl["state_dict"]), uids=pl.get("uids", []),
                                            skipped_uids=pl.get("skipped_uids", []), success_rate=pl.get("success_rate", 0.0))
            elif start_w == target_w - 1:
                sync_block = (start_w + 1) * instance.hparams.blocks_per_window
                ts = await asyncio.get_running_loop().run_in_executor(None, instance.query_block_timestamp, sync_block)
                tmin = tmax = None
                if ts is not None:
                    tmin = datetime.fromtimestamp(ts, tz=timezone.utc)
                    tmax = tmin + timedelta(seconds=instance.hparams.time_window_delta_seconds)
                gather_ns = await instance.comms.gather(my_uid=instance.uid, uids=instance.comms.peers, window=start_w,
                                                        key="gradient", timeout=45, device=str(device), local=False,
                                                        stale_retention=10, totalks=instance.totalks,
                                                        compressor=instance.compressor, time_min=tmin, time_max=tmax)
                logger.info("    ↳ gather-fallback " + ("succeeded – applying" if gather_ns is not None else "failed – skipping"))
            else:
                logger.warning("    ↳ aggregated gradients not available – skipping")
        skip = torch.tensor([1 if (instance.is_master and gather_ns is None) else 0], dtype=torch.int32,
                            device=instance.config.device)
        dist_helper.broadcast(skip, src=0)
        if bool(skip.item()):
            start_w += 1
            continue
        dist_helper.safe_barrier("catchup_pre_outer_step", getattr(instance, "local_rank", 0))
        outer_step(instance.model, instance.outer_optimizer, gather_result=gather_ns, transformer=instance.transformer,
                   compressor=instance.compressor, xshapes=instance.xshapes, totalks=instance.totalks,
                   device=instance.config.device, is_master=instance.is_master, world_size=instance.world_size,
                   use_dct=instance.hparams.use_dct, wandb_run=None, global_step=instance.global_step)
        sched = getattr(instance, "inner_scheduler", None)
        if sched is not None:
            for _ in range(instance.hparams.inner_steps):
                if not instance.should_skip_scheduler_step():
                    sched.step()
                instance.inner_scheduler_step_count += 1
        gather_ns = None
        gc.collect()
        try:
            if instance.is_master:
                dbg = await instance.comms.get(uid=str(leader), window=start_w, key="debug", local=False, stale_retention=10)
                if dbg.success and isinstance(dbg.data, dict):
                    for name, cur in param_samples(instance.model, 0, 2).items():
                        cur = cur.detach().cpu()
                        if name in prev_state:
                            delta = (cur - prev_state[name]).abs()
                            if name not in avg_change:
                                avg_change[name] = delta.clone()
                            else:
                                avg_change[name].mul_(1 - alpha).add_(delta * alpha)
                        prev_state[name] = cur.clone()
                    cmp = await compare_model_with_debug_dict(model=instance.model, debug_dict=dbg.data,
                                                              learning_rate=instance.outer_optimizer.param_groups[0]["lr"],
                                                              index_range=(0, 2), param_avg_change=avg_change)
                    if cmp["success"]:
                        logger.info(f"[catch-up] window {start_w} avg_steps_behind={cmp['avg_steps_behind']:.3f}, "
                                    f"l2_norm={cmp['l2_norm']:.4f}")
                else:
                    logger.warning(f"[catch-up] no debug-dict found for window {start_w}")
        except Exception as exc:  # noqa: BLE001
            logger.warning(f"[catch-up] debug-dict processing error: {exc}")
        instance.global_step += 1
        start_w += 1
        dist_helper.safe_barrier("catchup_post_window", getattr(instance, "local_rank", 0))
        if instance.current_window > target_w:
            target_w = instance.current_window
    logger.info("Catch-up finished – model now in sync.")


def param_samples(model: nn.Module, lo: int, hi: int) -> dict[str, torch.Tensor]:
    """``{name: flatten()[lo:hi]}`` of every parameter with at least ``hi`` elements: the slices that nodes publish
    as debug information and compare for the sync score.  Read from the module tree, or, when the engine holds the
    parameters as shards only, from the elements the ranks collected at the last window boundary."""
    engine = _engine_of(model)
    if engine is not None and getattr(engine, "fsdp", False):
        return engine.param_samples(lo, hi)
    out = {}
    for name, p in _named_parameters(model):
        flat = (p.to_local() if _is_dtensor(p) else p).detach().flatten()
        if flat.numel() >= hi:
            out[name] = flat[lo:hi]
    return out


# --------------------------------------------------------------------------------------- #
# sync metric
# --------------------------------------------------------------------------------------- #
async def compare_model_with_debug_dict(model: nn.Module, debug_dict: dict, learning_rate: float,
                                        param_avg_change: dict | None = None, *, min_step_size: float = 1e-9,
                                        index_range: tuple[int, int] = (0, 2)) -> dict:
    """Distance between local weights and a peer's published ``<name>_debug`` slices, also expressed
    in "outer steps behind" (|diff| / typical per-step change; interquartile mean over elements)."""
    sq = ab = 0.0
    count = tensors = 0
    max_diff = max_steps = 0.0
    ratios = []
    lo, hi = index_range
    engine = _engine_of(model)
    sharded = param_samples(model, lo, hi) if engine is not None and getattr(engine, "fsdp", False) else None
    for name, p in _named_parameters(model):
        ref = debug_dict.get(name + "_debug")
        if not isinstance(ref, list):
            continue
        if sharded is not None:
            if name not in sharded:
                continue
            cur = sharded[name]
        else:
            cur = (p.to_local() if _is_dtensor(p) else p).data.flatten()[lo:hi]
        diff = cur - torch.tensor(ref, dtype=cur.dtype, device=cur.device)
        a = diff.abs()
        sq += float((diff.float() ** 2).sum())
        ab += float(a.sum())
        max_diff = max(max_diff, float(a.max()))
        count += a.numel()
        step = None
        if param_avg_change and name in param_avg_change:
            step = torch.clamp(param_avg_change[name].to(cur.device), min=min_step_size)
            if step.numel() != a.numel():
                step = None
        if step is None:
            step = a.new_full(a.size(), learning_rate)
        r = a / step
        ratios.append(r.float())
        max_steps = max(max_steps, float(r.max()))
        tensors += 1
    l2 = math.sqrt(sq)
    if ratios:
        allr = torch.cat([r.flatten() for r in ratios])
        q1, q3 = float(allr.quantile(0.25)), float(allr.quantile(0.75))
        iqm = float(allr[(allr >= q1) & (allr <= q3)].mean())
    else:
        iqm = max_steps = math.inf
    return {"success": True, "l2_norm": l2, "avg_l2_norm": math.inf if tensors == 0 else l2 / count,
            "avg_abs_diff": math.inf if tensors == 0 else ab / count, "max_diff": max_diff,
            "avg_steps_behind": iqm, "interquartile_mean_steps_behind": iqm, "max_steps_behind": max_steps,
            "param_count": count, "learning_rate": learning_rate}


# --------------------------------------------------------------------------------------- #
# index overlap (copy detection)
# --------------------------------------------------------------------------------------- #
@torch.no_grad()
async def check_uid_index_overlap(neuron, gather_result, window: int, *, overlap_threshold: float = 0.90) -> dict:
    """Size-weighted mean, over all tensors, of the per-chunk fraction of peer *i*'s top-k indices
    that peer *j* also selected; pairs at or above the threshold are flagged and the later uploader
    is the offender.  Membership bitmaps make a pair cost O(chunks * k) instead of O(chunks * k^2)."""
    uids = list(getattr(gather_result, "uids", []))
    n = len(uids)
    empty = dict(pairs_checked=0, pairs_high_ovlap=0, ratio_high_ovlap=0.0, mean_overlap=0.0, min_overlap=0.0,
                 max_overlap=0.0, pairs_over_thresh=[], uids_over_thresh={})
    if n < 2:
        return empty
    stamps = await asyncio.gather(*[neuron.comms.gradient_timestamp(u, window - 1) for u in uids])
    ts = dict(zip(uids, stamps))
    acc: dict[tuple[int, int], list[float]] = defaultdict(lambda: [0.0, 0.0])
    tot_w = tot = 0.0
    device = neuron.config.device
    eng = getattr(neuron, "engine", None)
    staged = getattr(neuron, "staged_peers", None)
    m = getattr(neuron, "overlap_matrix", None)          # a sharded engine's ranks computed it together beforehand
    if m is not None and tuple(m.shape) != (n, n):
        m = None
    if m is None and eng is not None and eng.cuda and eng.world_size == 1 and staged == n:
        # the gathered payloads already sit in the engine's peer slots (slot j = uids[j]): one kernel over the
        # packed indices gives every pair's overlap
        m = eng.index_overlap(n)
    if m is not None:
        m = m.cpu()
        for i in range(n):
            for j in range(i + 1, n):
                acc[(i, j)] = [float(m[i, j]), 1.0]
                tot_w += float(m[i, j])
                tot += 1.0
    for pname, _ in (neuron.model.named_parameters() if not acc else ()):
        idxs_all = getattr(gather_result.state_dict, pname + "idxs", None)
        vals_all = getattr(gather_result.state_dict, pname + "vals", None)
        if idxs_all is None or vals_all is None:
            continue
        unpacked = []
        for i in range(n):
            ii = idxs_all[i] if isinstance(idxs_all, list) else idxs_all
            vv = vals_all[i] if isinstance(vals_all, list) else vals_all
            unpacked.append(unpack_12bit_indices(ii.to(device), vv.shape))
        idx = torch.stack(unpacked, 0)
        k = idx.shape[-1]
        if idx.numel() == 0:
            # nothing was kept for this tensor: the pairs count as compared, with nothing in common
            for i in range(n):
                for j in range(i + 1, n):
                    acc[(i, j)][1] += 0.0
            continue
        idx = idx.reshape(n, -1, k)
        C = idx.shape[1]
        width = int(idx.max().item()) + 1
        member = torch.zeros(n, C, width, dtype=torch.bool, device=idx.device)
        member.scatter_(-1, idx, True)
        weight = C * k
        for i in range(n):
            for j in range(i + 1, n):
                frac = float(member[j].gather(-1, idx[i]).sum(-1).float().div(k).mean())
                tot_w += frac * weight
                tot += weight
                acc[(i, j)][0] += frac * weight
                acc[(i, j)][1] += weight
        del member
    high, over, offenders = 0, [], {}
    mn, mx, mn_pair, mx_pair = 1.0, 0.0, None, None
    for (i, j), (ws, wt) in acc.items():
        avg = ws / wt if wt > 0 else 0.0
        if avg < mn:
            mn, mn_pair = avg, (uids[i], uids[j])
        if avg > mx:
            mx, mx_pair = avg, (uids[i], uids[j])
        if avg >= overlap_threshold:
            high += 1
            ui, uj = uids[i], uids[j]
            offenders[ui if ts[ui] >= ts[uj] else uj] = determine_slash_egregiousness(avg)
            over.append((ui, uj, avg))
    mean = tot_w / tot if tot else 0.0
    logger.info(f"[overlap] {len(acc)} pairs, {high} ≥{overlap_threshold * 100:.0f}%, size-weighted mean {mean * 100:.1f}%")
    if offenders:
        logger.warning(f"[overlap] offenders: {sorted(offenders)}")
    return dict(pairs_checked=len(acc), pairs_high_ovlap=high, ratio_high_ovlap=high / len(acc) if acc else 0.0,
                mean_overlap=mean, min_overlap=mn if mn_pair is not None else 0.0,
                max_overlap=mx if mx_pair is not None else 0.0, pairs_over_thresh=over, uids_over_thresh=offenders)


def determine_slash_egregiousness(overlap_pct: float) -> str:
    if overlap_pct < 0.0 or overlap_pct > 1.0:
        raise ValueError(f"overlap_pct must be between 0.0 and 1.0, got {overlap_pct}")
    if overlap_pct >= 0.6:
        return "mega"
    if overlap_pct >= 0.5:
        return "max"
    return "high"


def instantiate_slashing_multiplier() -> dict[str, float]:
    """Score multipliers applied per overlap level."""
    return {"high": 0.5, "max": 0.0, "mega": 0.0}
