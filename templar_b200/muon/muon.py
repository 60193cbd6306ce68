"""Muon optimizers.

* :class:`SingleDeviceMuonWithAuxAdam` — momentum (lerp) + Nesterov, Newton–Schulz orthogonalisation,
  ``max(1, rows/cols)^0.5`` scaling, decoupled weight decay; Adam for the auxiliary groups
  (reference: src/tplr/muon/muon.py:25-186).
* :class:`Muon` — the sharded variant (reference: src/tplr/muon/muon_fsdp2.py:31-370): every 2-D
  parameter has an owner rank ``index % world``; the gradient shards are gathered to the owner, which
  orthogonalises the full matrix (``0.2 * sqrt(max(shape))`` RMS scaling when ``rms_scale``) and scatters
  the update shards back; up to ``prefetch`` gathers are in flight.  DTensor parameters sharded on
  dim 0 use ``dist.gather`` / ``dist.scatter``; plain tensors take the single-device path.  Tensor- and
  expert-parallel meshes are rejected, as in the reference.
"""

from __future__ import annotations

from collections import deque

import torch
import torch.distributed as dist

from .newton_schulz import newton_schulz, zeropower_via_newtonschulz5

zeropower_via_newtonschulz5_optimized = newton_schulz       # the kernel-backed chain, under the reference's name for it


def apply_momentum(grad, momentum, beta: float, nesterov: bool):
    """Momentum step in place (``momentum <- lerp(momentum, grad, 1 - beta)``) and the direction to orthogonalise:
    the Nesterov look-ahead (written into ``grad``) or the momentum itself; 4-D filters flattened to matrices
    (reference: src/tplr/muon/muon_fsdp2.py:31-36)."""
    momentum.lerp_(grad, 1 - beta)
    update = grad.lerp_(momentum, beta) if nesterov else momentum
    if update.ndim == 4:
        update = update.view(len(update), -1)
    return update


def apply_scaling(update, rms_scale: bool = False):
    """Step-size scaling of an orthogonalised [rows, cols] direction: ``0.2 * sqrt(max(rows, cols))`` (matches the
    RMS of an Adam step) or ``sqrt(max(1, rows / cols))`` (reference: src/tplr/muon/muon_fsdp2.py:39-47)."""
    rows, cols = update.shape[-2], update.shape[-1]
    return update * (0.2 * max(rows, cols) ** 0.5 if rms_scale else max(1, rows / cols) ** 0.5)


def muon_update(grad, momentum, beta: float = 0.95, nesterov: bool = True, rms_scale: bool = False):
    update = apply_momentum(grad, momentum, beta, nesterov)
    return apply_scaling(newton_schulz(update).to(grad.dtype), rms_scale)


def adam_update(grad, buf1, buf2, step, betas, eps):
    buf1.lerp_(grad, 1 - betas[0])
    buf2.lerp_(grad.square(), 1 - betas[1])
    return (buf1 / (1 - betas[0] ** step)) / ((buf2 / (1 - betas[1] ** step)).sqrt() + eps)


def _normalise_groups(param_groups, sharded: bool):
    for g in param_groups:
        assert "use_muon" in g, "every group needs use_muon"
        if g["use_muon"]:
            g.setdefault("lr", 0.02)
            g.setdefault("momentum", 0.95)
            g.setdefault("weight_decay", 0)
            if sharded:
                g.setdefault("rms_scale", True)
                g.setdefault("nesterov", True)
        else:
            g.setdefault("lr", 3e-4)
            g.setdefault("betas", (0.9, 0.95))
            g.setdefault("eps", 1e-10)
            g.setdefault("weight_decay", 0)
    return param_groups


def _adam_group_step(opt, group):
    for p in group["params"]:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        st = opt.state[p]
        if not st:
            st["exp_avg"], st["exp_avg_sq"], st["step"] = torch.zeros_like(p), torch.zeros_like(p), 0
        st["step"] += 1
        upd = adam_update(p.grad, st["exp_avg"], st["exp_avg_sq"], st["step"], group["betas"], group["eps"])
        p.mul_(1 - group["lr"] * group["weight_decay"])
        p.add_(upd, alpha=-group["lr"])


class SingleDeviceMuonWithAuxAdam(torch.optim.Optimizer):
    def __init__(self, param_groups):
        super().__init__(_normalise_groups(param_groups, sharded=False), dict())

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if not group["use_muon"]:
                _adam_group_step(self, group)
                continue
            for p in group["params"]:
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                st = self.state[p]
                if not st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                upd = muon_update(p.grad, st["momentum_buffer"], beta=group["momentum"])
                p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(upd.reshape(p.shape), alpha=-group["lr"])
        return loss


class _LocalWork:
    def __init__(self, p, state, group, index):
        self.p, self.state, self.group = p, state, group

    def start(self):
        g = self.group
        upd = muon_update(self.p.grad, self.state["momentum_buffer"], g["momentum"], g["nesterov"], g["rms_scale"])
        self.p.mul_(1 - g["lr"] * g["weight_decay"])
        self.p.add_(upd.reshape(self.p.shape), alpha=-g["lr"])

    def finish(self):
        return None


class _ShardedWork:
    """dim-0 sharded DTensor parameter on a 1-D mesh: gather shards → owner orthogonalises → scatter."""

    def __init__(self, p, state, group, index):
        self.p, self.state, self.group, self.index = p, state, group, index
        self.mesh = p.device_mesh
        self.pg = self.mesh.get_group()
        self.world, self.rank = dist.get_world_size(self.pg), dist.get_rank(self.pg)
        self.owner = index % self.world
        self.handle = None

    def start(self):
        g = self.group
        grad = self.p.grad.to_local()
        mom = self.state["momentum_buffer"].to_local()
        self.local = apply_momentum(grad, mom, g["momentum"], g["nesterov"]).contiguous()
        self.gathered = ([torch.empty_like(self.local) for _ in range(self.world)] if self.rank == self.owner else None)
        self.handle = dist.gather(self.local, self.gathered, dst=dist.get_global_rank(self.pg, self.owner), group=self.pg,
                                  async_op=True)

    def finish(self):
        g = self.group
        self.handle.wait()
        out = torch.empty_like(self.local)
        parts = None
        if self.rank == self.owner:
            full = torch.cat(self.gathered, dim=0)
            upd = apply_scaling(newton_schulz(full).to(self.local.dtype), g["rms_scale"])
            parts = [c.contiguous() for c in upd.chunk(self.world, dim=0)]
        dist.scatter(out, parts, src=dist.get_global_rank(self.pg, self.owner), group=self.pg)
        local_p = self.p.to_local()
        local_p.mul_(1 - g["lr"] * g["weight_decay"])
        local_p.add_(out, alpha=-g["lr"])


class Muon(torch.optim.Optimizer):
    PREFETCH = 8

    def __init__(self, param_groups):
        super().__init__(_normalise_groups(param_groups, sharded=True), dict())

    @staticmethod
    def _work_class(p):
        if hasattr(p, "device_mesh") and hasattr(p, "to_local"):
            if p.device_mesh.ndim == 1:
                return _ShardedWork, Muon.PREFETCH
            raise NotImplementedError("Muon on tensor-/expert-parallel meshes is not supported")
        return _LocalWork, 1

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        dq: deque = deque()
        for group in self.param_groups:
            if not group["use_muon"]:
                _adam_group_step(self, group)
                continue
            for i, p in enumerate(group["params"]):
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                st = self.state[p]
                if not st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                cls, depth = self._work_class(p)
                w = cls(p, st, group, i)
                w.start()
                dq.append(w)
                if len(dq) > depth:
                    dq.popleft().finish()
        for w in dq:
            w.finish()
        return loss
