"""Device-resident window pipeline of a miner / validator node.

One object owns every per-window buffer of a rank and drives the fused kernels:

    snapshot()            theta0 <- master                       (start of a window)
    micro_step()          forward + backward of one micro-batch, fp32 gradient accumulation
    optimizer_step()      cross-rank gradient reduction into the owned shard, global-norm clip,
                          fused AdamW on the shard, bf16 parameters pushed to every rank
    compress()            e <- gamma e + (theta0 - theta); chunk DCT; top-k; 12-bit pack; residual
    load_peer_payload()   place a peer's packed payload in a device slot
    outer_step()          per-peer norms -> median clip -> pull/unpack/mean/iDCT -> theta <- theta0 - lr g
    apply_single_peer()/restore()   the validator's before/after evaluation of one peer

Differences from the reference's flow (neurons/miner.py:536-795, src/tplr/neurons.py:47-476,
src/tplr/distributed.py:364-545): the parameter snapshot stays in HBM instead of pinned
host memory, every rank compresses and aggregates its own chunk-aligned shard instead of an
owner rank handling whole tensors and rank 0 decompressing everything, and no step reads a
scalar back to the host.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from .. import compress as C
from ..ops import functional as OF
from ..ops import native
from .flat import FlatParamStore


@dataclass
class EngineConfig:
    topk: int = 32
    target_chunk: int = 64
    use_dct: bool = True
    momentum_decay: float = 0.95
    outer_lr: float = 0.4
    outer_update: str = "sgd"          # "sgd" (reference behaviour) or "sign"
    outer_weight_decay: float = 0.0
    inner_lr: float = 1.17e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    max_peers: int = 8
    val_dtype: torch.dtype = torch.float32
    inner_optimizer: str = "adamw"     # "adamw" (fused kernel) or "muon" (Newton-Schulz on the own GEMM + auxiliary Adam)
    muon_momentum: float = 0.95
    muon_nesterov: bool = True
    muon_weight_decay: float = 0.01
    muon_aux_lr_scale: tuple = (("head", 0.5), ("embed", 0.5), ("scalar", 0.2))
    quantize: bool = False             # 8-bit value codes on the wire (the reference miner's format)
    quant_bins: int = 256
    quant_range: float = 6.0
    shard_params: bool = False         # weights and gradients held as shards too (the FSDP role), gathered per block
    gather_buffers: int = 0            # block buffers in rotation; >= the number of blocks keeps every block gathered;
                                       # 0: all blocks when the weights are at most 8 GiB, else two


def peer_slice(state_dict: dict, j: int) -> dict:
    """Peer ``j``'s entries of a gathered state dict whose values are per-peer lists."""
    return {k: (v[j] if isinstance(v, list) else v) for k, v in state_dict.items()}


class WindowEngine:
    def __init__(self, model: torch.nn.Module, cfg: EngineConfig, *, device=None, rank: int = 0,
                 world_size: int = 1, group=None, heap=None, compute_dtype: torch.dtype | None = None,
                 materialize=None, replicate_group=None, replicate_size: int = 1):
        """``rank`` / ``world_size`` / ``group`` / ``heap`` describe the ranks that share one copy of the sharded
        state.  ``replicate_group`` (``replicate_size`` ranks, one from every such copy, all holding the same
        shard) adds the reference's ``dp_replicate`` dimension: the gradient shards are summed over it with one
        all-reduce per inner step, after which every copy takes the same step.  ``world_size == 1`` with a
        replicate group is plain data parallelism (whole state on every rank, bucketed gradient all-reduce);
        both together are the hybrid layout (src/tplr/model_factory.py:122-176, torchtitan's HSDP / DDP)."""
        self.cfg = cfg
        self.model = model
        self.rank, self.world_size, self.group = rank, world_size, group
        self.replicate_group, self.replicate_size = replicate_group, max(1, int(replicate_size))
        if self.replicate_size > 1 and replicate_group is None:
            raise ValueError("replicate_size > 1 needs the process group of the replicas")
        self.dp_size = world_size * self.replicate_size       # ranks whose gradients are averaged
        self.replica = dist.get_rank(replicate_group) if self.replicate_size > 1 else 0     # which copy this rank is in
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        if self.device.type == "meta":
            raise ValueError("the model is on the meta device: pass the device its shards are to live on")
        self.cuda = self.device.type == "cuda"
        self.heap = heap
        if materialize is not None and not cfg.shard_params:
            raise ValueError("a model on the meta device is materialised tensor by tensor only with shard_params")
        if compute_dtype is None:
            compute_dtype = torch.bfloat16 if self.cuda else torch.float32
        alloc = None
        if heap is not None:
            def alloc(n, dtype, symmetric=False):
                if symmetric:
                    return heap.alloc(n, dtype)
                return torch.zeros(n, dtype=dtype, device=self.device)
        self.status = OF.status_word(self.device) if self.cuda else torch.zeros(1, dtype=torch.int32)
        self.fsdp = bool(cfg.shard_params)
        if self.fsdp and self.cuda and world_size > 1 and heap is None:
            raise ValueError("shard_params on CUDA with several ranks needs the symmetric heap (peer-memory gathers)")
        self.store = FlatParamStore(model, compute_dtype=compute_dtype, device=self.device,
                                    target_chunk=cfg.target_chunk, topk=cfg.topk, rank=rank,
                                    world_size=world_size, alloc=alloc, shard_params=self.fsdp,
                                    n_buffers=cfg.gather_buffers, group=group, heap=heap, status=self.status,
                                    materialize=materialize)
        L = self.layout = self.store.layout
        n_shard = self.store.n_shard
        z = lambda n, dt=torch.float32: torch.zeros(n, dtype=dt, device=self.device)
        self.exp_avg, self.exp_avg_sq = z(n_shard), z(n_shard)
        self.theta0 = z(n_shard)
        self.ef = z(n_shard)
        self.adam_step = 0
        # payload: this node's own (full layout) + peer slots
        palloc = (lambda n, dt: heap.alloc(n, dt)) if heap is not None else z
        self.own_idx = palloc(L.idx_bytes, torch.uint8)
        self.own_val = palloc(L.val_elems, torch.float32)
        self.peer_idx = [palloc(L.idx_bytes, torch.uint8) for _ in range(self._slots())]
        self.peer_val = [palloc(L.val_elems, cfg.val_dtype) for _ in range(self._slots())]
        self.basis = L.basis_table().to(self.device)
        self._desc = {}
        for square in (True, False):
            arr = L.descriptors(rank if world_size > 1 else None, square=square)
            self._desc[square] = (torch.from_numpy(arr.view(np.uint8).reshape(-1).copy()).to(self.device), len(arr),
                                  int(arr["n_chunks"].sum()) if len(arr) else 0)
        # the tensor-core DCT kernels need every chunk of the square table to be 64 x 64 with 16-byte aligned rows
        import os
        sq = L.descriptors(rank if world_size > 1 else None, square=True)
        self._dct_on_tensor_cores = bool(
            self.cuda and len(sq) and (sq["h"] == 64).all() and (sq["w"] == 64).all()
            and (sq["cols"] % 4 == 0).all() and (sq["elem_off"] % 4 == 0).all()
            and os.environ.get("TPLR_DCT_BACKEND", "tcgen05") == "tcgen05")
        self._compress_on_tensor_cores = os.environ.get("TPLR_COMPRESS_BACKEND", "tcgen05") == "tcgen05"
        full = L.descriptors(None, square=None)
        self._desc_full = (torch.from_numpy(full.view(np.uint8).reshape(-1).copy()).to(self.device), len(full))
        P = cfg.max_peers
        self.sumsq_partial = z(P * L.n_params * 8)
        self.peer_norms, self.clip = z(P * L.n_params), z(P * L.n_params)
        self.median = z(L.n_params)
        self.skip = z(L.n_params, torch.int32)
        self.gnorm_sq = z(1)
        self._sumsq_scratch = z(native.lib().tplr_sumsq_blocks() if self.cuda else 1)
        self.window_open = False
        self.peer_group = None                    # set by LocalPeerGroup.attach(): co-located nodes on the same heap
        self._h2d_stream = None                   # side stream of load_peer_payloads_async
        self._h2d_pending = None                  # event: payloads staged on the side stream and not yet joined
        self.rank_payloads: dict = {}             # CPU stand-in for peer memory: rank -> (own_idx, own_val) copies
        model._window_engine = self
        model._param_gather = self.store.gather          # None unless shard_params: the model gates its blocks on it
        if self.fsdp and self.cuda:
            rec = self.store.stage_blocks()
            self._grad_stage_table = (torch.tensor(rec, dtype=torch.int64, device=self.device).reshape(-1, 3), len(rec))
        self._refresh_samples()

    # -- phase marks ------------------------------------------------------------------------------
    def start_trace(self) -> None:
        """Record a CUDA event at every named point of the window from now on (read with :meth:`trace_ms`)."""
        self._trace = []
        self._mark("start")

    def _mark(self, name: str) -> None:
        tr = getattr(self, "_trace", None)
        if tr is None or not self.cuda:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        tr.append((name, ev))

    def trace_ms(self) -> dict:
        """Device time between consecutive marks since :meth:`start_trace`, summed per name; ends the trace.
        A mark's time includes any wait for another rank that its kernels contain (the barriers)."""
        tr, self._trace = self._trace, None
        torch.cuda.synchronize(self.device)
        out: dict[str, float] = {}
        for (_, a), (name, b) in zip(tr, tr[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    def _slots(self) -> int:
        """Peer-payload slots held by this rank: with a symmetric heap the peers are spread
        round-robin over the ranks, otherwise every rank keeps all of them."""
        if self.heap is None:
            return self.cfg.max_peers
        return -(-self.cfg.max_peers // self.world_size)

    def slot_of(self, peer: int) -> tuple[int, int]:
        """(owner rank, slot index) of peer ``peer``'s payload."""
        if self.heap is None:
            return self.rank, peer
        return peer % self.world_size, peer // self.world_size

    # ------------------------------------------------------------------------------------ #
    # inner loop
    # ------------------------------------------------------------------------------------ #
    @torch.no_grad()
    def snapshot(self) -> None:
        """theta0 <- master: opens a window (the next compress / outer step refer to this snapshot)."""
        self.theta0.copy_(self.store.master_shard)
        self._mark("snapshot")
        self.window_open = True

    def zero_grad(self) -> None:
        self.store.zero_grad()
        if self.fsdp and self.world_size > 1:
            self._barrier()                         # peers add into this shard: none may start before it is zero

    def micro_step(self, tokens: torch.Tensor, labels: torch.Tensor, grad_scale: float = 1.0) -> torch.Tensor:
        """Forward + backward of one micro-batch; returns the (device) mean loss."""
        loss = self.model.loss(tokens, labels, grad_scale)
        loss.backward()
        self._mark("micro_steps")
        return loss.detach()

    @torch.no_grad()
    def optimizer_step(self, lr: float | None = None) -> None:
        """Clip by global norm and apply AdamW on the owned shard; refresh the compute copy."""
        cfg, st = self.cfg, self.store
        lr = cfg.inner_lr if lr is None else lr
        self.adam_step += 1
        if self.fsdp:
            return self._muon_step_sharded(lr) if cfg.inner_optimizer == "muon" else self._optimizer_step_sharded(lr)
        if self.world_size > 1:
            self._reduce_grads()
        self._replicate_reduce(st.grad[st.lo:st.hi])
        if cfg.inner_optimizer == "muon":
            return self._muon_step(lr)
        gshard = st.grad[st.lo:st.hi]
        n = st.hi - st.lo
        if self.cuda:
            L = native.lib()
            native.check(L.tplr_sumsq(gshard.data_ptr(), n, self._sumsq_scratch.data_ptr(), self.gnorm_sq.data_ptr(),
                                      native.stream_ptr()), "sumsq")
            if self.world_size > 1:
                dist.all_reduce(self.gnorm_sq, group=self.group)
            self._mark("opt.grad_norm_allreduce")
            shadows = self._compute_shadow_ptrs()
            native.check(L.tplr_adamw(st.master_shard.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                                      gshard.data_ptr(), native.ptr_array(shadows), len(shadows), n, lr, cfg.betas[0],
                                      cfg.betas[1], cfg.eps, cfg.weight_decay, self.adam_step, 1.0 / self.dp_size,
                                      cfg.max_grad_norm, self.gnorm_sq.data_ptr(), 1, native.stream_ptr()), "adamw")
            self._mark("opt.adamw_and_weight_push")
            if self.world_size > 1:
                self._barrier()
                self._mark("opt.barrier_after_push")
                st.grad.zero_()
                self._mark("opt.zero_grad")
            return
        # CPU path (same arithmetic); gradients were summed over ranks, the mean is what is applied
        g = gshard / self.dp_size
        self.gnorm_sq.copy_((g * g).sum().reshape(1))
        if self.world_size > 1:
            dist.all_reduce(self.gnorm_sq, group=self.group)
        coef = torch.clamp(cfg.max_grad_norm / (self.gnorm_sq.sqrt() + 1e-6), max=1.0) if cfg.max_grad_norm > 0 else 1.0
        g = g * coef
        b1, b2 = cfg.betas
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.adam_step, 1 - b2 ** self.adam_step
        p = st.master_shard
        p.mul_(1 - lr * cfg.weight_decay)
        p.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt() + cfg.eps, value=-lr)
        st.grad.zero_()
        self._publish_compute()

    @torch.no_grad()
    def _optimizer_step_sharded(self, lr: float) -> None:
        """Inner step under ``shard_params``.  The matrices' gradients are already summed in the owners' shards
        (the weight-gradient GEMMs added them there); what was accumulated locally in full size (embedding rows,
        norm weights; on CPU everything) is reduced into the shards now.  Then global-norm clip and AdamW on the
        shard, writing the new bf16 weights into this rank's own weight shard, from which the peers gather.

        Ordering across ranks: (1) a barrier so that every rank's backward pass, and with it every remote add
        into this shard, is complete; (2) the norm all-reduce also orders every rank's pull of the staged
        gradients before anybody zeroes its staging buffer; (3) a barrier after the zeroing, because the next
        backward pass of a peer adds into this rank's shard."""
        cfg, st = self.cfg, self.store
        n = st.n_shard
        gshard = st.grad_shard[:n]
        self._barrier()
        self._mark("opt.barrier_before_reduce")
        if self.cuda:
            L = native.lib()
            table, n_rec = self._grad_stage_table
            if n_rec:
                stages = ([self.heap.peer_ptr(st.stage, r) for r in range(self.world_size)]
                          if (self.heap is not None and self.world_size > 1) else [st.stage.data_ptr()])
                native.check(L.tplr_reduce_blocks(native.ptr_array(stages), len(stages), table.data_ptr(), n_rec,
                                                  st.grad_shard.data_ptr(), native.stream_ptr()), "reduce_blocks")
            self._mark("opt.reduce_staged")
            self._replicate_reduce(gshard)
            native.check(L.tplr_sumsq(gshard.data_ptr(), n, self._sumsq_scratch.data_ptr(), self.gnorm_sq.data_ptr(),
                                      native.stream_ptr()), "sumsq")
            if self.world_size > 1:
                dist.all_reduce(self.gnorm_sq, group=self.group)
            self._mark("opt.grad_norm_allreduce")
            shadows = [st.compute_shard.data_ptr()]
            native.check(L.tplr_adamw(st.master_shard.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                                      gshard.data_ptr(), native.ptr_array(shadows), 1, n, lr, cfg.betas[0],
                                      cfg.betas[1], cfg.eps, cfg.weight_decay, self.adam_step, 1.0 / self.dp_size,
                                      cfg.max_grad_norm, self.gnorm_sq.data_ptr(), 1, native.stream_ptr()), "adamw")
            self._mark("opt.adamw")
        else:
            self._reduce_staged_cpu()
            self._replicate_reduce(gshard)
            g = gshard / self.dp_size
            self.gnorm_sq.copy_((g * g).sum().reshape(1))
            if self.world_size > 1:
                dist.all_reduce(self.gnorm_sq, group=self.group)
            coef = torch.clamp(cfg.max_grad_norm / (self.gnorm_sq.sqrt() + 1e-6), max=1.0) if cfg.max_grad_norm > 0 else 1.0
            g = g * coef
            b1, b2 = cfg.betas
            self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
            self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1, bc2 = 1 - b1 ** self.adam_step, 1 - b2 ** self.adam_step
            p = st.master_shard
            p.mul_(1 - lr * cfg.weight_decay)
            p.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt() + cfg.eps, value=-lr)
            st.compute_shard[:n].copy_(p.to(st.compute_dtype))
        st.zero_grad()
        self._mark("opt.zero_grad")
        st.gather.invalidate()
        self._barrier()
        self._mark("opt.barrier_after_zero")

    # -- Muon on sharded parameters ---------------------------------------------------------------------- #
    def _reduce_staged(self) -> None:
        """Staged gradients (embedding rows, norm weights; on CPU everything) into the owners' gradient shards."""
        st = self.store
        if not self.cuda:
            return self._reduce_staged_cpu()
        table, n_rec = self._grad_stage_table
        if n_rec:
            stages = ([self.heap.peer_ptr(st.stage, r) for r in range(self.world_size)]
                      if (self.heap is not None and self.world_size > 1) else [st.stage.data_ptr()])
            native.check(native.lib().tplr_reduce_blocks(native.ptr_array(stages), len(stages), table.data_ptr(), n_rec,
                                                         st.grad_shard.data_ptr(), native.stream_ptr()), "reduce_blocks")

    def _matrix_tables(self):
        """Per orthogonalised matrix: its owner rank (round-robin, as the reference's sharded Muon assigns them,
        src/tplr/muon/muon_fsdp2.py:319-343) and every rank's rows of it as (rank, first element in the matrix,
        elements, offset in that rank's shard arrays)."""
        if getattr(self, "_muon_tables", None) is None:
            out, k = [], 0
            for sp in self.layout.specs:
                if self.muon_class(sp.name, len(sp.shape)) != "muon":
                    continue
                parts = []
                for r in range(self.world_size):
                    for s2, a, b, la in self.layout.segments(r):
                        if s2 is sp:
                            parts.append((r, a - sp.offset, b - a, la))
                out.append((sp, k % self.world_size, parts))
                k += 1
            self._muon_tables = out
        return self._muon_tables

    def _move_rows(self, parts, full: torch.Tensor, to_full: bool) -> None:
        """CUDA: rows of one matrix between the ranks' gradient shards (peer memory) and ``full`` on this rank."""
        st = self.store
        rec = []
        for r, off, n, la in parts:
            base = (self.heap.peer_ptr(st.grad_shard, r) if (self.heap is not None and self.world_size > 1)
                    else st.grad_shard.data_ptr()) + la * 4
            mine = full.data_ptr() + off * 4
            for o in range(0, n * 4, 1 << 20):
                m = min(1 << 20, n * 4 - o)
                rec.append((base + o, mine + o, m) if to_full else (mine + o, base + o, m))
        table = torch.tensor(rec, dtype=torch.int64, device=self.device)
        native.check(native.lib().tplr_copy_blocks(table.data_ptr(), len(rec), 0, native.stream_ptr()), "copy_blocks")
        self._keep_alive.append(table)

    @torch.no_grad()
    def _muon_step_sharded(self, lr: float) -> None:
        """Muon on sharded parameters.  Momentum and the Nesterov blend are element-wise and run on the shards; the
        blended direction of every hidden matrix is then collected on that matrix's owner rank (matrices are dealt
        round-robin), orthogonalised there (Newton-Schulz on the own GEMM) and its rows are sent back to the ranks
        that hold them, which apply them to their master shards.  Embeddings, the head and vectors get Adam, as in
        :meth:`_muon_step`.  The reference does the same with ``dist.gather`` / ``dist.scatter`` per matrix
        (src/tplr/muon/muon_fsdp2.py:77-158); here the rows move over peer memory between two barriers."""
        from ..muon.muon import adam_update
        from ..muon.newton_schulz import newton_schulz

        cfg, st = self.cfg, self.store
        n = st.n_shard
        self._barrier()                                     # every rank's backward pass (remote adds) is complete
        self._reduce_staged()
        g = st.grad_shard[:n]
        self._replicate_reduce(g)
        g.mul_(1.0 / self.dp_size)
        self.gnorm_sq.copy_((g * g).sum().reshape(1))
        if self.world_size > 1:
            dist.all_reduce(self.gnorm_sq, group=self.group)
        if cfg.max_grad_norm > 0:
            g.mul_(torch.clamp(cfg.max_grad_norm / (self.gnorm_sq.sqrt() + 1e-6), max=1.0))
        beta = cfg.muon_momentum
        segs = [(sp, self.muon_class(sp.name, len(sp.shape)), a, b, la) for sp, a, b, la in self.layout.segments(self.rank)]
        for sp, cls, a, b, la in segs:
            if cls != "muon":
                continue
            gs, ms = g[la: la + (b - a)], self.exp_avg[la: la + (b - a)]
            ms.lerp_(gs, 1 - beta)
            if cfg.muon_nesterov:
                gs.lerp_(ms, beta)
            else:
                gs.copy_(ms)
        self._barrier()                                     # every rank's directions are in its gradient shard
        self._keep_alive = []
        for sp, owner, parts in self._matrix_tables():
            shape = (sp.shape[0], sp.numel // sp.shape[0])
            if self.cuda:
                if owner != self.rank:
                    continue
                full = torch.empty(shape, dtype=torch.float32, device=self.device)
                self._move_rows(parts, full, to_full=True)
                o = (newton_schulz(full).float() * max(1.0, shape[0] / shape[1]) ** 0.5).contiguous()
                self._move_rows(parts, o, to_full=False)
            else:
                # gloo: every rank rebuilds the matrix from broadcasts and orthogonalises it (tiny test models)
                full = torch.zeros(shape, dtype=torch.float32)
                flat = full.view(-1)
                for r, off, cnt, la in parts:
                    piece = flat[off: off + cnt]
                    if r == self.rank:
                        piece.copy_(g[la: la + cnt])
                    if self.world_size > 1:
                        dist.broadcast(piece, src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                                       group=self.group)
                o = (newton_schulz(full).float() * max(1.0, shape[0] / shape[1]) ** 0.5).reshape(-1)
                for r, off, cnt, la in parts:
                    if r == self.rank:
                        g[la: la + cnt].copy_(o[off: off + cnt])
        self._barrier()                                     # the orthogonalised rows have arrived
        self._keep_alive = []
        scale = dict(cfg.muon_aux_lr_scale)
        for sp, cls, a, b, la in segs:
            p = st.master_shard[la: la + (b - a)]
            if cls == "muon":
                p.mul_(1 - lr * cfg.muon_weight_decay)
                p.add_(g[la: la + (b - a)], alpha=-lr)
            else:
                upd = adam_update(g[la: la + (b - a)], self.exp_avg[la: la + (b - a)], self.exp_avg_sq[la: la + (b - a)],
                                  self.adam_step, cfg.betas, cfg.eps)
                lr_c = lr * scale.get(cls, 1.0)
                p.mul_(1 - lr_c * cfg.weight_decay)
                p.add_(upd, alpha=-lr_c)
        if self.cuda:
            native.check(native.lib().tplr_cast_bf16(st.master_shard.data_ptr(), st.compute_shard.data_ptr(), n,
                                                     native.stream_ptr()), "cast_bf16")
        else:
            st.compute_shard[:n].copy_(st.master_shard.to(st.compute_dtype))
        st.zero_grad()
        st.gather.invalidate()
        self._barrier()

    def _reduce_staged_cpu(self) -> None:
        """CPU / gloo: every tensor's gradient was accumulated locally in full size (``stage``); the parts that a
        rank owns are summed onto it, piece by piece in an order that is the same on every rank."""
        st, L = self.store, self.layout
        for r in range(self.world_size):
            dst = dist.get_global_rank(self.group, r) if self.group is not None else r
            for sp, a, b, la in L.segments(r):
                so = st.stage_off[sp.name] + (a - sp.offset)
                part = st.stage[so: so + (b - a)].clone()
                if self.world_size > 1:
                    dist.reduce(part, dst=dst, group=self.group)
                if r == self.rank:
                    st.grad_shard[la: la + (b - a)].add_(part)

    # -- Muon as the inner optimizer ------------------------------------------------------------- #
    @staticmethod
    def muon_class(name: str, ndim: int) -> str:
        """Parameter classes of the reference's Muon set-up (neurons/trainer.py:338-390): matrices of the
        blocks are orthogonalised, embeddings / the output head / vectors get Adam with their own LR scale."""
        if "embed" in name:
            return "embed"
        if "lm_head" in name or name == "output.weight":
            return "head"
        return "muon" if ndim >= 2 else "scalar"

    def _segments(self):
        """[(spec, class, a, b)]: the part [a, b) (flat element range) of every tensor inside this rank's shard."""
        return [(s, self.muon_class(s.name, len(s.shape)), a, b) for s, a, b, _ in self.layout.segments(self.rank)]

    @torch.no_grad()
    def _muon_step(self, lr: float) -> None:
        """One inner step with Muon on the hidden matrices and Adam on the rest, on the flat sharded state.

        Gradient clipping by the global norm first, as for AdamW.  ``exp_avg`` is the Muon momentum for the
        matrices and Adam's first moment for the others.  The momentum-blended direction is written back into
        the gradient shard, the shards are exchanged so that every rank holds whole matrices, and each rank
        orthogonalises the matrices that intersect its shard (Newton-Schulz on the own GEMM) and updates its
        part of the fp32 master weights.  Scaling ``max(1, rows / cols) ** 0.5`` and decoupled weight decay as in
        the reference's single-device Muon (src/tplr/muon/muon.py:25-186)."""
        from ..muon.muon import adam_update
        from ..muon.newton_schulz import newton_schulz

        cfg, st = self.cfg, self.store
        g = st.grad[st.lo:st.hi]
        g.mul_(1.0 / self.dp_size)
        self.gnorm_sq.copy_((g * g).sum().reshape(1))
        if self.world_size > 1:
            dist.all_reduce(self.gnorm_sq, group=self.group)
        if cfg.max_grad_norm > 0:
            g.mul_(torch.clamp(cfg.max_grad_norm / (self.gnorm_sq.sqrt() + 1e-6), max=1.0))
        segs = self._segments()
        beta = cfg.muon_momentum
        for s, cls, a, b in segs:
            if cls != "muon":
                continue
            gs, ms = g[a - st.lo: b - st.lo], self.exp_avg[a - st.lo: b - st.lo]
            ms.lerp_(gs, 1 - beta)
            if cfg.muon_nesterov:
                gs.lerp_(ms, beta)
            else:
                gs.copy_(ms)
        if self.world_size > 1:
            self._allgather_grad()                  # every rank now holds the whole direction of every matrix
        scale = dict(cfg.muon_aux_lr_scale)
        for s, cls, a, b in segs:
            p = st.master_shard[a - st.lo: b - st.lo]
            if cls == "muon":
                u = st.grad[s.offset: s.offset + s.numel].view(s.shape)
                if u.ndim > 2:
                    u = u.reshape(u.shape[0], -1)
                rows, cols = u.shape
                o = newton_schulz(u).float() * max(1.0, rows / cols) ** 0.5
                p.mul_(1 - lr * cfg.muon_weight_decay)
                p.add_(o.reshape(-1)[a - s.offset: b - s.offset], alpha=-lr)
            else:
                lo_, hi_ = a - st.lo, b - st.lo
                upd = adam_update(g[lo_:hi_], self.exp_avg[lo_:hi_], self.exp_avg_sq[lo_:hi_], self.adam_step,
                                  cfg.betas, cfg.eps)
                lr_c = lr * scale.get(cls, 1.0)
                p.mul_(1 - lr_c * cfg.weight_decay)
                p.add_(upd, alpha=-lr_c)
        if self.cuda and st.compute is not st.master_shard:
            native.check(native.lib().tplr_cast_bf16(st.master_shard.data_ptr(),
                                                     st.compute.data_ptr() + st.lo * st.compute.element_size(),
                                                     st.hi - st.lo, native.stream_ptr()), "cast_bf16")
            if self.world_size > 1:
                self._barrier()
                self._allgather_compute_native()
        else:
            self._publish_compute()
        if self.world_size > 1:
            self._barrier()
        st.grad.zero_()

    def _allgather_grad(self) -> None:
        """Every rank's gradient shard to every other rank's full-size gradient buffer."""
        st = self.store
        if self.cuda and self.heap is not None:
            self._barrier()                         # nobody still reads the ranges that are overwritten now
            n = st.hi - st.lo
            src = st.grad.data_ptr() + st.lo * 4
            dsts = [self.heap.peer_ptr(st.grad, r) + st.lo * 4 for r in range(self.world_size) if r != self.rank]
            native.check(native.lib().tplr_push_copy(src, native.ptr_array(dsts), len(dsts), n * 4, native.stream_ptr()),
                         "push_copy")
            self._barrier()
            return
        for r in range(self.world_size):
            a, b = self.layout.shard_range(r)
            dist.broadcast(st.grad[a:b], src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                           group=self.group)

    def _compute_shadow_ptrs(self) -> list[int]:
        st = self.store
        if self.fsdp:
            return [st.compute_shard.data_ptr()]
        if st.compute is st.master_shard:
            return []
        esz = st.compute.element_size()
        if self.heap is not None and self.world_size > 1:
            return [self.heap.peer_ptr(st.compute, r) + st.lo * esz for r in range(self.world_size)]
        return [st.compute.data_ptr() + st.lo * esz]

    def _publish_compute(self) -> None:
        """CPU / generic path: compute[lo:hi] <- master shard, then make every rank's copy whole."""
        st = self.store
        if self.fsdp:
            st.refresh_compute_from_master()
            self._refresh_samples()
            return
        if st.compute is not st.master_shard:
            st.compute[st.lo:st.hi].copy_(st.master_shard.to(st.compute.dtype))
        if self.world_size > 1:
            self._allgather_compute()

    def _allgather_compute(self) -> None:
        st = self.store
        parts = [st.compute[a:b] for a, b in (self.layout.shard_range(r) for r in range(self.world_size))]
        for r, part in enumerate(parts):
            dist.broadcast(part, src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                           group=self.group)

    def _reduce_grads(self) -> None:
        st = self.store
        if self.cuda and self.heap is not None:
            self._barrier()
            self._mark("opt.barrier_before_reduce")
            ptrs = [self.heap.peer_ptr(st.grad, r) for r in range(self.world_size)]
            native.check(native.lib().tplr_reduce_shards(native.ptr_array(ptrs), self.world_size, self.rank, st.lo,
                                                         st.hi - st.lo, native.stream_ptr()), "reduce_shards")
            self._mark("opt.reduce_shards")
            return
        for r in range(self.world_size):
            a, b = self.layout.shard_range(r)
            dist.reduce(st.grad[a:b], dst=dist.get_global_rank(self.group, r) if self.group is not None else r,
                        group=self.group)

    def _global(self, r: int) -> int:
        """Global rank of rank ``r`` of this engine's group."""
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    REPLICATE_BUCKET = 64 * 1024 * 1024       # elements per all-reduce over the replicas (256 MB of fp32)

    def _replicate_reduce(self, gshard: torch.Tensor) -> None:
        """Sum this rank's gradient shard over the replicas (the ranks of the other copies that hold the same
        shard).  Issued in buckets so that no single collective holds more than a quarter of a gigabyte of
        NCCL work in flight; all of them are enqueued before the first wait."""
        if self.replicate_size <= 1 or gshard.numel() == 0:
            return
        works = [dist.all_reduce(gshard[a:a + self.REPLICATE_BUCKET], group=self.replicate_group, async_op=True)
                 for a in range(0, gshard.numel(), self.REPLICATE_BUCKET)]
        for w in works:
            w.wait()
        self._mark("opt.replicate_allreduce")

    def _barrier(self) -> None:
        self.join_payloads()                      # a barrier publishes this rank's slots to the ranks that pull from them
        if self.world_size > 1:
            if self.heap is not None and self.cuda:
                self.heap.barrier()
            else:
                dist.barrier(group=self.group)

    # ------------------------------------------------------------------------------------ #
    # compression of the window's pseudo-gradient
    # ------------------------------------------------------------------------------------ #
    @torch.no_grad()
    def compress(self, null_round: bool = False, own_slot_ptrs: tuple[int, int] | None = None) -> None:
        """Runs the fused compress kernel over the owned shard.

        Reads theta0 and the current master (delta = theta0 - theta), updates the error feedback
        in place and writes this rank's part of the node payload into ``own_idx`` / ``own_val``
        (or into ``own_slot_ptrs``, e.g. the hosting rank's buffers in peer memory).
        """
        cfg, st = self.cfg, self.store
        self._own_merged = False
        if not self.cuda:
            return self._compress_torch(null_round)
        idx_ptr, val_ptr = own_slot_ptrs or (self.own_idx.data_ptr(), self.own_val.data_ptr())
        if self.world_size > 1 and own_slot_ptrs is None:
            self.own_idx.zero_()                    # only this rank's chunks are written: the rest must read as
            self.own_val.zero_()                    # zero for merge_own_payload()
        bias = 0                                    # descriptor offsets address the shard arrays directly
        L = native.lib()
        for square in (True, False):
            desc, n_desc, n_chunks = self._desc[square]
            if n_chunks == 0:
                continue
            if square and cfg.use_dct and self._dct_on_tensor_cores and self._compress_on_tensor_cores:
                native.check(L.tplr_compress_chunks_tc(desc.data_ptr(), n_desc, n_chunks, self.basis.data_ptr(),
                                                       self.ef.data_ptr() - bias, self.theta0.data_ptr() - bias,
                                                       st.master_shard.data_ptr() - bias, idx_ptr, val_ptr,
                                                       self.status.data_ptr(), cfg.momentum_decay, 1, int(null_round), 1,
                                                       native.stream_ptr()), "compress_tc")
                continue
            native.check(L.tplr_compress_chunks(desc.data_ptr(), n_desc, n_chunks, self.basis.data_ptr(),
                                                self.ef.data_ptr() - bias, self.theta0.data_ptr() - bias,
                                                st.master_shard.data_ptr() - bias, idx_ptr, val_ptr,
                                                self.status.data_ptr(), cfg.momentum_decay, int(cfg.use_dct), 1,
                                                int(null_round), 1, int(not square), native.stream_ptr()), "compress")
        self._mark("compress.kernels")
        if cfg.quantize:
            self._quantize_own(on_rank0=own_slot_ptrs is not None)

    def _quant_buffers(self, n_bins: int | None = None):
        """codes [val_elems] uint8, table [n_params, bins + 2] fp32 (lookup | shift | scale), scratch."""
        nb, np_ = (self.cfg.quant_bins if n_bins is None else n_bins), self.layout.n_params
        if getattr(self, "_q_codes", None) is None or self._q_table.shape[1] != nb + 2:
            z = lambda n, dt: (self.heap.alloc(n, dt) if self.heap is not None
                               else torch.zeros(n, dtype=dt, device=self.device))
            self._q_codes = z(self.layout.val_elems, torch.uint8)
            self._q_table = z(np_ * (nb + 2), torch.float32).view(np_, nb + 2)
            self._q_scratch = torch.zeros(np_ * (16 + 4 * nb), dtype=torch.float32, device=self.device)
        return self._q_codes, self._q_table, self._q_scratch

    def _quantize_own(self, on_rank0: bool) -> None:
        """Encode the node's payload values as 8-bit codes with per-tensor tables (``tplr_quantize_values``),
        add the quantisation error back into the error feedback and leave the dequantised values in the
        payload, which is what the reference's miner does by decompressing with its quantisation parameters
        before it forms the residual (src/tplr/neurons.py:157-171).

        Sharded: every rank has written its chunks into rank 0's payload (``on_rank0``); rank 0 encodes the
        whole payload (the statistics are per tensor), then every rank corrects its own chunks, reading the
        codes and tables from rank 0's memory."""
        cfg, st = self.cfg, self.store
        native.require(cfg.quant_bins <= 256, "at most 256 quantisation bins")
        native.require(self.world_size == 1 or (on_rank0 and self.heap is not None),
                       "a sharded engine quantises the payload assembled in rank 0's symmetric buffers")
        codes, table, scratch = self._quant_buffers()
        L = native.lib()
        if self.world_size > 1:
            self._barrier()                        # every rank's chunks have landed on rank 0
            self._mark("compress.barrier_payload_assembled")
        if self.rank == 0:
            desc_full, n_full = self._desc_full
            native.check(L.tplr_quantize_values(desc_full.data_ptr(), n_full, self.own_val.data_ptr(), codes.data_ptr(),
                                                table.data_ptr(), scratch.data_ptr(), self.layout.n_params,
                                                cfg.quant_bins, float(cfg.quant_range), native.stream_ptr()),
                         "quantize_values")
        self._mark("compress.quantize_on_rank0")
        if self.world_size > 1:
            self._barrier()                        # codes and tables are complete
            self._mark("compress.barrier_codes_ready")
        at0 = (lambda t: self.heap.peer_ptr(t, 0)) if self.world_size > 1 else (lambda t: t.data_ptr())
        bias = 0
        for square in (True, False):
            desc, n_desc, n_chunks = self._desc[square]
            if n_chunks == 0:
                continue
            native.check(L.tplr_requant_residual(desc.data_ptr(), n_desc, n_chunks, self.basis.data_ptr(),
                                                 self.ef.data_ptr() - bias, at0(self.own_idx), at0(self.own_val),
                                                 at0(codes), at0(table), cfg.quant_bins, int(cfg.use_dct),
                                                 int(not square), native.stream_ptr()), "requant_residual")
        self._mark("compress.requant_residual")

    def merge_own_payload(self) -> None:
        """Sharded engine without a symmetric heap: every rank has written only its own chunks of the node's
        payload (the rest of the buffers is zero), so the sum over ranks is the whole payload on every rank.
        With a heap the ranks write straight into rank 0's buffers and nothing is left to merge."""
        if self.world_size == 1 or self.heap is not None or getattr(self, "_own_merged", False):
            return
        self._own_merged = True                       # once per compress(): a second sum would scale the values
        dist.all_reduce(self.own_val, group=self.group)
        idx32 = self.own_idx.to(torch.int32)          # the byte ranges are disjoint: a sum is a merge
        dist.all_reduce(idx32, group=self.group)
        self.own_idx.copy_(idx32.to(torch.uint8))

    def _compress_torch(self, null_round: bool) -> None:
        """CPU oracle path: the same arithmetic through :mod:`templar_b200.compress`, tensor by tensor.

        Unsharded with ``quantize``: the reference's literal flow (compress with a quantising compressor,
        residual against the dequantised values).  Sharded with ``quantize``: exact values first, merge of the
        payload over the ranks, the per-tensor statistics on the whole tensors (the same on every rank), then
        each rank adds decode(exact - dequantised) of its own chunks back into its error feedback."""
        cfg, st, L = self.cfg, self.store, self.layout
        sharded = self.world_size > 1
        tr = C.ChunkingTransformer(None, cfg.target_chunk)
        comp = C.TopKCompressor(use_quantization=cfg.quantize and not sharded, quantization_bins=cfg.quant_bins,
                                quantization_range=int(cfg.quant_range))
        if cfg.quantize:
            codes, table, _ = self._quant_buffers()
        if sharded:
            self.own_idx.zero_()
            self.own_val.zero_()
        entries = L.shard_entries(self.rank) if (sharded or self.fsdp) else [(s, 0, s.chunk_rows, s.offset) for s in L.specs]
        parts = []
        for s, r0, nrows, a in entries:
            b = a + nrows * s.h * s.cols
            shape = (nrows * s.h, s.cols) if len(s.shape) >= 2 else (s.cols,)
            tr.register_shape(shape)
            e = self.ef[a:b].view(shape)
            if null_round:
                e.zero_()
            else:
                e.mul_(cfg.momentum_decay).add_((self.theta0[a:b] - st.master_shard[a:b]).view(shape))
            enc = tr.encode(e, use_dct=cfg.use_dct)
            out = comp.compress(enc, cfg.topk)
            idx, val, xshape, totalk = out[:4]
            qp = out[4] if len(out) == 5 else None
            dec = tr.decode(comp.decompress(e, idx, val, xshape, totalk, qp), use_dct=cfg.use_dct)
            e.sub_(dec)
            k = s.topk(cfg.topk)
            c0 = r0 * s.chunks_x
            io = L.idx_off[s.name] + c0 * (k // 2) * 3
            vo = L.val_off[s.name] + c0 * k
            self.own_idx[io: io + idx.numel()].copy_(idx)
            parts.append((s, e, shape, idx, val, xshape, totalk, vo))
            if qp is not None:                      # the payload keeps what a receiver decodes
                codes[vo: vo + val.numel()].copy_(val.reshape(-1))
                shift, scale, _, lookup, _ = qp
                table[s.index, : cfg.quant_bins] = lookup
                table[s.index, cfg.quant_bins], table[s.index, cfg.quant_bins + 1] = float(shift), float(scale)
                val = comp._dequantize_values(val, qp)
            self.own_val[vo: vo + val.numel()].copy_(val.reshape(-1))
        if not (cfg.quantize and sharded):
            return
        self.merge_own_payload()
        qcomp = C.TopKCompressor(use_quantization=True, quantization_bins=cfg.quant_bins,
                                 quantization_range=int(cfg.quant_range))
        for s in L.specs:                           # whole tensors: identical statistics on every rank
            _, v = L.payload_views(self.own_idx, self.own_val, s.name)
            _, c = L.payload_views(self.own_idx, codes, s.name)
            q, (shift, scale, _, lookup, _) = qcomp._quantize_values(v.float())
            c.copy_(q.reshape(c.shape))
            table[s.index, : cfg.quant_bins] = lookup
            table[s.index, cfg.quant_bins], table[s.index, cfg.quant_bins + 1] = float(shift), float(scale)
            v.copy_((lookup[q.long()] + shift).reshape(v.shape))
        plain = C.TopKCompressor(use_quantization=False)
        for s, e, shape, idx, val, xshape, totalk, vo in parts:
            tr.register_shape(shape)
            diff = val - self.own_val[vo: vo + val.numel()].view(val.shape)
            e.add_(tr.decode(plain.decompress(e, idx, diff, xshape, totalk), use_dct=cfg.use_dct))

    def own_payload(self, quantize: bool | None = None, n_bins: int | None = None,
                    range_in_sigmas: float | None = None) -> dict:
        """Reference-format gradient dict (``<name>idxs`` / ``<name>vals`` / ``<name>quant_params``)
        as views of the flat payload buffers, in named_parameters() order.

        ``quantize`` (default: the engine's ``cfg.quantize``): values as uint8 codes with the reference's
        per-tensor ``(shift, scale, offset, lookup, dtype)`` tuples (src/tplr/compress.py:585-636).  An engine
        configured with ``quantize`` returns the codes that :meth:`compress` computed; otherwise the payload is
        encoded here, on CUDA (unsharded) by one group of kernels (``tplr_quantize_values``), else tensor by
        tensor through :class:`templar_b200.compress.TopKCompressor`."""
        cfg = self.cfg
        quantize = cfg.quantize if quantize is None else quantize
        n_bins = cfg.quant_bins if n_bins is None else n_bins
        range_in_sigmas = cfg.quant_range if range_in_sigmas is None else range_in_sigmas
        specs = sorted(self.layout.specs, key=lambda s: s.index)
        out = {}
        if not quantize:
            for s in specs:
                idx, val = self.layout.payload_views(self.own_idx, self.own_val, s.name)
                out[s.name + "idxs"], out[s.name + "vals"], out[s.name + "quant_params"] = idx, val, None
            return out
        computed = cfg.quantize and n_bins == cfg.quant_bins and getattr(self, "_q_codes", None) is not None
        if computed or (self.cuda and self.world_size == 1 and n_bins <= 256):
            if not computed:
                codes, table, scratch = self._quant_buffers(n_bins)
                desc_full, n_full = self._desc_full
                native.check(native.lib().tplr_quantize_values(desc_full.data_ptr(), n_full, self.own_val.data_ptr(),
                                                               codes.data_ptr(), table.data_ptr(), scratch.data_ptr(),
                                                               self.layout.n_params, n_bins, float(range_in_sigmas),
                                                               native.stream_ptr()), "quantize_values")
            tab = self._q_table.cpu()                       # one small D2H copy for all tensors
            for s in specs:
                idx, codes = self.layout.payload_views(self.own_idx, self._q_codes, s.name)
                row = tab[s.index]
                out[s.name + "idxs"], out[s.name + "vals"] = idx, codes
                out[s.name + "quant_params"] = (row[n_bins].clone(), float(row[n_bins + 1]), n_bins // 2,
                                                row[:n_bins].clone(), torch.float32)
            return out
        comp = C.TopKCompressor(use_quantization=True, quantization_bins=n_bins, quantization_range=int(range_in_sigmas))
        for s in specs:
            idx, val = self.layout.payload_views(self.own_idx, self.own_val, s.name)
            q, qp = comp._quantize_values(val.float())
            out[s.name + "idxs"], out[s.name + "vals"], out[s.name + "quant_params"] = idx, q, qp
        return out

    # ------------------------------------------------------------------------------------ #
    # gather side
    # ------------------------------------------------------------------------------------ #
    @torch.no_grad()
    def load_peer_payload(self, slot: int, payload, non_blocking: bool = True) -> None:
        """``payload``: (idx_flat uint8, val_flat) or (idx_flat uint8, codes uint8, table) in this layout, or a
        reference-format dict."""
        if isinstance(payload, dict):
            for s in self.layout.specs:
                idx, val = self.layout.payload_views(self.peer_idx[slot], self.peer_val[slot], s.name)
                idx.copy_(payload[s.name + "idxs"].reshape(-1), non_blocking=non_blocking)
                val.copy_(self._payload_values(payload, s.name, val.device).reshape(val.shape),
                          non_blocking=non_blocking)
            return
        if len(payload) == 3:                     # quantised flat form: indices, 8-bit codes, per-tensor tables
            idx_flat, codes, table = payload
            self.peer_idx[slot][: idx_flat.numel()].copy_(idx_flat, non_blocking=non_blocking)
            self._decode_flat(codes, table, self.peer_val[slot], non_blocking)
            return
        idx_flat, val_flat = payload
        self.peer_idx[slot][: idx_flat.numel()].copy_(idx_flat, non_blocking=non_blocking)
        self.peer_val[slot][: val_flat.numel()].copy_(val_flat, non_blocking=non_blocking)

    def load_peer_payloads_async(self, items) -> None:
        """Stage several peers' payloads (``[(slot, payload), ...]``, payloads as for :meth:`load_peer_payload`, host
        tensors pinned) on a side stream: the copy engines and the small decode kernel run beside whatever the compute
        stream is doing (this node's own compress, or the end of its backward pass).  The slots were last read by the
        previous outer step, which the side stream waits for; everything that reads the slots
        (:meth:`compute_peer_norms`, :meth:`outer_step`, :meth:`index_overlap`, :meth:`apply_single_peer`, the barrier
        that publishes them to the other ranks) first joins the side stream (:meth:`join_payloads`)."""
        if not self.cuda:
            for slot, payload in items:
                self.load_peer_payload(slot, payload)
            return
        if self._h2d_stream is None:
            self._h2d_stream = torch.cuda.Stream(self.device)
        side = self._h2d_stream
        done = getattr(self, "_slots_read", None)
        if done is not None:
            side.wait_event(done)
        with torch.cuda.stream(side):
            for slot, payload in items:
                self.load_peer_payload(slot, payload)
            ev = torch.cuda.Event()
            ev.record(side)
        self._h2d_pending = ev

    def join_payloads(self) -> None:
        """The compute stream waits for the payloads staged by :meth:`load_peer_payloads_async` (no host wait)."""
        if self._h2d_pending is not None:
            torch.cuda.current_stream(self.device).wait_event(self._h2d_pending)
            self._h2d_pending = None

    def _decode_flat(self, codes: torch.Tensor, table: torch.Tensor, out: torch.Tensor, non_blocking: bool) -> None:
        """out <- lookup[code] + shift per tensor.  ``codes`` [val_elems] uint8 and ``table`` [n_params, bins + 2]
        (lookup | shift | scale) may live on the host: they cross the link as they are (one byte per value) and
        are decoded on the device by one kernel."""
        n_bins = table.shape[1] - 2
        if not self.cuda or out.dtype != torch.float32:
            lut = table.to(out.device, torch.float32)
            codes = codes.to(out.device)
            for s in self.layout.specs:
                _, c = self.layout.payload_views(self.own_idx, codes, s.name)
                _, o = self.layout.payload_views(self.own_idx, out, s.name)
                o.copy_((lut[s.index, :n_bins][c.long().clamp(max=n_bins - 1)] + lut[s.index, n_bins]).reshape(o.shape))
            return
        if getattr(self, "_stage_codes", None) is None or self._stage_table.shape != table.shape:
            self._stage_codes = torch.empty(self.layout.val_elems, dtype=torch.uint8, device=self.device)
            self._stage_table = torch.empty(table.shape, dtype=torch.float32, device=self.device)
        self._stage_codes[: codes.numel()].copy_(codes, non_blocking=non_blocking)
        self._stage_table.copy_(table, non_blocking=non_blocking)
        desc_full, n_full = self._desc_full
        native.check(native.lib().tplr_dequantize_values(desc_full.data_ptr(), n_full, self._stage_codes.data_ptr(),
                                                         self._stage_table.data_ptr(), out.data_ptr(), n_bins,
                                                         native.stream_ptr()), "dequantize_values")

    @torch.no_grad()
    def encode_values(self, val_flat: torch.Tensor, n_bins: int | None = None,
                      range_in_sigmas: float | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """8-bit codes and per-tensor tables ([n_params, bins + 2]: lookup | shift | scale) of any value buffer
        in this layout (CUDA, full layout); the inverse is the 3-tuple form of :meth:`load_peer_payload`."""
        native.require(self.cuda and val_flat.is_cuda and val_flat.dtype == torch.float32, "encode_values runs on CUDA fp32")
        n_bins = self.cfg.quant_bins if n_bins is None else n_bins
        range_in_sigmas = self.cfg.quant_range if range_in_sigmas is None else range_in_sigmas
        np_ = self.layout.n_params
        codes = torch.empty(self.layout.val_elems, dtype=torch.uint8, device=self.device)
        table = torch.zeros(np_, n_bins + 2, dtype=torch.float32, device=self.device)
        scratch = torch.zeros(np_ * (16 + 4 * n_bins), dtype=torch.float32, device=self.device)
        desc_full, n_full = self._desc_full
        native.check(native.lib().tplr_quantize_values(desc_full.data_ptr(), n_full, val_flat.data_ptr(), codes.data_ptr(),
                                                       table.data_ptr(), scratch.data_ptr(), np_, n_bins,
                                                       float(range_in_sigmas), native.stream_ptr()), "quantize_values")
        return codes, table

    @staticmethod
    def _payload_values(payload: dict, name: str, device=None) -> torch.Tensor:
        """The values of one tensor of a reference-format payload; uint8 codes are decoded with the payload's
        ``<name>quant_params`` = (shift, scale, offset, lookup, dtype), as the reference does before it
        decompresses (src/tplr/compress.py:624-644).  With ``device`` the codes are moved there first, so a
        quantised payload crosses the host link as one byte per value and is decoded on the device."""
        vals = payload[name + "vals"]
        if vals.dtype != torch.uint8:
            return vals
        qp = payload.get(name + "quant_params")
        if qp is None:
            raise ValueError(f"{name}vals holds 8-bit codes but the payload has no {name}quant_params")
        shift, _, _, lookup, _ = qp
        lookup = torch.as_tensor(lookup)
        # the codes are uint8, so a table of 256 entries can never be indexed out of range; a shorter one is
        # padded with its last entry (gather's acceptance test has already rejected codes beyond the table)
        if lookup.dim() != 1 or lookup.numel() < 1:
            raise ValueError(f"{name}quant_params: the lookup table must be a non-empty 1-D tensor")
        if device is not None:
            vals = vals.to(device, non_blocking=True)
        lookup = lookup.to(vals.device, torch.float32)
        if lookup.numel() < 256:
            lookup = torch.cat((lookup, lookup[-1:].expand(256 - lookup.numel())))
        shift = torch.as_tensor(shift).to(vals.device, torch.float32)
        return lookup[vals.long()] + shift

    def _peer_list(self, n_peers, include_own: bool, peers=None) -> list[int]:
        """Peer ids taking part: ``peers`` when given, else 0..n_peers-1; id -1 denotes this node's own payload."""
        ids = list(peers) if peers is not None else list(range(n_peers))
        if include_own and peers is None and ids:
            ids[0] = -1
        return ids

    def _payload_buffers(self, j):
        """Host-addressable (index, value) buffers of peer ``j`` (CPU paths)."""
        if isinstance(j, tuple):
            return self.rank_payloads[int(j[1])]
        if j < 0:
            return self.own_idx, self.own_val
        return self.peer_idx[self.slot_of(j)[1]], self.peer_val[self.slot_of(j)[1]]

    def _peer_ptrs(self, ids: list[int]):
        """Pointers of the payloads: -1 = this node's own payload (held by rank 0), ``("rank", r)`` = the own payload
        of the co-located node that runs as rank r (see parallel/peer_group.py), the others live round-robin in
        the ranks' slots (peer j on rank j % world, slot j // world)."""
        idx_ptrs, val_ptrs = [], []
        for j in ids:
            if isinstance(j, tuple):                 # ("rank", r): the own payload of the node that runs as rank r
                r = int(j[1])
                if self.heap is None or self.cuda is False:
                    ib, vb = self.rank_payloads[r]
                    idx_ptrs.append(ib.data_ptr())
                    val_ptrs.append(vb.data_ptr())
                else:
                    idx_ptrs.append(self.heap.peer_ptr(self.own_idx, r))
                    val_ptrs.append(self.heap.peer_ptr(self.own_val, r))
                continue
            if j < 0:
                owner = 0
                ib, vb = self.own_idx, self.own_val
            else:
                owner, slot = self.slot_of(j)
                ib, vb = self.peer_idx[slot], self.peer_val[slot]
            if self.heap is not None and self.world_size > 1:
                idx_ptrs.append(self.heap.peer_ptr(ib, owner))
                val_ptrs.append(self.heap.peer_ptr(vb, owner))
            else:
                idx_ptrs.append(ib.data_ptr())
                val_ptrs.append(vb.data_ptr())
        return idx_ptrs, val_ptrs

    @torch.no_grad()
    def compute_peer_norms(self, n_peers: int | None = None, *, include_own: bool = False, peers=None) -> torch.Tensor:
        """Per-(peer, tensor) value norms, their per-tensor lower median, clip factors and skip flags
        (all left on the device in ``peer_norms`` / ``median`` / ``clip`` / ``skip``).  Returns the medians."""
        self.join_payloads()
        ids = self._peer_list(n_peers, include_own, peers)
        np_ = self.layout.n_params
        if not self.cuda:
            norms = torch.zeros(len(ids), np_)
            for a, j in enumerate(ids):
                ib, vb = self._payload_buffers(j)
                for s in self.layout.specs:
                    norms[a, s.index] = self.layout.payload_views(ib, vb, s.name)[1].float().norm()
            med = norms.median(dim=0).values
            self.peer_norms[: len(ids) * np_].copy_(norms.reshape(-1))
            self.median.copy_(med)
            self.clip[: len(ids) * np_].copy_(torch.clamp(med / (norms + 1e-8), max=1.0).reshape(-1))
            self.skip.copy_((~torch.isfinite(norms).all(dim=0)).to(torch.int32))
            return self.median
        L = native.lib()
        _, val_ptrs = self._peer_ptrs(ids)
        vdt = {torch.float32: 0, torch.bfloat16: 1}[self.cfg.val_dtype]
        stream = native.stream_ptr()
        desc_full, n_full = self._desc_full
        native.check(L.tplr_peer_sumsq(desc_full.data_ptr(), n_full, np_, len(ids), native.ptr_array(val_ptrs), vdt,
                                       None, 0, self.sumsq_partial.data_ptr(), stream), "peer_sumsq")
        native.check(L.tplr_clip_factors(self.sumsq_partial.data_ptr(), np_, len(ids), self.peer_norms.data_ptr(),
                                         self.clip.data_ptr(), self.median.data_ptr(), self.skip.data_ptr(),
                                         self.status.data_ptr(), stream), "clip_factors")
        return self.median

    @torch.no_grad()
    def outer_step(self, n_peers: int | None = None, *, lr: float | None = None, include_own: bool = True,
                   clip_norm: bool = True, base: str = "theta0", peers=None, clip_override: torch.Tensor | None = None) -> None:
        """Aggregate the payloads of ``peers`` (default: peers 0..n_peers-1, peer 0 being this node's own
        payload when ``include_own``) and apply the outer update to the owned shard.

        ``base='theta0'`` applies the update to the window-start snapshot (the miner's flow:
        restore, then outer step); ``base='theta'`` applies it to the current master.
        ``clip_override`` ([len(peers), n_params] scale factors) replaces the median-norm clip.
        """
        cfg, st = self.cfg, self.store
        lr = cfg.outer_lr if lr is None else lr
        self.join_payloads()
        ids = self._peer_list(n_peers, include_own, peers)
        n_peers = len(ids)
        if clip_override is not None:
            self.clip[: clip_override.numel()].copy_(clip_override.reshape(-1).to(self.clip.dtype))
            self.skip.zero_()
        elif clip_norm:
            self.compute_peer_norms(peers=ids)
        self._mark("outer.peer_norms")
        use_clip = clip_norm or clip_override is not None
        if not self.cuda:
            return self._outer_step_torch(ids, lr, use_clip, base)
        L = native.lib()
        idx_ptrs, val_ptrs = self._peer_ptrs(ids)
        vdt = {torch.float32: 0, torch.bfloat16: 1}[cfg.val_dtype]
        stream = native.stream_ptr()
        np_ = self.layout.n_params
        bias = 0
        base_buf = self.theta0 if base == "theta0" else st.master_shard
        shadow = None                        # the compute-dtype copy of the shard, addressed like the shard arrays
        if self.fsdp:
            shadow = st.compute_shard.data_ptr()
        elif st.compute is not st.master_shard:
            shadow = st.compute.data_ptr() + st.lo * st.compute.element_size()
        mode = {"sgd": 0, "sign": 1}[cfg.outer_update]
        for square in (True, False):
            desc, n_desc, n_chunks = self._desc[square]
            if n_chunks == 0:
                continue
            if square and cfg.use_dct and self._dct_on_tensor_cores:
                # every chunk of this table is 64 x 64: inverse DCT as tcgen05 GEMMs against the basis
                native.check(L.tplr_aggregate_apply_tc(desc.data_ptr(), n_desc, n_chunks, self.basis.data_ptr(), n_peers,
                                                       native.ptr_array(idx_ptrs), native.ptr_array(val_ptrs), vdt, None, 0,
                                                       np_, self.clip.data_ptr() if use_clip else None,
                                                       self.skip.data_ptr() if use_clip else None,
                                                       base_buf.data_ptr() - bias, st.master_shard.data_ptr() - bias,
                                                       shadow, None, lr, cfg.outer_weight_decay, mode,
                                                       self.status.data_ptr(), stream), "aggregate_apply_tc")
                continue
            native.check(L.tplr_aggregate_apply(desc.data_ptr(), n_desc, n_chunks, self.basis.data_ptr(), n_peers,
                                                native.ptr_array(idx_ptrs), native.ptr_array(val_ptrs), vdt, None, 0, np_,
                                                self.clip.data_ptr() if use_clip else None,
                                                self.skip.data_ptr() if use_clip else None,
                                                base_buf.data_ptr() - bias, st.master_shard.data_ptr() - bias, shadow, None,
                                                lr, cfg.outer_weight_decay, int(cfg.use_dct), mode, int(not square),
                                                self.status.data_ptr(), stream), "aggregate_apply")
        self._mark("outer.aggregate_apply")
        if self.fsdp:
            st.gather.invalidate()
            self._barrier()
            self._mark("outer.barrier")
            self._refresh_samples()
        elif self.world_size > 1:
            self._barrier()
            self._mark("outer.barrier")
            self._allgather_compute_native()
            self._mark("outer.weight_allgather")
        # the peer slots may be refilled from here on (every rank's aggregate kernel is past the barrier above)
        self._slots_read = torch.cuda.Event()
        self._slots_read.record()

    def _allgather_compute_native(self) -> None:
        """Push the owned range of the compute buffer to every other rank (plain stores over NVLink)."""
        st = self.store
        esz = st.compute.element_size()
        n = st.hi - st.lo
        src = st.compute.data_ptr() + st.lo * esz
        dsts = [self.heap.peer_ptr(st.compute, r) + st.lo * esz for r in range(self.world_size) if r != self.rank]
        native.check(native.lib().tplr_push_copy(src, native.ptr_array(dsts), len(dsts), n * esz, native.stream_ptr()),
                     "push_copy")
        self._barrier()

    def _outer_step_torch(self, ids, lr, use_clip, base) -> None:
        """CPU path: same result through :mod:`templar_b200.compress`, with the clip factors already in ``self.clip``."""
        cfg, st, L = self.cfg, self.store, self.layout
        tr = C.ChunkingTransformer(None, cfg.target_chunk)
        comp = C.TopKCompressor(use_quantization=False)
        bufs = [self._payload_buffers(j) for j in ids]
        base_buf = self.theta0 if base == "theta0" else st.master_shard
        clip = self.clip[: len(ids) * L.n_params].view(len(ids), L.n_params)
        mine: dict[str, list] = {}
        for s, a, b, la in L.segments(self.rank):
            mine.setdefault(s.name, []).append((a, b, la))
        for s in L.specs:
            if s.name not in mine:
                continue
            tr.register_shape(s.shape)
            idxs, vals = zip(*(L.payload_views(ib, vb, s.name) for ib, vb in bufs))
            vals = [v.float() * (clip[a, s.index] if use_clip else 1.0) for a, v in enumerate(vals)]
            ref = torch.empty(s.shape, dtype=torch.float32, device=self.device)
            if use_clip and bool(self.skip[s.index]):
                vals = [v * float("nan") for v in vals]
            full = tr.decode(comp.batch_decompress(ref, list(idxs), list(vals), L.xshape(s.name), s.totalk,
                                                   clip_norm=False), use_dct=cfg.use_dct).reshape(-1)
            finite = bool(torch.isfinite(full).all())       # a tensor is applied whole or not at all
            for a, b, la in mine[s.name]:
                g = full[a - s.offset: b - s.offset]
                if not finite:
                    st.master_shard[la: la + (b - a)].copy_(base_buf[la: la + (b - a)])
                    continue
                step = torch.sign(g) if cfg.outer_update == "sign" else g
                st.master_shard[la: la + (b - a)].copy_(
                    base_buf[la: la + (b - a)] * (1 - lr * cfg.outer_weight_decay) - lr * step)
        self._publish_compute()

    # ------------------------------------------------------------------------------------ #
    # validator: index overlap, single-peer apply and restore
    # ------------------------------------------------------------------------------------ #
    @torch.no_grad()
    def index_overlap(self, n_peers: int) -> torch.Tensor:
        """[n_peers, n_peers] matrix whose (i, j), i < j, entry is the fraction of (chunk, index) selections that
        the staged peers i and j share over the whole payload (one kernel over the packed indices; CUDA).
        Equals the size-weighted mean over tensors of the per-chunk overlap fraction.

        A sharded engine counts over the chunks of its own shard, reading the packed indices from the slots of the
        ranks that hold them, and the counts are summed over the ranks: a collective, so every rank calls it."""
        native.require(self.cuda, "index_overlap needs the CUDA engine")
        self.join_payloads()
        ids = list(range(n_peers))
        idx_ptrs, _ = self._peer_ptrs(ids)
        counts = torch.zeros(n_peers * n_peers, dtype=torch.int64, device=self.device)
        if self.world_size == 1:
            desc, n_desc = self._desc_full
            n_chunks = sum(s.n_chunks for s in self.layout.specs)
        else:
            if getattr(self, "_desc_rank_all", None) is None:
                arr = self.layout.descriptors(self.rank, square=None)
                self._desc_rank_all = (torch.from_numpy(arr.view(np.uint8).reshape(-1).copy()).to(self.device), len(arr),
                                       int(arr["n_chunks"].sum()) if len(arr) else 0)
            desc, n_desc, n_chunks = self._desc_rank_all
        if n_chunks:
            native.check(native.lib().tplr_index_overlap(desc.data_ptr(), n_desc, n_chunks, n_peers,
                                                         native.ptr_array(idx_ptrs), counts.data_ptr(),
                                                         native.stream_ptr()), "index_overlap")
        if self.world_size > 1:
            dist.all_reduce(counts, group=self.group)
        total = sum(s.n_chunks * s.topk(self.layout.topk) for s in self.layout.specs)
        return counts.view(n_peers, n_peers).double() / float(total)

    @torch.no_grad()
    def apply_single_peer(self, peer: int, lr: float, median: torch.Tensor | None = None) -> None:
        """theta <- theta0 - lr * decode(peer's payload), the peer's values clipped per tensor to
        ``min(1, median / (norm + 1e-8))`` where ``median`` is the per-tensor median norm over the
        gathered peers (validator scoring; reference neurons/validator.py:3563-3770)."""
        np_ = self.layout.n_params
        clip = None
        if median is not None:
            med = median.clone()
            self.compute_peer_norms(peers=[peer])
            clip = torch.clamp(med / (self.peer_norms[:np_] + 1e-8), max=1.0)
            clip = torch.where(torch.isfinite(clip), clip, torch.zeros_like(clip))
        self.outer_step(peers=[peer], lr=lr, include_own=False, clip_norm=False, base="theta0",
                        clip_override=clip.view(1, np_) if clip is not None else None)

    @torch.no_grad()
    def restore(self) -> None:
        """master <- theta0 and compute copy refreshed (undo of an evaluation-time apply)."""
        st = self.store
        st.master_shard.copy_(self.theta0)
        if self.fsdp:
            if self.cuda:
                native.check(native.lib().tplr_cast_bf16(st.master_shard.data_ptr(), st.compute_shard.data_ptr(),
                                                         st.n_shard, native.stream_ptr()), "cast_bf16")
                st.gather.invalidate()
            else:
                st.refresh_compute_from_master()
            self._barrier()
            self._refresh_samples()
            return
        if self.cuda and st.compute is not st.master_shard:
            native.check(native.lib().tplr_cast_bf16(st.master_shard.data_ptr(),
                                                     st.compute.data_ptr() + st.lo * st.compute.element_size(),
                                                     st.hi - st.lo, native.stream_ptr()), "cast_bf16")
            if self.world_size > 1:
                self._barrier()
                self._allgather_compute_native()
        else:
            self._publish_compute()

    # ------------------------------------------------------------------------------------ #
    # payload distribution and state dicts
    # ------------------------------------------------------------------------------------ #
    @torch.no_grad()
    def pack_payload(self, payload: dict, device=None):
        """Reference-format dict (one peer) -> (idx_flat uint8, val_flat) in this layout."""
        L = self.layout
        device = device or "cpu"
        idx = torch.zeros(L.idx_bytes, dtype=torch.uint8, device=device)
        val = torch.zeros(L.val_elems, dtype=self.cfg.val_dtype, device=device)
        for s in L.specs:
            i, v = L.payload_views(idx, val, s.name)
            i.copy_(payload[s.name + "idxs"].reshape(-1))
            v.copy_(self._payload_values(payload, s.name, v.device).reshape(v.shape))
        return idx, val

    @torch.no_grad()
    def distribute_peer_payloads(self, state_dict: dict | None, n_peers: int) -> None:
        """Rank 0 holds the gathered per-key lists; peer j's payload ends up in ``slot_of(j)``.
        With a symmetric heap rank 0 stores straight into the owner's slot over NVLink; without
        one the flat buffers are broadcast and every rank keeps all peers."""
        L = self.layout
        for j in range(n_peers):
            owner, slot = self.slot_of(j)
            if self.heap is not None:
                if self.rank == 0:
                    one = peer_slice(state_dict, j)
                    idx, val = self.pack_payload(one, device=self.device)
                    for src, dst in ((idx, self.peer_idx[slot]), (val, self.peer_val[slot])):
                        native.check(native.lib().tplr_push_copy(
                            src.data_ptr(), native.ptr_array([self.heap.peer_ptr(dst, owner)]), 1,
                            -(-src.numel() * src.element_size() // 16) * 16, native.stream_ptr()), "push_copy")
            else:
                if self.rank == 0:
                    one = peer_slice(state_dict, j)
                    idx, val = self.pack_payload(one, device=self.device)
                    self.peer_idx[slot].copy_(idx)
                    self.peer_val[slot].copy_(val)
                if self.world_size > 1:
                    dist.broadcast(self.peer_idx[slot], src=self._global(0), group=self.group)
                    dist.broadcast(self.peer_val[slot], src=self._global(0), group=self.group)
        self._barrier()

    @torch.no_grad()
    def stage_single_peer(self, payload: dict | None, peer: int) -> None:
        """One peer's reference-format payload (held by rank 0; ``None`` elsewhere) into the slot of peer index
        ``peer``: the validator stages the upload of the uid it is about to score this way.  With a symmetric heap
        rank 0 stores into the owner's slot over NVLink, otherwise the flat buffers are broadcast."""
        owner, slot = self.slot_of(peer)
        if self.world_size == 1:
            self.load_peer_payload(slot, payload)
            return
        if self.heap is not None:
            if self.rank == 0:
                idx, val = self.pack_payload(payload, device=self.device)
                for src, dst in ((idx, self.peer_idx[slot]), (val, self.peer_val[slot])):
                    native.check(native.lib().tplr_push_copy(
                        src.data_ptr(), native.ptr_array([self.heap.peer_ptr(dst, owner)]), 1,
                        -(-src.numel() * src.element_size() // 16) * 16, native.stream_ptr()), "push_copy")
        else:
            if self.rank == 0:
                idx, val = self.pack_payload(payload, device=self.device)
                self.peer_idx[slot].copy_(idx)
                self.peer_val[slot].copy_(val)
            dist.broadcast(self.peer_idx[slot], src=self._global(0), group=self.group)
            dist.broadcast(self.peer_val[slot], src=self._global(0), group=self.group)
        self._barrier()

    @torch.no_grad()
    def full_master(self) -> torch.Tensor:
        """The whole fp32 master vector on every rank (shards exchanged by broadcast)."""
        st = self.store
        if self.world_size == 1 and not self.fsdp:
            return st.master_shard
        full = torch.zeros(self.layout.total, dtype=torch.float32, device=self.device)
        for p in self.layout.pieces(self.rank):
            full[p.g_lo:p.g_hi].copy_(st.master_shard[p.local: p.local + (p.g_hi - p.g_lo)])
        for r in range(self.world_size if self.world_size > 1 else 0):
            for p in self.layout.pieces(r):
                dist.broadcast(full[p.g_lo:p.g_hi], src=dist.get_global_rank(self.group, r) if self.group is not None else r,
                               group=self.group)
        return full

    @torch.no_grad()
    def full_state_dict(self) -> dict:
        """fp32 tensors keyed like ``model.state_dict()`` (parameters from the master weights, buffers as is)."""
        full = self.full_master()
        out = {}
        for k, v in self.model.state_dict().items():
            s = self.layout.by_name.get(k)
            out[k] = full[s.offset: s.offset + s.numel].view(s.shape) if s is not None else v
        return out

    @torch.no_grad()
    def load_full_state_dict(self, state: dict) -> None:
        st = self.store
        for s, a, b, la in self.layout.segments(self.rank):
            if s.name not in state:
                continue
            src = state[s.name].reshape(-1)[a - s.offset: b - s.offset].to(device=self.device, dtype=torch.float32)
            st.master_shard[la: la + (b - a)].copy_(src)
            if self.fsdp:
                st.compute_shard[la: la + (b - a)].copy_(src.to(st.compute_dtype))
        if self.fsdp:
            st.gather.invalidate()
            self._barrier()
            self._refresh_samples()
        for s in self.layout.specs:
            if s.name not in state or self.fsdp:
                continue
            if st.compute is not st.master_shard:
                src = state[s.name].reshape(-1).to(device=self.device, dtype=torch.float32)
                st.compute[s.offset: s.offset + s.numel].copy_(src.to(st.compute.dtype))
        for k, v in state.items():
            if k not in self.layout.by_name:
                buf = dict(self.model.named_buffers()).get(k)
                if buf is not None and torch.is_tensor(v):
                    buf.copy_(v.to(buf.device))

    # -- a few elements of every tensor, for the nodes' debug / sync bookkeeping ------------------------ #
    SAMPLE_RANGES = ((0, 2), (10, 12))

    @torch.no_grad()
    def _refresh_samples(self) -> None:
        """With sharded parameters no rank can read a tensor's elements from the module tree (the parameters are
        views of gather buffers).  The elements that the nodes publish and compare (``flatten()[0:2]`` and
        ``[10:12]`` of every tensor, reference neurons/miner.py:822-832, neurons/validator.py:2589-2598) are
        therefore collected from the owners' master shards whenever the weights change at a window boundary:
        one small all-reduce, called by every rank, so that the master-only readers need no collective."""
        if not self.fsdp:
            return
        L, st = self.layout, self.store
        width = sum(b - a for a, b in self.SAMPLE_RANGES)
        if getattr(self, "_sample_index", None) is None:          # (positions in the shard, positions in the table)
            src, dst, col = [], [], 0
            for lo, hi in self.SAMPLE_RANGES:
                for sp, a, b, la in L.segments(self.rank):
                    x, y = max(sp.offset + lo, a), min(sp.offset + min(hi, sp.numel), b)
                    for e in range(x, y):
                        src.append(la + (e - a))
                        dst.append(sp.index * width + col + (e - sp.offset - lo))
                col += hi - lo
            self._sample_index = (torch.tensor(src, dtype=torch.long, device=self.device),
                                  torch.tensor(dst, dtype=torch.long, device=self.device))
        src, dst = self._sample_index
        buf = torch.zeros(L.n_params * width, dtype=torch.float32, device=self.device)
        buf[dst] = st.master_shard[src]
        if self.world_size > 1:
            dist.all_reduce(buf, group=self.group)
        self._samples = buf.view(L.n_params, width).cpu()

    def param_samples(self, lo: int, hi: int) -> dict[str, torch.Tensor]:
        """``{name: flatten()[lo:hi]}`` of every tensor with at least ``hi`` elements (fp32, host), for one of
        :attr:`SAMPLE_RANGES`."""
        col = 0
        for a, b in self.SAMPLE_RANGES:
            if (a, b) == (lo, hi):
                if getattr(self, "_samples", None) is None:
                    raise RuntimeError("parameter samples are collected by every rank at window boundaries; none yet")
                return {sp.name: self._samples[sp.index, col: col + (b - a)].clone() for sp in self.layout.specs
                        if sp.numel >= hi}
            col += b - a
        raise KeyError(f"elements [{lo}:{hi}] are not among the cached sample ranges {self.SAMPLE_RANGES}")

    def check_status(self) -> int:
        """Reads (and clears) the kernel status word — a host sync; call between windows."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
        return v
