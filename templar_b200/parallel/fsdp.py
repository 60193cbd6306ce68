"""Run-time side of parameter sharding (the FSDP role): gathering a group's weights ahead of its use, and
reducing weight gradients into their owners' shards from inside the GEMM that produces them.

Layout (see :mod:`templar_b200.parallel.flat`): every unit (a packed matrix or a single tensor) is cut into one
run of chunk rows per rank; a rank keeps only its pieces of the bf16 weights, the fp32 gradients and the
optimizer state.  The units of one *group* (a transformer block, what precedes the blocks, what follows them)
are gathered together into a full-size buffer whose address never changes, so the parameters of the model are
fixed views of those buffers and only the buffers' contents come and go.

* :class:`ParamGather` owns the buffers.  Blocks share ``n_buffers`` buffers in rotation; while block ``i``
  computes, the pieces of the next block (the previous one in the backward pass) are pulled from the peers'
  shards over NVLink by a copy kernel on a side stream.  The peers' shards only change in the optimizer and
  outer steps, which are fenced by barriers, so a gather needs no hand-shake with the peers at all.
* :class:`GradScatter` stands in for a weight's ``main_grad``: the weight-gradient GEMM's epilogue reduce-adds
  every tile straight into the shard of the rank that owns those rows (``tplr_gemm2_scatter_v``), so the
  fp32 gradient of a matrix exists only as shards and its reduce-scatter is finished when the backward pass is.

The reference gets the same roles from FSDP2: an NCCL all-gather before each block's forward and backward and an
fp32 reduce-scatter after each block's backward (torchtitan models/llama3/infra/parallelize.py:357-422,
src/tplr/model_factory.py:153,183).  On CPU (gloo) the gather is a set of broadcasts and the gradients are
accumulated in full size and reduced piece by piece, which checks the layout arithmetic without a GPU.
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch
import torch.distributed as dist

from ..ops import native


class GradScatter:
    """Target of a weight-gradient GEMM under parameter sharding: ``accumulate(dy, x)`` adds ``dy^T x`` (fp32) into
    the owners' gradient shards.  ``bounds[o] .. bounds[o + 1]`` are the rows of the (packed) matrix that rank
    ``o`` owns and ``ptrs[o]`` the address, in this process, of that rank's [rows_o, cols] piece."""

    def __init__(self, rows: int, cols: int, bounds: list[int], ptrs: list[int], rank: int, status: torch.Tensor):
        self.rows, self.cols, self.rank, self.world = rows, cols, rank, len(ptrs)
        self.bounds = (ctypes.c_int * (self.world + 1))(*bounds)
        self.ptrs = native.ptr_array(ptrs)
        self.status = status

    def accumulate(self, dy2: torch.Tensor, x2: torch.Tensor) -> None:
        native.require(dy2.shape[1] == self.rows and x2.shape[1] == self.cols and dy2.shape[0] == x2.shape[0],
                       "GradScatter: operand shapes do not match the weight")
        err = native.lib().tplr_gemm2_scatter_v(dy2.data_ptr(), x2.data_ptr(), self.rows, self.cols, dy2.shape[0],
                                                dy2.stride(0), x2.stride(0), 1, 1, self.world, self.rank, self.bounds,
                                                self.ptrs, self.status.data_ptr(), native.stream_ptr())
        native.check(err, "tplr_gemm2_scatter_v")


class ParamGather:
    """Buffers and schedule of the gathered weights of a :class:`~templar_b200.parallel.flat.FlatParamStore`
    with ``shard_params``."""

    def __init__(self, layout, compute_shard: torch.Tensor, *, rank: int, world_size: int, group=None, heap=None,
                 n_buffers: int = 2, copy_ctas: int = 32, engine: str | None = None):
        self.layout, self.shard = layout, compute_shard
        self.rank, self.world_size, self.group, self.heap = rank, world_size, group, heap
        self.device, self.dtype = compute_shard.device, compute_shard.dtype
        self.cuda = self.device.type == "cuda"
        self.copy_ctas = copy_ctas
        # who moves the bytes of a gather: "dma" = the copy engines (one asynchronous peer copy per piece, no SM and no
        # L2 traffic of its own beside the GEMMs), "sm" = the block-table copy kernel (one launch per gather, plain
        # loads from the peers' shards).  Measured on the 1B window at 2 GPUs with two rotating buffers: 541 ms per
        # window with the copy engines, 561 ms with the kernel (whole weights on every rank: 534 ms).
        # TPLR_GATHER_ENGINE overrides.
        import os

        self.engine = engine or os.environ.get("TPLR_GATHER_ENGINE", "dma")
        if self.engine not in ("sm", "dma"):
            raise ValueError(f"gather engine must be 'sm' or 'dma', got {self.engine!r}")
        L = layout
        self.names = list(L.groups)                                  # gather groups in storage order
        self.layer_names = [g for g in self.names if g.startswith("layers.")]
        self.range = {g: (L.units[u[0]].g_lo, L.units[u[-1]].g_hi) for g, u in L.groups.items()}
        size = lambda g: self.range[g][1] - self.range[g][0]
        n_layers = len(self.layer_names)
        if n_buffers <= 0:
            # automatic: keep every block gathered between optimizer steps when the whole model's weights are a small
            # part of the device memory (nothing is re-gathered in the backward pass or in later micro-batches), else
            # rotate two buffers
            whole = sum(size(g) for g in self.layer_names) * compute_shard.element_size()
            n_buffers = n_layers if whole <= 8 * 2 ** 30 else 2
        self.n_buffers = max(min(n_buffers, n_layers), min(2, n_layers))
        layer_elems = max((size(g) for g in self.layer_names), default=0)
        z = lambda n: torch.zeros(max(n, 1), dtype=self.dtype, device=self.device)
        self.layer_bufs = [z(layer_elems) for _ in range(self.n_buffers)]
        self.slot: dict[str, int] = {}
        self.buf: dict[str, torch.Tensor] = {}
        for i, g in enumerate(self.layer_names):
            self.slot[g] = i % self.n_buffers
            self.buf[g] = self.layer_bufs[self.slot[g]]
        for g in self.names:
            if g not in self.buf:
                self.slot[g] = -1 - len([x for x in self.buf if not x.startswith("layers.")])
                self.buf[g] = z(size(g))
        self.holds: dict[int, str | None] = {}                      # slot -> group whose weights it contains
        self.ready: dict[int, object] = {}                          # slot -> event: the gather into it has finished
        self.waited: set[int] = set()                               # slots whose gather the compute stream has joined
        self.comm = torch.cuda.Stream(self.device) if self.cuda else None
        self.gathers = 0                                            # gathers issued (for tests and the bench)
        self.in_backward = False                                    # direction of the pass, for the look-ahead
        self._tables: dict[str, tuple[torch.Tensor, int]] = {}
        self._copies: dict[str, list] = {}
        if self.cuda:
            for g in self.names:
                if self.engine == "dma":
                    self._copies[g] = self._copy_list(g)
                else:
                    self._tables[g] = self._block_table(g)

    # -- static description ------------------------------------------------------------------
    def param_view(self, spec) -> torch.Tensor:
        """The fixed view of tensor ``spec`` inside its group's buffer."""
        for g, units in self.layout.groups.items():
            lo, hi = self.range[g]
            if lo <= spec.offset < hi:
                return self.buf[g][spec.offset - lo: spec.offset - lo + spec.numel].view(spec.shape)
        raise KeyError(spec.name)

    def _peer_base(self, r: int) -> int:
        if self.heap is not None and self.world_size > 1:
            return self.heap.peer_ptr(self.shard, r)
        return self.shard.data_ptr()

    def _block_table(self, g: str):
        """Device table of {src, dst, bytes} records: every rank's piece of every unit of group ``g``, cut into
        blocks of at most 64 KiB (more for very large groups, to bound the table)."""
        esz = self.shard.element_size()
        lo, hi = self.range[g]
        block = max(65536, -(-((hi - lo) * esz // 4096) // 16) * 16)
        dst0 = self.buf[g].data_ptr()
        rec = []
        for ui in self.layout.groups[g]:
            for r, p in enumerate(self.layout.unit_pieces[ui]):
                if p is None:
                    continue
                src = self._peer_base(r) + p.local * esz
                dst = dst0 + (p.g_lo - lo) * esz
                n = (p.g_hi - p.g_lo) * esz
                # checked on the host: a record outside the shard or the buffer would be a stray access on the device
                native.require(0 <= p.local and (p.local + p.g_hi - p.g_lo) <= self.shard.numel()
                               and 0 <= p.g_lo - lo and p.g_hi - lo <= self.buf[g].numel()
                               and src % 16 == 0 and dst % 16 == 0 and n % 16 == 0,
                               f"gather table of {g}: piece of rank {r} does not fit its shard or buffer")
                for off in range(0, n, block):
                    rec.append((src + off, dst + off, min(block, n - off)))
        arr = np.array(rec, dtype=np.int64).reshape(-1, 3)
        return torch.from_numpy(arr).to(self.device), len(rec)

    def _copy_list(self, g: str):
        """[(destination view, source view)] of group ``g``: every rank's piece of every unit; the source views
        address the peers' shards as mapped into this process."""
        from .symmetric import _DeviceBlock

        esz = self.shard.element_size()
        lo, _ = self.range[g]
        if not hasattr(self, "_peer_shards"):
            self._peer_shards = []
            for r in range(self.world_size):
                if r == self.rank or self.heap is None or self.world_size == 1:
                    self._peer_shards.append(self.shard)
                else:
                    blk = _DeviceBlock(self._peer_base(r), self.shard.numel() * esz)
                    self._peer_blocks = getattr(self, "_peer_blocks", []) + [blk]
                    self._peer_shards.append(torch.as_tensor(blk, device=self.device).view(self.dtype))
        out = []
        for ui in self.layout.groups[g]:
            for r, p in enumerate(self.layout.unit_pieces[ui]):
                if p is None:
                    continue
                n = p.g_hi - p.g_lo
                out.append((self.buf[g][p.g_lo - lo: p.g_lo - lo + n], self._peer_shards[r][p.local: p.local + n]))
        return out

    # -- schedule ------------------------------------------------------------------------------
    def invalidate(self) -> None:
        """The shards changed (optimizer or outer step): nothing gathered so far is current."""
        self.holds.clear()
        self.ready.clear()
        self.waited.clear()

    def _gather(self, g: str) -> None:
        """Fill ``g``'s buffer from the shards.  CUDA: on the side stream, after everything the compute stream has
        been given so far (which includes the last use of the buffer's previous contents)."""
        slot = self.slot[g]
        self.gathers += 1
        if self.cuda:
            cur = torch.cuda.current_stream(self.device)
            self.comm.wait_stream(cur)
            with torch.cuda.stream(self.comm):
                if self.engine == "dma":
                    for dst, src in self._copies[g]:
                        dst.data.copy_(src, non_blocking=True)      # `.data`: no version bump on views autograd holds
                else:
                    table, n = self._tables[g]
                    native.check(native.lib().tplr_copy_blocks(table.data_ptr(), n, self.copy_ctas,
                                                               self.comm.cuda_stream), "copy_blocks")
                ev = torch.cuda.Event()
                ev.record(self.comm)
            self.ready[slot] = ev
            self.waited.discard(slot)
        else:
            lo, _ = self.range[g]
            # `.data` has its own version counter: autograd has saved views of this buffer for the backward pass
            # and, as on CUDA where a kernel refills it, must not take the refill for an in-place edit
            buf = self.buf[g].data
            for ui in self.layout.groups[g]:
                for r, p in enumerate(self.layout.unit_pieces[ui]):
                    if p is None:
                        continue
                    part = buf[p.g_lo - lo: p.g_hi - lo]
                    if r == self.rank:
                        part.copy_(self.shard[p.local: p.local + (p.g_hi - p.g_lo)])
                    if self.world_size > 1:
                        src = dist.get_global_rank(self.group, r) if self.group is not None else r
                        dist.broadcast(part, src=src, group=self.group)
        self.holds[slot] = g

    def prefetch(self, g: str | None) -> None:
        """Start gathering ``g`` unless its buffer already holds it.  On CPU the gather is a collective and is
        left to :meth:`acquire`, which every rank reaches at the same point."""
        if g is None or not self.cuda or self.holds.get(self.slot[g]) == g:
            return
        self._gather(g)

    def acquire(self, g: str) -> None:
        """After this call the current stream may read ``g``'s weights."""
        slot = self.slot[g]
        if self.holds.get(slot) != g:
            self._gather(g)
        if self.cuda and slot not in self.waited:
            torch.cuda.current_stream(self.device).wait_event(self.ready[slot])
            self.waited.add(slot)

    def begin_forward(self) -> None:
        """Start of a forward pass: the first group is brought in and the first block is on its way."""
        self.in_backward = False
        if "pre" in self.slot:
            self.acquire("pre")
        if self.layer_names:
            self.prefetch(self.layer_names[0])

    def neighbour(self, g: str, step: int) -> str | None:
        i = self.layer_names.index(g) + step
        return self.layer_names[i] if 0 <= i < len(self.layer_names) else None

    # -- gates placed around a block by the model ------------------------------------------------
    def enter(self, g: str, *tensors):
        """Before block ``g``: its weights are current for the forward pass (and for a recomputation of it), and
        the next block's are on their way."""
        return _Gate.apply(self, g, 0, *tensors)

    def leave(self, g: str, *tensors):
        """After block ``g``: in the backward pass, which reaches this point first, the block's weights are
        brought back and the previous block's are on their way."""
        return _Gate.apply(self, g, 1, *tensors)


class _Gate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pg: ParamGather, g: str, side: int, *tensors):
        ctx.pg, ctx.g, ctx.side = pg, g, side
        if side == 0:
            pg.acquire(g)
            if not pg.in_backward:               # a recomputation inside the backward pass looks ahead the other way
                nxt = pg.neighbour(g, +1)
                pg.prefetch(nxt if nxt is not None else ("post" if "post" in pg.slot else None))
        return tensors if len(tensors) > 1 else tensors[0]

    @staticmethod
    def backward(ctx, *grads):
        pg, g = ctx.pg, ctx.g
        if ctx.side == 1:
            pg.in_backward = True
            pg.acquire(g)
            pg.prefetch(pg.neighbour(g, -1))
        return (None, None, None, *grads)
