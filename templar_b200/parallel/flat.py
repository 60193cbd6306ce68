"""Flat parameter storage and chunk-aligned sharding.

All parameters of a model live in ONE contiguous buffer per role:

* ``compute``  — the dtype the forward/backward reads (bf16 on a B200), full size on every rank;
* ``grad``     — fp32 gradient accumulator (``p.main_grad`` views), full size on every rank;
* ``master``   — fp32 master weights, and the optimizer / error-feedback / snapshot state that
  goes with them; a rank holds only its shard ``[lo, hi)`` of these.

The shard boundaries fall on *chunk rows* (``h`` consecutive rows of a 2-D tensor, where
``h`` is the compression chunk edge), so that every 64x64 compression chunk, every AdamW
element and every reduce-scatter slice of a rank is a contiguous range of the flat buffer
and the per-window compression needs no re-layout: each rank compresses, aggregates and
updates exactly the range it owns.  The reference instead shards per tensor along dim 0
(FSDP2, torchtitan models/llama3/infra/parallelize.py:357-422) and compresses whole
tensors on an owner rank (neurons/miner.py:235-243).

Tensors that the model multiplies as one packed matrix (``[wq; wk; wv]`` and ``[w1; w3]``)
are placed adjacently so the packed operand is a view.

Two ways of cutting the flat space into per-rank shards:

* ``shard_params=False``: rank ``r`` owns ONE contiguous range ``[lo, hi)`` of the flat space; the bf16
  weights and the fp32 gradient accumulator stay whole on every rank (optimizer-state sharding).
* ``shard_params=True`` (the FSDP role): every *unit* (a packed matrix such as ``[wq; wk; wv]``, or a single
  tensor) is cut into ``world`` runs of chunk rows, one per rank, so a rank's shard is the concatenation of
  its piece of every unit.  bf16 weights, fp32 gradients and all optimizer state are held as shards only; the
  units of a *group* (a transformer block; what precedes the blocks; what follows them) are gathered into a
  transient full-size buffer for the forward and backward of that group and every rank's gradient tiles are
  reduce-added into the owner's shard.  The reference shards every tensor along dim 0 with FSDP2 the same way
  (torchtitan models/llama3/infra/parallelize.py:357-422), one all-gather / reduce-scatter per block.

Either way a shard is described by :class:`Piece` records ``(g_lo, g_hi, local)``: global element range
and where it starts in the rank's shard arrays.
"""

from __future__ import annotations

import re
from dataclasses import dataclass

import numpy as np
import torch

from ..compress import chunk_size_for, dct_basis

ALIGN = 64  # elements; keeps every tensor 16-byte aligned in bf16 and fp32


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    numel: int
    offset: int          # element offset in the flat buffers
    rows: int            # logical 2-D view used for chunking (1-D: rows = 1)
    cols: int
    h: int               # chunk edge along rows / cols
    w: int
    index: int           # position in named_parameters() order (the ids used by side tables)

    @property
    def chunk_rows(self) -> int:
        return self.rows // self.h

    @property
    def chunks_x(self) -> int:
        return self.cols // self.w

    @property
    def n_chunks(self) -> int:
        return self.chunk_rows * self.chunks_x

    @property
    def totalk(self) -> int:
        return self.h * self.w

    def topk(self, k: int) -> int:
        k = max(min(int(k), self.totalk), 2)
        return k - (k % 2)


@dataclass
class Piece:
    g_lo: int            # element range [g_lo, g_hi) of the flat (whole-model) space ...
    g_hi: int
    local: int           # ... and the offset of its first element in the owning rank's shard arrays
    unit: int = -1       # index of the sharding unit it was cut from (shard_params only)


@dataclass
class Unit:
    """Tensors sharded together: adjacent in the flat space, same number of columns."""
    specs: list          # ParamSpec, storage order
    group: str           # gather group: "pre", "layers.<i>", "post"
    g_lo: int = 0
    g_hi: int = 0

    @property
    def cols(self) -> int:
        return self.specs[0].cols

    @property
    def rows(self) -> int:
        return sum(s.rows for s in self.specs)


_LAYER_ORDER = ["attention_norm.weight", "attention.wq.weight", "attention.wk.weight", "attention.wv.weight",
                "attention.wo.weight", "ffn_norm.weight", "feed_forward.w1.weight", "feed_forward.w3.weight",
                "feed_forward.w2.weight"]


def _storage_order(names: list[str]) -> list[str]:
    """named_parameters() order, except that inside a transformer layer the tensors that are
    multiplied as one packed matrix become neighbours."""
    out, seen = [], set()
    by_layer: dict[str, list[str]] = {}
    for n in names:
        m = re.match(r"^(layers\.\d+)\.(.+)$", n)
        if m:
            by_layer.setdefault(m.group(1), []).append(m.group(2))
    for n in names:
        if n in seen:
            continue
        m = re.match(r"^(layers\.\d+)\.(.+)$", n)
        if not m:
            out.append(n)
            seen.add(n)
            continue
        prefix = m.group(1)
        members = by_layer[prefix]
        ordered = [x for x in _LAYER_ORDER if x in members] + [x for x in members if x not in _LAYER_ORDER]
        for x in ordered:
            out.append(f"{prefix}.{x}")
            seen.add(f"{prefix}.{x}")
    return out


class FlatLayout:
    """Geometry only (no tensors): offsets, chunk shapes, shard ranges, kernel descriptor tables."""

    DESC_DTYPE = np.dtype([
        ("elem_off", "<i8"), ("idx_off", "<i8"), ("val_off", "<i8"),
        ("rows", "<i4"), ("cols", "<i4"), ("h", "<i4"), ("w", "<i4"),
        ("chunks_x", "<i4"), ("chunk_row0", "<i4"), ("chunk_begin", "<i4"), ("n_chunks", "<i4"),
        ("k", "<i4"), ("fh_off", "<i4"), ("fw_off", "<i4"), ("param_id", "<i4"),
    ], align=True)

    def __init__(self, named_shapes: list[tuple[str, tuple]], target_chunk: int = 64, topk: int = 32,
                 world_size: int = 1, shard_params: bool = False):
        self.target_chunk = int(target_chunk)
        self.topk = int(topk)
        self.world_size = int(world_size)
        self.shard_params = bool(shard_params)
        index = {n: i for i, (n, _) in enumerate(named_shapes)}
        shapes = dict(named_shapes)
        self.specs: list[ParamSpec] = []
        off = 0
        for name in _storage_order([n for n, _ in named_shapes]):
            shape = tuple(int(s) for s in shapes[name])
            numel = int(np.prod(shape)) if len(shape) else 1
            if len(shape) >= 2:
                rows, cols = shape[0], numel // shape[0]
            else:
                rows, cols = 1, numel
            h = chunk_size_for(rows, self.target_chunk) if len(shape) >= 2 else 1
            w = chunk_size_for(cols, self.target_chunk)
            self.specs.append(ParamSpec(name, shape, numel, off, rows, cols, h, w, index[name]))
            off += -(-numel // ALIGN) * ALIGN
        self.total = -(-off // (ALIGN * max(self.world_size, 1))) * ALIGN * max(self.world_size, 1)
        self.by_name = {s.name: s for s in self.specs}
        self.n_params = len(self.specs)
        # payload layout (full model, storage order): packed indices then values
        self.idx_off, self.val_off = {}, {}
        io = vo = 0
        for s in self.specs:
            k = s.topk(self.topk)
            self.idx_off[s.name], self.val_off[s.name] = io, vo
            io += s.n_chunks * (k // 2) * 3
            vo += s.n_chunks * k
        self.idx_bytes = -(-io // 16) * 16
        self.val_elems = -(-vo // 4) * 4
        # DCT basis table: one n x n matrix per distinct chunk edge
        self.basis_off: dict[int, int] = {}
        bo = 0
        for s in self.specs:
            for n in (s.h, s.w):
                if n not in self.basis_off:
                    self.basis_off[n] = bo
                    bo += n * n
        self.basis_elems = bo
        self._units = self._build_units()
        self.shard_units = self._partition(self._units, self.world_size)
        self.units: list[Unit] = []
        self.groups: dict[str, list[int]] = {}
        if self.shard_params:
            self._build_param_sharding()
        else:
            self.rank_pieces = []
            for r in range(self.world_size):
                lo, hi = self.shard_range(r)
                self.rank_pieces.append([Piece(lo, hi, 0)])

    # -- sharding ---------------------------------------------------------------------------
    def _build_units(self):
        units = []  # (spec_i, chunk_row, elem_begin, elem_end)
        for i, s in enumerate(self.specs):
            per = s.h * s.cols
            for r in range(s.chunk_rows):
                units.append((i, r, s.offset + r * per, s.offset + (r + 1) * per))
        return units

    @staticmethod
    def _partition(rows, world: int):
        """Cut the chunk rows ``rows`` ([(spec_i, chunk_row, begin, end)], contiguous) into ``world`` runs of
        about equal element count; returns the (first, end) row indices per rank."""
        ends = np.array([u[3] for u in rows], dtype=np.int64)
        begin = int(rows[0][2]) if len(rows) else 0
        total = int(ends[-1]) - begin if len(ends) else 0
        cuts = [0]
        for r in range(1, world):
            target = begin + total * r / world
            j = int(np.searchsorted(ends, target, side="left"))
            j = min(max(j + 1, cuts[-1]), len(rows))
            cuts.append(j)
        cuts.append(len(rows))
        return [(cuts[r], cuts[r + 1]) for r in range(world)]

    def _build_param_sharding(self) -> None:
        """Units (packed matrices / single tensors), their gather groups, and every rank's pieces."""
        first_layer = next((i for i, s in enumerate(self.specs) if s.name.startswith("layers.")), len(self.specs))
        last_layer = max((i for i, s in enumerate(self.specs) if s.name.startswith("layers.")), default=-1)

        def group_of(i: int, s: ParamSpec) -> str:
            m = re.match(r"^(layers\.\d+)\.", s.name)
            if m:
                return m.group(1)
            return "pre" if i < first_layer else ("post" if i > last_layer else "pre")

        packs = (("attention.wq.weight", "attention.wk.weight", "attention.wv.weight"),
                 ("feed_forward.w1.weight", "feed_forward.w3.weight"))
        i = 0
        while i < len(self.specs):
            s = self.specs[i]
            members = [s]
            for pack in packs:
                if s.name.endswith(pack[0]):
                    pre = s.name[: -len(pack[0])]
                    cand = self.specs[i: i + len(pack)]
                    ok = (len(cand) == len(pack) and all(c.name == pre + n for c, n in zip(cand, pack))
                          and all(c.cols == s.cols and c.h == s.h and len(c.shape) == 2 for c in cand)
                          and all(a.offset + a.numel == b.offset for a, b in zip(cand, cand[1:])))
                    if ok:
                        members = list(cand)
            u = Unit(members, group_of(i, s), members[0].offset, members[-1].offset + members[-1].numel)
            self.groups.setdefault(u.group, []).append(len(self.units))
            self.units.append(u)
            i += len(members)
        spec_index = {id(s): k for k, s in enumerate(self.specs)}
        self.rank_pieces = [[] for _ in range(self.world_size)]
        self.unit_pieces: list[list[Piece | None]] = []       # [unit][rank] (None: that rank owns nothing of the unit)
        self.unit_rows: list[list[tuple[int, int]]] = []      # [unit][rank] = (first chunk-row index, end) in _units
        local = [0] * self.world_size
        for ui, u in enumerate(self.units):
            rows = [x for x in self._units if spec_index[id(u.specs[0])] <= x[0] <= spec_index[id(u.specs[-1])]]
            cuts = self._partition(rows, self.world_size)
            per_rank, per_rows = [], []
            for r, (a, b) in enumerate(cuts):
                if a == b:
                    per_rank.append(None)
                    per_rows.append((0, 0))
                    continue
                p = Piece(rows[a][2], rows[b - 1][3], local[r], ui)
                local[r] += -(-(p.g_hi - p.g_lo) // ALIGN) * ALIGN
                self.rank_pieces[r].append(p)
                per_rank.append(p)
                per_rows.append((self._units.index(rows[a]), self._units.index(rows[b - 1]) + 1))
            self.unit_pieces.append(per_rank)
            self.unit_rows.append(per_rows)
        self._shard_sizes = local

    def shard_size(self, rank: int) -> int:
        """Elements of ``rank``'s shard arrays."""
        if self.shard_params:
            return self._shard_sizes[rank]
        lo, hi = self.shard_range(rank)
        return hi - lo

    @property
    def shard_size_max(self) -> int:
        return max(self.shard_size(r) for r in range(self.world_size))

    def pieces(self, rank: int) -> list[Piece]:
        return self.rank_pieces[rank]

    def segments(self, rank: int):
        """[(spec, a, b, local_a)]: for every tensor, the parts ``[a, b)`` (flat element range) that ``rank`` owns
        and where each starts in the rank's shard arrays; storage order."""
        cache = self.__dict__.setdefault("_segments_cache", {})
        if rank in cache:
            return cache[rank]
        out = []
        starts = [s.offset for s in self.specs]
        for p in self.rank_pieces[rank]:
            i = max(int(np.searchsorted(starts, p.g_lo, side="right")) - 1, 0)
            while i < len(self.specs) and self.specs[i].offset < p.g_hi:
                s = self.specs[i]
                a, b = max(s.offset, p.g_lo), min(s.offset + s.numel, p.g_hi)
                if a < b:
                    out.append((s, a, b, p.local + (a - p.g_lo)))
                i += 1
        out.sort(key=lambda t: t[1])
        cache[rank] = out
        return out

    def shard_range(self, rank: int) -> tuple[int, int]:
        """Element range ``[lo, hi)`` of the flat buffers owned by ``rank`` (whole chunk rows); only without
        ``shard_params``, where a shard is one range."""
        if self.shard_params and self.world_size > 1:
            raise ValueError("with shard_params a rank's shard is a list of pieces: use pieces() / segments()")
        u0, u1 = self.shard_units[rank]
        if self.world_size == 1:
            return 0, self.total
        lo = self._units[u0][2] if u0 < len(self._units) else self.total
        hi = self._units[u1][2] if u1 < len(self._units) else self.total
        if rank == 0:
            lo = 0
        return lo, hi

    def shard_entries(self, rank: int):
        """[(spec, chunk_row0, n_chunk_rows, local)] owned by ``rank`` in storage order; ``local`` is the offset
        of the first of those rows in the rank's shard arrays."""
        if self.shard_params:
            runs = [(a, b, p.local, p.g_lo) for p, (a, b) in
                    ((self.unit_pieces[ui][rank], self.unit_rows[ui][rank]) for ui in range(len(self.units)))
                    if p is not None]
        else:
            u0, u1 = self.shard_units[rank]
            lo = self.shard_range(rank)[0]
            runs = [(u0, u1, 0, lo)]
        out = []
        for a, b, local, g_lo in runs:
            for (si, r, begin, _) in self._units[a:b]:
                if out and out[-1][0] is self.specs[si] and out[-1][1] + out[-1][2] == r:
                    out[-1][2] += 1
                else:
                    out.append([self.specs[si], r, 1, local + (begin - g_lo)])
        return [(s, r0, n, loc) for s, r0, n, loc in out]

    # -- kernel descriptor tables ---------------------------------------------------------
    def descriptors(self, rank: int | None = None, square: bool | None = None) -> np.ndarray:
        """Descriptor table for the chunk rows of ``rank`` (``None``: the whole model, offsets into full-size
        buffers).  With a rank, ``elem_off`` addresses the rank's shard arrays (see :meth:`shard_entries`).

        ``square=True`` keeps tensors whose two chunk edges share one DCT matrix (h == w),
        ``square=False`` the others (e.g. 1-D tensors, h = 1); ``None`` keeps all.
        """
        entries = (self.shard_entries(rank) if rank is not None
                   else [(s, 0, s.chunk_rows, s.offset) for s in self.specs])
        rows = []
        begin = 0
        for s, r0, nrows, local in entries:
            if square is not None and (s.h == s.w) != square:
                continue
            k = s.topk(self.topk)
            n_chunks = nrows * s.chunks_x
            c0 = r0 * s.chunks_x
            # the kernels address element (row, col) of the tensor at elem_off + row * cols + col with rows counted
            # from the tensor's first row, so the entry's offset is that of a (virtual) row 0 in the shard arrays
            rows.append((local - r0 * s.h * s.cols, self.idx_off[s.name] + c0 * (k // 2) * 3, self.val_off[s.name] + c0 * k,
                         s.rows, s.cols, s.h, s.w, s.chunks_x, r0, begin, n_chunks, k,
                         self.basis_off[s.h], self.basis_off[s.w], s.index))
            begin += n_chunks
        return np.array(rows, dtype=self.DESC_DTYPE)

    def basis_table(self) -> torch.Tensor:
        t = torch.zeros(max(self.basis_elems, 1), dtype=torch.float32)
        for n, off in self.basis_off.items():
            t[off:off + n * n] = dct_basis(n).reshape(-1)
        return t

    def payload_views(self, idx_buf: torch.Tensor, val_buf: torch.Tensor, name: str):
        """(packed indices uint8 [n_pairs*3], values [y, x, k] or [x, k]) views of one tensor."""
        s = self.by_name[name]
        k = s.topk(self.topk)
        io, vo = self.idx_off[name], self.val_off[name]
        idx = idx_buf[io: io + s.n_chunks * (k // 2) * 3]
        val = val_buf[vo: vo + s.n_chunks * k]
        val = val.view(s.chunk_rows, s.chunks_x, k) if len(s.shape) >= 2 else val.view(s.chunks_x, k)
        return idx, val

    def xshape(self, name: str):
        s = self.by_name[name]
        return (s.chunk_rows, s.chunks_x, s.h, s.w) if len(s.shape) >= 2 else (s.chunks_x, s.w)


class FlatParamStore:
    """Owns the flat buffers and re-points a model's parameters into them.

    ``alloc(nbytes_elems, dtype, symmetric)`` may be supplied to place buffers that peers
    read or write (``compute``, ``grad``) in the symmetric heap.
    """

    def __init__(self, model: torch.nn.Module, *, compute_dtype: torch.dtype | None = None,
                 device=None, target_chunk: int = 64, topk: int = 32, rank: int = 0, world_size: int = 1,
                 alloc=None, shard_params: bool = False, n_buffers: int = 2, group=None, heap=None,
                 status: torch.Tensor | None = None, materialize=None):
        named = [(n, p) for n, p in model.named_parameters()]
        # parameters on the meta device are created one at a time by `materialize(name) -> tensor`
        self._materialize = materialize
        self.model = model
        self.device = torch.device(device) if device is not None else named[0][1].device
        self.compute_dtype = compute_dtype or named[0][1].dtype
        self.rank, self.world_size = rank, world_size
        self.shard_params = bool(shard_params)
        self.layout = FlatLayout([(n, tuple(p.shape)) for n, p in named], target_chunk, topk, world_size,
                                 shard_params=shard_params)
        L = self.layout
        alloc = alloc or (lambda n, dtype, symmetric=False: torch.zeros(n, dtype=dtype, device=self.device))
        self.n_shard = L.shard_size(rank)
        if self.shard_params:
            self._init_sharded(named, alloc, n_buffers, group, heap, status)
            return
        self.gather = None
        self.lo, self.hi = L.shard_range(rank)
        self.master = alloc(L.total, torch.float32, False) if world_size == 1 else None
        self.master_shard = (self.master if world_size == 1
                             else alloc(self.hi - self.lo, torch.float32, False))
        if self.compute_dtype == torch.float32 and world_size == 1:
            self.compute = self.master
        else:
            self.compute = alloc(L.total, self.compute_dtype, True)
        self.grad = alloc(L.total, torch.float32, True)
        with torch.no_grad():
            for n, p in named:
                s = L.by_name[n]
                view = self.compute[s.offset: s.offset + s.numel].view(s.shape)
                src = p.detach().to(device=self.device)
                view.copy_(src.to(self.compute_dtype))
                if self.master_shard is not self.compute:
                    a, b = max(s.offset, self.lo), min(s.offset + s.numel, self.hi)
                    if a < b:
                        self.master_shard[a - self.lo: b - self.lo].copy_(
                            src.reshape(-1)[a - s.offset: b - s.offset].to(torch.float32))
                p.data = view
                p.main_grad = self.grad[s.offset: s.offset + s.numel].view(s.shape)
        self._attach_packed()

    # -- parameter sharding -----------------------------------------------------------------------
    def _init_sharded(self, named, alloc, n_buffers: int, group, heap, status) -> None:
        """``shard_params``: weights (compute dtype), gradients and master weights as shards; the model's
        parameters become fixed views of the gather buffers (:class:`templar_b200.parallel.fsdp.ParamGather`).

        Gradients.  On CUDA the matrices of the blocks and the output head get a
        :class:`~templar_b200.parallel.fsdp.GradScatter` as ``main_grad`` (their weight-gradient GEMM adds into the
        owners' shards); the tensors whose gradient is not a GEMM (norm weights, the embedding table) accumulate
        in ``stage``, a local full-size fp32 buffer of just those tensors, reduced into the shards once per inner
        step.  On CPU every tensor is staged."""
        from .fsdp import GradScatter, ParamGather

        L = self.layout
        cuda = self.device.type == "cuda"
        n_max = L.shard_size_max
        self.lo = self.hi = None                                   # a shard is a list of pieces here
        self.master = None
        self.master_shard = alloc(self.n_shard, torch.float32, False)
        self.compute_shard = alloc(n_max, self.compute_dtype, True)
        self.grad_shard = alloc(n_max, torch.float32, True)
        self.compute = self.grad = None                            # no full-size weight or gradient buffer exists
        self.gather = ParamGather(L, self.compute_shard, rank=self.rank, world_size=self.world_size, group=group,
                                  heap=heap, n_buffers=n_buffers)
        # which tensors are staged, and where
        unit_of = {}
        for ui, u in enumerate(L.units):
            for sp in u.specs:
                unit_of[sp.name] = ui
        tied = len({id(p) for _, p in named}) != len(named)

        def scatterable(u) -> bool:
            return (cuda and not tied and all(len(sp.shape) == 2 for sp in u.specs) and u.group != "pre"
                    and all(sp.h % 32 == 0 for sp in u.specs) and u.cols % 4 == 0)

        self.stage_off: dict[str, int] = {}
        off = 0
        for u in L.units:
            if not scatterable(u):
                for sp in u.specs:
                    self.stage_off[sp.name] = off
                    off += -(-sp.numel // ALIGN) * ALIGN
        self.stage = alloc(max(off, ALIGN), torch.float32, True)
        self.scatter: dict[int, GradScatter] = {}
        esz = 4
        for ui, u in enumerate(L.units):
            if not scatterable(u):
                continue
            bounds, ptrs, row = [0], [], 0
            for r, p in enumerate(L.unit_pieces[ui]):
                rows = 0 if p is None else (p.g_hi - p.g_lo) // u.cols
                row += rows
                bounds.append(row)
                base = heap.peer_ptr(self.grad_shard, r) if (heap is not None and self.world_size > 1) \
                    else self.grad_shard.data_ptr()
                ptrs.append(base + (0 if p is None else p.local) * esz)
                if p is not None and (p.local + rows * u.cols > self.grad_shard.numel() or (p.g_hi - p.g_lo) % u.cols):
                    raise ValueError(f"gradient piece of unit {ui} on rank {r} does not fit the gradient shard")
            if row != u.rows:
                raise ValueError(f"unit {ui}: the ranks' pieces cover {row} of {u.rows} rows")
            self.scatter[ui] = GradScatter(u.rows, u.cols, bounds, ptrs, self.rank, status)
        mine: dict[str, list] = {}
        for s2, a, b, la in L.segments(self.rank):
            mine.setdefault(s2.name, []).append((a, b, la))
        with torch.no_grad():
            for n, p in named:
                sp = L.by_name[n]
                if n in mine or not p.is_meta:
                    flat = self._initial_value(n, p).reshape(-1)
                    for a, b, la in mine.get(n, ()):
                        self.master_shard[la: la + (b - a)].copy_(flat[a - sp.offset: b - sp.offset].to(torch.float32))
                        self.compute_shard[la: la + (b - a)].copy_(flat[a - sp.offset: b - sp.offset].to(self.compute_dtype))
                    del flat
                p = self._repoint(n, p, self.gather.param_view(sp))
                if n in self.stage_off:
                    o = self.stage_off[n]
                    p.main_grad = self.stage[o: o + sp.numel].view(sp.shape)
                else:
                    u = L.units[unit_of[n]]
                    p.main_grad = self.scatter[unit_of[n]] if len(u.specs) == 1 else None
        self._attach_packed()

    def _initial_value(self, name: str, p: torch.Tensor) -> torch.Tensor:
        if p.is_meta:
            if self._materialize is None:
                raise ValueError(f"parameter {name} is on the meta device and no `materialize` function was given")
            return self._materialize(name).to(self.device)
        return p.detach().to(device=self.device)

    def _repoint(self, name: str, p: torch.nn.Parameter, view: torch.Tensor) -> torch.nn.Parameter:
        """Make the model's parameter ``name`` a view of flat storage; a meta parameter is replaced by a new one."""
        if not p.is_meta:
            p.data = view
            return p
        mod = self.model
        *path, leaf = name.split(".")
        for part in path:
            mod = getattr(mod, part) if not part.isdigit() or not hasattr(mod, "__getitem__") else mod[part]
        new = torch.nn.Parameter(view, requires_grad=p.requires_grad)
        setattr(mod, leaf, new)
        return new

    def stage_blocks(self, block: int = 16384):
        """[(src_off, dst_off, n)] records for the reduction of the staged gradients: the parts of staged tensors
        that this rank owns, as offsets into ``stage`` and into the gradient shard."""
        rec = []
        for sp, a, b, la in self.layout.segments(self.rank):
            if sp.name not in self.stage_off:
                continue
            so = self.stage_off[sp.name] + (a - sp.offset)
            for off in range(0, b - a, block):
                rec.append((so + off, la + off, min(block, b - a - off)))
        return rec

    def _packed(self, names: list[str]):
        specs = [self.layout.by_name.get(n) for n in names]
        if any(s is None for s in specs):
            return None
        for a, b in zip(specs, specs[1:]):
            if a.offset + a.numel != b.offset or a.cols != b.cols:
                return None
        rows = sum(s.rows for s in specs)
        o, n = specs[0].offset, sum(s.numel for s in specs)
        if self.shard_params:
            first = self.gather.param_view(specs[0])
            weight = torch.as_strided(first, (rows, specs[0].cols), (specs[0].cols, 1))
            ui = next(i for i, u in enumerate(self.layout.units) if u.specs[0] is specs[0])
            if len(self.layout.units[ui].specs) != len(specs):
                return None
            if ui in self.scatter:
                return (weight, self.scatter[ui])
            so = self.stage_off[specs[0].name]                  # staged tensors of a unit are adjacent in `stage`
            return (weight, self.stage[so: so + n].view(rows, specs[0].cols))
        return (self.compute[o:o + n].view(rows, specs[0].cols), self.grad[o:o + n].view(rows, specs[0].cols))

    def _attach_packed(self):
        layers = getattr(self.model, "layers", None)
        if layers is None:
            return
        items = layers.items() if hasattr(layers, "items") else enumerate(layers)
        for key, layer in items:
            pre = f"layers.{key}"
            att, ff = getattr(layer, "attention", None), getattr(layer, "feed_forward", None)
            if att is not None and hasattr(att, "packed"):
                att.packed = self._packed([f"{pre}.attention.wq.weight", f"{pre}.attention.wk.weight",
                                           f"{pre}.attention.wv.weight"])
            if ff is not None and hasattr(ff, "packed"):
                ff.packed = self._packed([f"{pre}.feed_forward.w1.weight", f"{pre}.feed_forward.w3.weight"])

    # -- helpers ----------------------------------------------------------------------------
    def zero_grad(self):
        if self.shard_params:
            self.grad_shard.zero_()
            self.stage.zero_()
            return
        self.grad.zero_()

    def view(self, buf: torch.Tensor, name: str, sharded: bool = False) -> torch.Tensor:
        s = self.layout.by_name[name]
        base = self.lo if sharded else 0
        return buf[s.offset - base: s.offset - base + s.numel].view(s.shape)

    def refresh_compute_from_master(self):
        """compute[lo:hi] <- cast(master shard) (single-rank or after an external master edit)."""
        if self.shard_params:
            self.compute_shard[: self.n_shard].copy_(self.master_shard.to(self.compute_dtype))
            self.gather.invalidate()
            return
        if self.compute is self.master_shard:
            return
        self.compute[self.lo:self.hi].copy_(self.master_shard.to(self.compute_dtype))
