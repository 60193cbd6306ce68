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
                 world_size: int = 1):
        self.target_chunk = int(target_chunk)
        self.topk = int(topk)
        self.world_size = int(world_size)
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
        self.shard_units = self._partition(self.world_size)

    # -- sharding ---------------------------------------------------------------------------
    def _build_units(self):
        units = []  # (spec_i, chunk_row, elem_begin, elem_end)
        for i, s in enumerate(self.specs):
            per = s.h * s.cols
            for r in range(s.chunk_rows):
                units.append((i, r, s.offset + r * per, s.offset + (r + 1) * per))
        return units

    def _partition(self, world: int):
        ends = np.array([u[3] for u in self._units], dtype=np.int64)
        total = int(ends[-1]) if len(ends) else 0
        cuts = [0]
        for r in range(1, world):
            target = total * r / world
            j = int(np.searchsorted(ends, target, side="left"))
            j = min(max(j + 1, cuts[-1]), len(self._units))
            cuts.append(j)
        cuts.append(len(self._units))
        return [(cuts[r], cuts[r + 1]) for r in range(world)]

    def shard_range(self, rank: int) -> tuple[int, int]:
        """Element range ``[lo, hi)`` of the flat buffers owned by ``rank`` (whole chunk rows)."""
        u0, u1 = self.shard_units[rank]
        if self.world_size == 1:
            return 0, self.total
        lo = self._units[u0][2] if u0 < len(self._units) else self.total
        hi = self._units[u1][2] if u1 < len(self._units) else self.total
        if rank == 0:
            lo = 0
        return lo, hi

    def shard_entries(self, rank: int):
        """[(spec, chunk_row0, n_chunk_rows)] owned by ``rank`` in storage order."""
        u0, u1 = self.shard_units[rank]
        out = []
        for (si, r, _, _) in self._units[u0:u1]:
            if out and out[-1][0] is self.specs[si] and out[-1][1] + out[-1][2] == r:
                out[-1][2] += 1
            else:
                out.append([self.specs[si], r, 1])
        return [(s, r0, n) for s, r0, n in out]

    # -- kernel descriptor tables ---------------------------------------------------------
    def descriptors(self, rank: int | None = None, square: bool | None = None) -> np.ndarray:
        """Descriptor table for the chunk rows of ``rank`` (``None``: the whole model).

        ``square=True`` keeps tensors whose two chunk edges share one DCT matrix (h == w),
        ``square=False`` the others (e.g. 1-D tensors, h = 1); ``None`` keeps all.
        """
        entries = (self.shard_entries(rank) if rank is not None
                   else [(s, 0, s.chunk_rows) for s in self.specs])
        rows = []
        begin = 0
        for s, r0, nrows in entries:
            if square is not None and (s.h == s.w) != square:
                continue
            k = s.topk(self.topk)
            n_chunks = nrows * s.chunks_x
            c0 = r0 * s.chunks_x
            rows.append((s.offset, self.idx_off[s.name] + c0 * (k // 2) * 3, self.val_off[s.name] + c0 * k,
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
                 alloc=None):
        named = [(n, p) for n, p in model.named_parameters()]
        self.model = model
        self.device = torch.device(device) if device is not None else named[0][1].device
        self.compute_dtype = compute_dtype or named[0][1].dtype
        self.rank, self.world_size = rank, world_size
        self.layout = FlatLayout([(n, tuple(p.shape)) for n, p in named], target_chunk, topk, world_size)
        L = self.layout
        alloc = alloc or (lambda n, dtype, symmetric=False: torch.zeros(n, dtype=dtype, device=self.device))
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

    def _packed(self, names: list[str]):
        specs = [self.layout.by_name.get(n) for n in names]
        if any(s is None for s in specs):
            return None
        for a, b in zip(specs, specs[1:]):
            if a.offset + a.numel != b.offset or a.cols != b.cols:
                return None
        rows = sum(s.rows for s in specs)
        o, n = specs[0].offset, sum(s.numel for s in specs)
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
        self.grad.zero_()

    def view(self, buf: torch.Tensor, name: str, sharded: bool = False) -> torch.Tensor:
        s = self.layout.by_name[name]
        base = self.lo if sharded else 0
        return buf[s.offset - base: s.offset - base + s.numel].view(s.shape)

    def refresh_compute_from_master(self):
        """compute[lo:hi] <- cast(master shard) (single-rank or after an external master edit)."""
        if self.compute is self.master_shard:
            return
        self.compute[self.lo:self.hi].copy_(self.master_shard.to(self.compute_dtype))
