"""Chunking, DCT, top-k sparsification, 12-bit index packing and value quantisation.

This module is the numerical specification of the compressed pseudo-gradient
format.  Everything here is plain PyTorch and runs on any device; it is the
oracle every CUDA kernel in :mod:`templar_b200.ops` is tested against, and the
path taken on CPU.  On a B200 the per-window pipeline does not call these
functions tensor by tensor — :class:`templar_b200.parallel.window_engine.WindowEngine`
runs the fused kernels over the whole flat parameter buffer — but the wire format
produced is byte-identical.

Behavioural parity with the reference (paths are relative to its project root):

* ``pack_12bit_indices`` / ``unpack_12bit_indices``  — src/tplr/compress.py:51-142
* ``ChunkingTransformer``                            — src/tplr/compress.py:145-292
* ``TopKCompressor``                                 — src/tplr/compress.py:295-696
* DCT-II / DCT-III orthonormal bases                 — src/tplr/compress.py:710-788
* chunk size = largest divisor <= target             — src/tplr/compress.py:820-872
"""

from __future__ import annotations

import math
import typing

import torch

__all__ = [
    "pack_12bit_indices",
    "unpack_12bit_indices",
    "ChunkingTransformer",
    "TopKCompressor",
    "dct_basis",
    "chunk_size_for",
    "ShapeT", "Shape4D", "TotK", "IdxT", "QuantParamsT", "ValT", "Q",
]

# names for the pieces of a payload, as annotations in callers' code use them (src/tplr/compress.py:35-48)
ShapeT = tuple[int, ...]                        # shape of the dense tensor
Shape4D = tuple[int, int, int, int]             # (rows of chunks, columns of chunks, chunk height, chunk width)
TotK = int                                      # elements per chunk
IdxT = torch.Tensor                             # packed 12-bit indices, uint8
ValT = torch.Tensor                             # kept values (or their 8-bit codes)
QuantParamsT = tuple[torch.Tensor, float, int, torch.Tensor, torch.dtype]      # shift, scale, offset, lookup, dtype
Q = typing.TypeVar("Q", typing.Literal[True], typing.Literal[False])           # "quantises" flag of a compressor type


# --------------------------------------------------------------------------- #
# 12-bit packing
# --------------------------------------------------------------------------- #
def pack_12bit_indices(indices: torch.Tensor) -> torch.Tensor:
    """Pack an even number of indices (< 4096) into 3 bytes per pair.

    Layout of one pair ``(a, b)``: ``byte0 = a[7:0]``, ``byte1 = a[11:8] | b[3:0] << 4``,
    ``byte2 = b[11:4]``.  Returns a flat ``uint8`` tensor on the input's device.
    """
    flat = indices.reshape(-1)
    n = flat.numel()
    if n % 2 != 0:
        raise ValueError(f"Number of indices must be even, got {n}")
    if n == 0:
        return torch.zeros(0, dtype=torch.uint8, device=indices.device)
    flat = flat.to(torch.int32)
    if int(flat.max()) >= 4096:
        raise ValueError(f"Index {int(flat.max())} exceeds 12-bit limit (4095)")
    if int(flat.min()) < 0:
        raise ValueError("Negative index cannot be packed")
    pairs = flat.view(-1, 2)
    a, b = pairs[:, 0], pairs[:, 1]
    out = torch.stack(
        (a & 0xFF, ((a >> 8) & 0xF) | ((b & 0xF) << 4), (b >> 4) & 0xFF), dim=1
    )
    return out.to(torch.uint8).reshape(-1)


def unpack_12bit_indices(packed: torch.Tensor, values_shape) -> torch.Tensor:
    """Inverse of :func:`pack_12bit_indices`; the result is ``int64`` shaped ``values_shape``."""
    shape = tuple(int(s) for s in values_shape)
    n = int(math.prod(shape)) if len(shape) else 1
    if n == 0:
        return torch.zeros(shape, dtype=torch.int64, device=packed.device)
    if n % 2 != 0:
        raise ValueError(f"Number of indices must be even, got {n}")
    trip = packed.reshape(-1)[: (n // 2) * 3].view(-1, 3).to(torch.int64)
    b0, b1, b2 = trip[:, 0], trip[:, 1], trip[:, 2]
    a = b0 | ((b1 & 0xF) << 8)
    b = ((b1 >> 4) & 0xF) | (b2 << 4)
    return torch.stack((a, b), dim=1).reshape(shape)


# --------------------------------------------------------------------------- #
# chunk geometry and DCT bases
# --------------------------------------------------------------------------- #
def chunk_size_for(n: int, target: int) -> int:
    """Largest divisor of ``n`` that is ``<= target`` (``n`` itself when ``n <= target``)."""
    n = int(n)
    target = int(target)
    if n <= target:
        return n
    for d in range(min(target, n), 0, -1):
        if n % d == 0:
            return d
    return 1


# kept under the reference's private name because neurons and tests call it
_get_smaller_split = chunk_size_for


def dct_basis(n: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Orthonormal DCT-II matrix ``F`` with ``F[k, j] = s_k * cos(pi (2j+1) k / 2n)``.

    ``F @ x`` is the forward transform of a column vector and ``F.T @ X`` its inverse.
    Built in float64 and rounded once so that every consumer (torch path, CUDA
    kernels) sees the same values.
    """
    k = torch.arange(n, dtype=torch.float64).view(-1, 1)
    j = torch.arange(n, dtype=torch.float64).view(1, -1)
    f = torch.cos(math.pi * (2.0 * j + 1.0) * k / (2.0 * n)) * math.sqrt(2.0 / n)
    f[0, :] = math.sqrt(1.0 / n)
    return f.to(dtype=dtype, device=device)


def _dct(x: torch.Tensor, norm: str | None = None) -> torch.Tensor:
    """DCT-II over the last dimension (``norm='ortho'`` or the unnormalised scipy form)."""
    n = x.shape[-1]
    f = dct_basis(n, dtype=torch.float64, device=x.device)
    if norm != "ortho":
        scale = torch.full((n, 1), math.sqrt(n / 2.0) * 2.0, dtype=torch.float64, device=x.device)
        scale[0, 0] = math.sqrt(n) * 2.0
        f = f * scale
    return (x.to(torch.float64) @ f.T).to(x.dtype)


def _idct(x: torch.Tensor, norm: str | None = None) -> torch.Tensor:
    """Inverse of :func:`_dct` over the last dimension."""
    n = x.shape[-1]
    f = dct_basis(n, dtype=torch.float64, device=x.device)
    xs = x.to(torch.float64)
    if norm != "ortho":
        scale = torch.full((n,), math.sqrt(n / 2.0) * 2.0, dtype=torch.float64, device=x.device)
        scale[0] = math.sqrt(n) * 2.0
        xs = xs / scale
    return (xs @ f).to(x.dtype)


class ChunkingTransformer:
    """Splits every parameter into ``<= target_chunk`` sized tiles, optionally DCT-transformed.

    ``shape_dict[s]`` is the tile edge chosen for a dimension of size ``s``;
    ``f_dict[n]`` / ``b_dict[n]`` are the forward / backward bases laid out so that
    ``x @ f_dict[n]`` is the DCT of the rows of ``x`` and ``X @ b_dict[n]`` the inverse.
    """

    @torch.no_grad()
    def __init__(self, model, target_chunk: int, norm: str = "ortho"):
        self.target_chunk = int(target_chunk)
        self.norm = norm
        self.shape_dict: dict[int, int] = {}
        self.f_dict: dict[int, torch.Tensor] = {}
        self.b_dict: dict[int, torch.Tensor] = {}
        if model is None:
            return
        for _, p in model.named_parameters():
            if not p.requires_grad:
                continue
            self.register_shape(p.shape, dtype=p.dtype, device=p.device)

    def register_shape(self, shape, dtype=torch.float32, device=None) -> None:
        for s in shape:
            s = int(s)
            sc = chunk_size_for(s, self.target_chunk)
            self.shape_dict[s] = sc
            if sc not in self.f_dict:
                eye = torch.eye(sc, dtype=torch.float32)
                self.f_dict[sc] = _dct(eye, norm=self.norm).to(dtype).to(device)
                self.b_dict[sc] = _idct(eye, norm=self.norm).to(dtype).to(device)

    def _basis(self, table: dict, n: int, like: torch.Tensor) -> torch.Tensor:
        w = table[n]
        if w.device != like.device or w.dtype != like.dtype:
            w = w.to(device=like.device, dtype=like.dtype)
            table[n] = w
        return w

    @torch.no_grad()
    def einsum_2d(self, x, b, d=None) -> torch.Tensor:
        if d is None:
            return torch.einsum("...ij,jb->...ib", x, b)
        return torch.einsum("...ijkl,kb,ld->...ijbd", x, b, d)

    @torch.no_grad()
    def einsum_2d_t(self, x, b, d=None) -> torch.Tensor:
        if d is None:
            return torch.einsum("...ij,jb->...ib", x, b)
        return torch.einsum("...ijbd,bk,dl->...ijkl", x, b, d)

    @torch.no_grad()
    def encode(self, x: torch.Tensor, *, use_dct: bool = False) -> torch.Tensor:
        if x.dim() > 1:
            n1 = self.shape_dict[x.shape[0]]
            n2 = self.shape_dict[x.shape[1]]
            y = x.reshape(x.shape[0] // n1, n1, x.shape[1] // n2, n2).permute(0, 2, 1, 3)
            if use_dct:
                y = self.einsum_2d(y, self._basis(self.f_dict, n1, x), self._basis(self.f_dict, n2, x))
            return y
        n1 = self.shape_dict[x.shape[0]]
        y = x.reshape(x.shape[0] // n1, n1)
        if use_dct:
            y = self.einsum_2d(y, self._basis(self.f_dict, n1, x))
        return y

    @torch.no_grad()
    def decode(self, x: torch.Tensor, *, use_dct: bool = False) -> torch.Tensor:
        if x.dim() > 2:
            if use_dct:
                n1, n2 = x.shape[2], x.shape[3]
                x = self.einsum_2d_t(x, self._basis(self.b_dict, n1, x), self._basis(self.b_dict, n2, x))
            y, xx, h, w = x.shape
            return x.permute(0, 2, 1, 3).reshape(y * h, xx * w)
        if use_dct:
            x = self.einsum_2d_t(x, self._basis(self.b_dict, x.shape[1], x))
        return x.reshape(-1)


# --------------------------------------------------------------------------- #
# top-k compressor
# --------------------------------------------------------------------------- #
def _to_local(x):
    to_local = getattr(x, "to_local", None)
    return to_local() if callable(to_local) else x


class TopKCompressor(typing.Generic[Q]):      # TopKCompressor[Literal[True]] in annotations: a quantising compressor
    """Per-chunk magnitude top-k with 12-bit packed indices and optional 8-bit values.

    ``compress`` returns ``(idx_u8, val, xshape, totalk)`` or, when quantisation is on,
    ``(idx_u8, val_u8, xshape, totalk, (shift, scale, offset, lookup, dtype))``.
    """

    def __init__(self, *, use_quantization: bool = False, quantization_bins: int = 256,
                 quantization_range: int = 6) -> None:
        self.use_quantization = bool(use_quantization)
        if self.use_quantization:
            self.n_bins = int(quantization_bins)
            self.range_in_sigmas = quantization_range

    @staticmethod
    def _clamp_topk(x, topk) -> int:
        topk = max(min(int(topk), int(x.shape[-1])), 2)
        return int(topk - (topk % 2))

    @torch.no_grad()
    def compress(self, x: torch.Tensor, topk: int):
        x = _to_local(x)
        xshape = x.shape
        if x.dim() > 2:
            x = x.reshape(x.shape[0], x.shape[1], x.shape[2] * x.shape[3])
        totalk = x.shape[-1]
        k = self._clamp_topk(x, topk)
        idx = torch.topk(x.abs(), k=k, dim=-1, largest=True, sorted=False).indices
        val = torch.gather(x, dim=-1, index=idx)
        packed = pack_12bit_indices(idx)
        if self.use_quantization:
            qval, qparams = self._quantize_values(val)
            return packed, qval, xshape, totalk, qparams
        return packed, val, xshape, totalk

    @torch.no_grad()
    def decompress(self, p, idx, val, xshape, totalk, quantize_params=None) -> torch.Tensor:
        if self.use_quantization and quantize_params is not None:
            val = self._dequantize_values(val, quantize_params)
        xshape = tuple(xshape)
        flat_shape = (xshape[0], xshape[1], xshape[2] * xshape[3]) if len(xshape) > 2 else xshape
        x = torch.zeros(flat_shape, device=p.device, dtype=p.dtype)
        if idx.dtype == torch.uint8:
            idx64 = unpack_12bit_indices(idx, val.shape)
        elif idx.dtype == torch.int64:
            idx64 = idx
        else:
            raise ValueError(f"Expected uint8 (packed) or int64 (unpacked) indices, got {idx.dtype}")
        if val.dtype != x.dtype:
            val = val.to(x.dtype)
        # mean over the contributors of each coefficient only; untouched ones stay 0
        x.scatter_reduce_(dim=-1, index=idx64.to(x.device), src=val.to(x.device),
                          reduce="mean", include_self=False)
        return x.reshape(xshape)

    @torch.no_grad()
    def batch_decompress(self, p, idx, val, xshape, totalk, quantize_params=None, *,
                         block_norms: torch.Tensor | None = None, normalise: bool = False,
                         clip_norm: bool = True) -> torch.Tensor:
        idx_list = list(idx) if isinstance(idx, (list, tuple)) else [idx]
        val_list = list(val) if isinstance(val, (list, tuple)) else [val]
        if quantize_params is not None and not isinstance(quantize_params, list):
            quantize_params = [quantize_params] * len(val_list)
        vals = val_list
        if self.use_quantization and quantize_params:
            vals = [self._dequantize_values(v, quantize_params[i]) for i, v in enumerate(val_list)]
        norms = median = None
        if clip_norm:
            norms = (block_norms.to(p.device) if block_norms is not None
                     else torch.stack([torch.linalg.vector_norm(v.float()) for v in vals]))
            median = torch.median(norms)
        processed = []
        for i, v in enumerate(vals):
            v = v.to(p.device)
            if normalise:
                if v.dim() >= 2:
                    v = v / (torch.linalg.vector_norm(v, dim=-1, keepdim=True) + 1e-8)
                else:
                    n = torch.linalg.vector_norm(v)
                    v = v / n if n > 1e-8 else v
            elif clip_norm:
                v = v * torch.clamp(median / (norms[i] + 1e-8), max=1)
            processed.append(v)
        unpacked = []
        for i, packed in enumerate(idx_list):
            if packed.dtype != torch.uint8:
                raise ValueError(f"Expected uint8 for 12-bit packed indices, got {packed.dtype}")
            unpacked.append(unpack_12bit_indices(packed.to(p.device), val_list[i].shape))
        return self.decompress(p, torch.cat(unpacked, dim=-1),
                               torch.cat(processed, dim=-1).to(p.dtype), xshape, totalk, None)

    # -- 8-bit value quantisation ------------------------------------------- #
    @torch.no_grad()
    def _quantize_values(self, val: torch.Tensor):
        offset = self.n_bins // 2
        shift = val.mean()
        centered = (val - shift).to(torch.float32)
        std = torch.linalg.vector_norm(centered) / math.sqrt(max(centered.numel() - 1, 1))
        scale = self.range_in_sigmas * std / self.n_bins
        if not bool(torch.isfinite(scale)) or float(scale) == 0.0:
            scale = torch.ones((), dtype=torch.float32, device=val.device)
        q = (centered / scale + offset).round().clamp(0, self.n_bins - 1).to(torch.uint8)
        flat_q = q.reshape(-1).long()
        sums = torch.zeros(self.n_bins, dtype=torch.float32, device=val.device)
        cnts = torch.zeros(self.n_bins, dtype=torch.float32, device=val.device)
        sums.scatter_add_(0, flat_q, centered.reshape(-1))
        cnts.scatter_add_(0, flat_q, torch.ones_like(centered.reshape(-1)))
        lookup = torch.where(cnts > 0, sums / cnts.clamp(min=1), torch.zeros_like(sums))
        return q, (shift, float(scale), offset, lookup, val.dtype)

    @torch.no_grad()
    def _dequantize_values(self, val: torch.Tensor, qparams) -> torch.Tensor:
        if val.dtype != torch.uint8:
            return val
        shift, _, _, lookup, orig_dtype = qparams
        if isinstance(lookup, torch.Tensor):
            lookup = lookup.to(val.device)
        if isinstance(shift, torch.Tensor):
            shift = shift.to(val.device)
        return (lookup[val.long()] + shift).to(orig_dtype)

    def maybe_dequantize_values(self, vals, qparams, device) -> list[torch.Tensor]:
        if not isinstance(vals, (list, tuple)):
            vals = [vals]
        if qparams is None or not all(v.dtype == torch.uint8 for v in vals):
            return list(vals)
        if isinstance(qparams, tuple) and len(qparams) == 5 and not all(
            isinstance(q, (tuple, list)) and len(q) == 5 for q in qparams
        ):
            qparams = [qparams]
        if not isinstance(qparams, list):
            qparams = [qparams]
        out = []
        for i, v in enumerate(vals):
            v = v.to(device)
            if v.dtype == torch.uint8:
                if i >= len(qparams) or qparams[i] is None:
                    break
                v = self._dequantize_values(v, qparams[i]).to(device)
            out.append(v)
        if len(out) != len(vals):
            raise IndexError(f"Mismatch in val lengths: dequant({len(out)}) vs original({len(vals)})")
        return out
