"""Seeded synthetic data for benchmarks and tests (there is no dataset or peer network offline)."""

from __future__ import annotations

import torch

from ..compress import pack_12bit_indices


@torch.no_grad()
def synthetic_payload(layout, seed: int, device="cpu", scale: float = 1e-3, val_dtype=torch.float32):
    """A full-model peer payload in ``layout``'s flat wire format: (packed indices uint8, values).

    Every chunk gets ``k`` distinct coefficient indices (an arithmetic progression with a random
    start and odd stride modulo the chunk size) and N(0, scale) values.
    """
    g = torch.Generator(device=device).manual_seed(seed)
    idx = torch.zeros(layout.idx_bytes, dtype=torch.uint8, device=device)
    val = torch.zeros(layout.val_elems, dtype=val_dtype, device=device)
    for s in layout.specs:
        k = s.topk(layout.topk)
        n, tk = s.n_chunks, s.totalk
        start = torch.randint(0, tk, (n, 1), generator=g, device=device)
        pow2 = tk & (tk - 1) == 0
        stride = (torch.randint(0, max(tk // 2, 1), (n, 1), generator=g, device=device) * 2 + 1) if pow2 else 1
        sel = (start + stride * torch.arange(k, device=device).view(1, k)) % tk
        io, vo = layout.idx_off[s.name], layout.val_off[s.name]
        idx[io: io + n * (k // 2) * 3] = pack_12bit_indices(sel)
        val[vo: vo + n * k] = (torch.randn(n * k, generator=g, device=device) * scale).to(val_dtype)
    return idx, val


def synthetic_tokens(batch: int, seq_len: int, vocab: int, seed: int, pin: bool = False):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, vocab, (batch, seq_len), generator=g)
    return t.pin_memory() if pin else t
