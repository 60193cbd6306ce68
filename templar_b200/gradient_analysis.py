"""Collect the compressed gradients that peers uploaded for a window and compare them.

    python -m templar_b200.gradient_analysis --uids 1 2 3 --window 1234 [--hparams-dir hparams] [--device cuda] [--json out.json]

For every uid whose ``gradient`` object of the window can be read (any store the environment selects, see
:func:`templar_b200.comms.default_store`): the payload is checked like a gathered one, its 12-bit indices are unpacked,
its 8-bit values dequantised, and the dense pseudo-gradient is rebuilt per tensor (scatter of the top-k coefficients,
inverse chunk DCT).  Reported per uid: L2 norm of the whole pseudo-gradient, number of transmitted coefficients, how
many of its (tensor, chunk, index) positions no other collected peer also sent; and the matrix of cosine similarities
between the peers' dense pseudo-gradients with each peer's mean / min / max similarity to the others.

Counterparts in the reference: scripts/analyser.py (norms, index statistics, peer cosine similarity of decoded
gradients) and scripts/collector.py (fetching the gradient objects of a window).
"""

from __future__ import annotations

import argparse
import asyncio
import json
from types import SimpleNamespace

import torch

from . import compress as C


def decode_payload(state: dict, model: torch.nn.Module, transformer, compressor, xshapes: dict, totalks: dict, *,
                   use_dct: bool, device="cpu") -> dict[str, torch.Tensor]:
    """Dense pseudo-gradient per tensor from one peer's payload (``<name>idxs`` / ``<name>vals`` /
    ``<name>quant_params`` entries).  Tensors that the payload does not carry are left out."""
    out = {}
    for name, p in model.named_parameters():
        idxs, vals = state.get(name + "idxs"), state.get(name + "vals")
        if idxs is None or vals is None:
            continue
        qp = state.get(name + "quant_params")
        idxs, vals = idxs.to(device), vals.to(device)
        vals_f = compressor.maybe_dequantize_values([vals], [qp] if qp is not None else None, device)[0]
        ref = torch.empty(p.shape, device=device, dtype=torch.float32)
        dense = compressor.decompress(ref, idxs, vals_f, xshapes[name], totalks[name])
        out[name] = transformer.decode(dense, use_dct=use_dct).float()
    return out


def index_positions(state: dict, names) -> set:
    """(tensor, chunk, coefficient) positions a payload transmits."""
    pos = set()
    for t, name in enumerate(names):
        idxs, vals = state.get(name + "idxs"), state.get(name + "vals")
        if idxs is None or vals is None:
            continue
        un = C.unpack_12bit_indices(idxs.cpu(), vals.shape).reshape(-1, vals.shape[-1])
        for chunk, row in enumerate(un.tolist()):
            pos.update((t, chunk, i) for i in row)
    return pos


def analyse(payloads: dict[int, dict], model: torch.nn.Module, *, topk: int, target_chunk: int = 64, use_dct: bool = True,
            device="cpu") -> dict:
    """Statistics of a set of peers' payloads (uid -> payload dict); see the module docstring."""
    transformer = C.ChunkingTransformer(model, target_chunk)
    compressor = C.TopKCompressor(use_quantization=False)
    xshapes, totalks = {}, {}
    names = [n for n, _ in model.named_parameters()]
    for n, p in model.named_parameters():
        enc = transformer.encode(torch.zeros(p.shape, device=device), use_dct=False)
        _, _, xshapes[n], totalks[n] = compressor.compress(enc, topk)[:4]
    uids = sorted(payloads)
    flat, positions, per_uid = {}, {}, {}
    for u in uids:
        dense = decode_payload(payloads[u], model, transformer, compressor, xshapes, totalks, use_dct=use_dct, device=device)
        flat[u] = torch.cat([dense[n].reshape(-1) if n in dense else torch.zeros(p.numel(), device=device)
                             for n, p in model.named_parameters()])
        positions[u] = index_positions(payloads[u], names)
        per_uid[u] = {"gradient_norm": float(flat[u].norm()), "coefficients": len(positions[u]),
                      "tensors": sum(1 for n in names if n + "vals" in payloads[u])}
    n = len(uids)
    sim = torch.eye(n)
    for i in range(n):
        for j in range(i + 1, n):
            a, b = flat[uids[i]], flat[uids[j]]
            sim[i, j] = sim[j, i] = float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))
    for i, u in enumerate(uids):
        others = [positions[v] for v in uids if v != u]
        shared = set().union(*others) if others else set()
        per_uid[u]["unique_position_ratio"] = (len(positions[u] - shared) / len(positions[u])) if positions[u] else 0.0
        if n > 1:
            row = torch.cat((sim[i, :i], sim[i, i + 1:]))
            per_uid[u].update(mean_peer_similarity=float(row.mean()), min_peer_similarity=float(row.min()),
                              max_peer_similarity=float(row.max()))
    return {"uids": uids, "per_uid": per_uid, "cosine_similarity": sim.tolist()}


async def collect(comms, uids, window: int, *, timeout: int = 30) -> dict[int, dict]:
    """The ``gradient`` objects of ``window`` that can be read from the uids' buckets (uid -> payload)."""
    async def one(u):
        res = await comms.get_with_retry(uid=str(u), window=window, key="gradient", timeout=timeout, local=False,
                                         stale_retention=10)
        data = getattr(res, "data", None) if res is not None else None
        return u, data if isinstance(data, dict) else None
    got = await asyncio.gather(*(one(u) for u in uids))
    return {u: d for u, d in got if d is not None and not (d.get("metadata") or {}).get("dummy")}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--uids", type=int, nargs="+", required=True)
    ap.add_argument("--window", type=int, required=True)
    ap.add_argument("--hparams-dir", default="hparams", help="directory of hparams.json (model shapes, top-k, chunk size)")
    ap.add_argument("--my-uid", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    from . import model_factory
    from .backends.chain import StaticWallet
    from .comms import Comms
    from .hparams import load_hparams

    hp = load_hparams(a.hparams_dir)
    model = model_factory.create_meta_model(hp, role="evaluator", world_size=1)
    comms = Comms(wallet=StaticWallet(f"hotkey-{a.my_uid}"), uid=a.my_uid, hparams=hp)
    payloads = asyncio.run(collect(comms, a.uids, a.window))
    if not payloads:
        raise SystemExit(f"no gradient of window {a.window} could be read for uids {a.uids}")
    shapes = SimpleNamespace(named_parameters=lambda: [(n, torch.empty(p.shape, device="meta")) for n, p in model.named_parameters()])
    rep = analyse(payloads, shapes, topk=int(getattr(hp, "topk_compression", 32)),
                  target_chunk=int(getattr(hp, "target_chunk", 64)), use_dct=bool(getattr(hp, "use_dct", False)), device=a.device)
    print(json.dumps(rep["per_uid"], indent=1))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rep, f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
