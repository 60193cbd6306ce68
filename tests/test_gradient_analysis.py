"""Gradient collection and comparison tool: norms, index statistics and peer cosine similarity of decoded payloads."""

import asyncio
from types import SimpleNamespace

import torch

import templar_b200 as tplr
from templar_b200 import compress as C
from templar_b200 import gradient_analysis as GA
from templar_b200.backends.chain import StaticChain, StaticWallet
from templar_b200.backends.store import MemoryStore


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Parameter(torch.zeros(128, 64))
        self.b = torch.nn.Parameter(torch.zeros(64))


def _payload(model, grads, topk, quantize=False):
    tr = C.ChunkingTransformer(model, 64)
    comp = C.TopKCompressor(use_quantization=quantize, quantization_bins=256, quantization_range=6)
    out = {}
    for n, _ in model.named_parameters():
        res = comp.compress(tr.encode(grads[n], use_dct=True), topk)
        out[n + "idxs"], out[n + "vals"] = res[0], res[1]
        out[n + "quant_params"] = res[4] if len(res) > 4 else None
    return out


def test_statistics_of_three_peers_two_of_them_nearly_equal():
    m = Tiny()
    g = torch.Generator().manual_seed(0)
    base = {n: torch.randn(p.shape, generator=g) for n, p in m.named_parameters()}
    other = {n: torch.randn(p.shape, generator=g) for n, p in m.named_parameters()}
    near = {n: v * 2.0 for n, v in base.items()}                       # same direction, twice the length
    payloads = {3: _payload(m, base, 8), 5: _payload(m, near, 8, quantize=True), 9: _payload(m, other, 8)}
    rep = GA.analyse(payloads, m, topk=8, use_dct=True)
    assert rep["uids"] == [3, 5, 9]
    sim = torch.tensor(rep["cosine_similarity"])
    assert sim[0, 1] > 0.98 and abs(sim[0, 2]) < 0.5 and torch.allclose(sim, sim.t()) and torch.allclose(sim.diag(), torch.ones(3))
    u3, u5, u9 = (rep["per_uid"][u] for u in (3, 5, 9))
    assert abs(u5["gradient_norm"] / u3["gradient_norm"] - 2.0) < 0.1          # 8-bit values: within the code width
    # dense norm of the top-k approximation: below the full gradient's, well above zero
    full = torch.cat([v.reshape(-1) for v in base.values()]).norm().item()
    assert 0.05 * full < u3["gradient_norm"] < full
    assert u3["coefficients"] == u9["coefficients"] == 2 * 8 + 1 * 8            # (128 x 64) is two chunks, the vector one
    # peers 3 and 5 picked the same positions (scaled copies): nothing of 3 is unique; peer 9 shares few
    assert u3["unique_position_ratio"] == 0.0 and u9["unique_position_ratio"] > 0.5
    assert u3["max_peer_similarity"] > 0.98 and u9["mean_peer_similarity"] < 0.5


def test_collect_reads_the_window_objects_of_the_peers_that_uploaded():
    store, chain = MemoryStore(), StaticChain(n=4, manual=True)
    hp = SimpleNamespace(topk_compression=8, blocks_per_window=4, recent_windows=2, active_check_interval=1)
    comms = {}
    for u in range(3):
        c = tplr.Comms(wallet=StaticWallet(f"hotkey-{u}"), config=SimpleNamespace(netuid=3, device="cpu"), hparams=hp, uid=u,
                       store=store, subtensor=chain)
        c.try_commit(c.wallet, c.bucket)
        comms[u] = c
    m = Tiny()
    g = torch.Generator().manual_seed(1)

    async def go():
        for c in comms.values():
            c.commitments = await c.get_commitments()
        for u in (1, 2):
            grads = {n: torch.randn(p.shape, generator=g) for n, p in m.named_parameters()}
            await comms[u].put(_payload(m, grads, 8), window=7, key="gradient", uid=str(u), global_step=1, local=False)
        return await GA.collect(comms[0], [1, 2, 3], 7, timeout=2)

    got = asyncio.run(go())
    assert sorted(got) == [1, 2]
    rep = GA.analyse(got, m, topk=8, use_dct=True)
    assert rep["uids"] == [1, 2] and all(v["gradient_norm"] > 0 for v in rep["per_uid"].values())
