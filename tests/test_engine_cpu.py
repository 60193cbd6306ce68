"""CPU checks of engine-level helpers that have a GPU fast path elsewhere."""

import torch

from templar_b200 import compress as C
from templar_b200.models.llama import ModelArgs, build_model
from templar_b200.parallel.tensor_parallel import TensorParallel
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine


def _engine():
    args = ModelArgs(dim=128, n_layers=1, n_heads=2, vocab_size=256, intermediate_size=256, max_seq_len=32)
    model = build_model(args, device="cpu", dtype=torch.float32, seed=2)
    eng = WindowEngine(model, EngineConfig(topk=8), device="cpu")
    eng.snapshot()
    eng.store.master_shard.add_(torch.randn_like(eng.store.master_shard) * 1e-3)
    eng.compress()
    return eng


def test_own_payload_quantised_roundtrip():
    """own_payload(quantize=True) is the reference wire format: uint8 codes whose lookup decodes to within one bin."""
    eng = _engine()
    plain, quant = eng.own_payload(), eng.own_payload(quantize=True)
    comp = C.TopKCompressor(use_quantization=True)
    assert set(plain) == set(quant)
    for s in eng.layout.specs:
        q, qp = quant[s.name + "vals"], quant[s.name + "quant_params"]
        assert q.dtype == torch.uint8 and q.shape == plain[s.name + "vals"].shape
        assert torch.equal(quant[s.name + "idxs"], plain[s.name + "idxs"])
        deq = comp._dequantize_values(q, qp)
        err = (deq - plain[s.name + "vals"].float()).abs().max()
        assert float(err) <= 1.01 * qp[1] * 128 + 1e-9
        inner = (q > 0) & (q < 255)                          # values not clamped to the outer bins
        if inner.any():
            assert float((deq - plain[s.name + "vals"].float()).abs()[inner].max()) <= 1.01 * qp[1]


def test_quantised_peer_payload_is_decoded_when_staged():
    """A peer that sends 8-bit codes (the reference miner's default) lands in the slot as decoded values,
    through the single-payload path and through the per-peer slice of a gathered state dict."""
    from templar_b200.parallel.window_engine import peer_slice

    eng = _engine()
    plain, quant = eng.own_payload(), eng.own_payload(quantize=True)
    gathered = {k: [v, v] for k, v in quant.items()}
    eng.load_peer_payload(0, peer_slice(gathered, 1), non_blocking=False)
    _, val = eng.pack_payload(quant)
    for s in eng.layout.specs:
        _, slot_val = eng.layout.payload_views(eng.peer_idx[0], eng.peer_val[0], s.name)
        _, packed_val = eng.layout.payload_views(eng.peer_idx[0], val, s.name)
        ref = plain[s.name + "vals"].float().reshape(slot_val.shape)
        tol = 1.01 * float(quant[s.name + "quant_params"][1]) * 128 + 1e-6
        assert float((slot_val.float() - ref).abs().max()) <= tol
        assert torch.equal(packed_val, slot_val)
    bad = {k: v for k, v in quant.items() if not k.endswith("quant_params")}
    try:
        eng.load_peer_payload(0, bad)
        raise AssertionError("8-bit codes without parameters must be refused")
    except ValueError:
        pass


def test_gather_cta_budget_grows_with_link_pressure():
    """More copier CTA pairs when the peers' rows must arrive faster; bounded by the link; idle pairs are used."""
    tp = TensorParallel.__new__(TensorParallel)
    tp.n_comm_pairs, tp.world = None, 8
    small = tp._comm_pairs(2.0 * 8192 * 28672 * 8192, 7 * 1024 * 8192 * 2, 4096)       # compute-heavy
    large = tp._comm_pairs(2.0 * 8192 * 1024 * 8192, 7 * 1024 * 8192 * 2, 128 * 4)     # communication-heavy
    tiny = tp._comm_pairs(2.0 * 2048 * 3584 * 8192, 7 * 256 * 8192 * 2, 8 * 14)        # two waves: idle pairs copy
    assert 1 <= small <= large <= 8
    assert tiny >= large
    tp.n_comm_pairs = 3
    assert tp._comm_pairs(1.0, 1.0, 1) == 3
    tp.n_comm_pairs, tp.world = None, 1
    assert tp._comm_pairs(1e12, 0.0, 100) == 1


def _decode_own(eng):
    """Dense decode of the engine's own payload, flat in the layout's element order."""
    L = eng.layout
    tr = C.ChunkingTransformer(None, eng.cfg.target_chunk)
    comp = C.TopKCompressor(use_quantization=False)
    out = torch.zeros(L.total, dtype=torch.float32)
    for s in L.specs:
        shape = tuple(s.shape) if len(s.shape) >= 2 else (s.cols,)
        tr.register_shape(shape)
        idx, val = L.payload_views(eng.own_idx.cpu(), eng.own_val.float().cpu(), s.name)
        dense = comp.decompress(torch.zeros(shape), idx, val, L.xshape(s.name), s.totalk)
        out[s.offset: s.offset + s.numel] = tr.decode(dense, use_dct=eng.cfg.use_dct).reshape(-1)
    return out


def quantised_window_identity(device):
    """With ``quantize`` the payload holds what a receiver decodes and the error feedback keeps the rest:
    ef_new + decode(payload) == momentum * ef_old + (theta0 - theta), and own_payload() returns the codes."""
    args = ModelArgs(dim=128, n_layers=1, n_heads=2, vocab_size=256, intermediate_size=256, max_seq_len=32)
    model = build_model(args, device=device, dtype=torch.float32 if device == "cpu" else torch.bfloat16, seed=2)
    eng = WindowEngine(model, EngineConfig(topk=8, quantize=True, quant_bins=16), device=device)
    g = torch.Generator().manual_seed(5)
    eng.ef.copy_(torch.randn(eng.ef.shape, generator=g) * 1e-3)
    ef_old = eng.ef.clone()
    eng.snapshot()
    eng.store.master_shard.add_((torch.randn(eng.ef.shape, generator=g) * 1e-3).to(eng.store.master_shard.device))
    x = (eng.cfg.momentum_decay * ef_old + (eng.theta0 - eng.store.master_shard)).float().cpu()
    eng.compress()
    sent = _decode_own(eng)
    assert float((eng.ef.float().cpu() + sent - x).abs().max()) < 2e-6
    pl = eng.own_payload()
    comp = C.TopKCompressor(use_quantization=True, quantization_bins=16)
    n_codes = 0
    for s in eng.layout.specs:
        q, qp = pl[s.name + "vals"], pl[s.name + "quant_params"]
        assert q.dtype == torch.uint8 and int(q.max()) < 16
        _, val = eng.layout.payload_views(eng.own_idx, eng.own_val, s.name)
        assert torch.allclose(comp._dequantize_values(q.cpu(), tuple(t.cpu() if torch.is_tensor(t) else t for t in qp)),
                              val.float().cpu().reshape(q.shape), atol=1e-7)
        n_codes += len(torch.unique(q))
    assert n_codes > len(eng.layout.specs)             # the codes are not all one bin
    # the flat quantised form (indices, codes, tables) staged as a peer decodes to the same values
    eng.load_peer_payload(0, (eng.own_idx, eng._q_codes, eng._q_table), non_blocking=False)
    assert torch.allclose(eng.peer_val[0].float(), eng.own_val.float(), atol=1e-7)
    # the quantisation error is in the buffer: it differs from the exact-value residual
    exact = WindowEngine(build_model(args, device=device, dtype=model.tok_embeddings.weight.dtype, seed=2),
                         EngineConfig(topk=8), device=device)
    exact.ef.copy_(ef_old)
    exact.theta0.copy_(eng.theta0)
    exact.store.master_shard.copy_(eng.store.master_shard)
    exact.window_open = True
    exact.compress()
    assert torch.equal(exact.own_idx.cpu(), eng.own_idx.cpu())
    assert float((exact.ef - eng.ef).abs().max()) > 1e-7
    return eng


def test_quantised_window_identity_cpu():
    quantised_window_identity("cpu")
