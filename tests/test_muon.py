"""Muon: Newton-Schulz orthogonalisation, the single-device optimizer with auxiliary Adam, the sharded variant."""

import json
import os
import subprocess
import sys

import pytest
import torch

from templar_b200.muon import (Muon, SingleDeviceMuonWithAuxAdam, adam_update, muon_update, newton_schulz,
                               zeropower_via_newtonschulz5)
from templar_b200.muon.newton_schulz import NS_CONSTS

HERE = os.path.dirname(os.path.abspath(__file__))


def _ns_reference(G: torch.Tensor) -> torch.Tensor:
    """The same five quintic iterations in fp32 matmuls."""
    X = G.float()
    t = X.size(-2) > X.size(-1)
    if t:
        X = X.mT
    X = X / (X.norm() + 1e-7)
    for a, b, c in NS_CONSTS:
        A = X @ X.mT
        X = a * X + (b * A + c * A @ A) @ X
    return X.mT if t else X


@pytest.mark.parametrize("shape", [(64, 64), (128, 64), (64, 192), (3, 64, 128)])
def test_newton_schulz_pushes_singular_values_to_one(shape):
    torch.manual_seed(0)
    G = torch.randn(*shape)
    X = newton_schulz(G).float()
    assert X.shape == G.shape
    sv = torch.linalg.svdvals(X)
    # all but the near-singular directions of a random matrix end close to 1
    assert float(sv.max()) < 1.3 and 0.9 < float(sv.median()) < 1.1 and float((sv > 0.5).float().mean()) > 0.9
    flatG, flatX = G.reshape(-1, *shape[-2:]), X.reshape(-1, *shape[-2:])
    for g, x in zip(flatG, flatX):
        U, _, Vh = torch.linalg.svd(g, full_matrices=False)
        polar = U @ Vh
        assert float((x * polar).sum() / (x.norm() * polar.norm())) > 0.95      # aligned with U V^T
        ref = _ns_reference(g)
        assert float((x - ref).norm() / ref.norm()) < 3e-2                      # bf16 operands vs fp32 matmuls


def test_fixed_coefficient_variant_and_errors():
    torch.manual_seed(1)
    G = torch.randn(48, 96)
    sv = torch.linalg.svdvals(zeropower_via_newtonschulz5(G).float())
    assert float(sv.max()) < 1.3 and float(sv.min()) > 0.3                   # 48 x 96: well conditioned
    with pytest.raises(ValueError):
        newton_schulz(torch.randn(7))


@pytest.mark.parametrize("nesterov,rms", [(True, False), (False, False), (True, True)])
def test_muon_update_formula(nesterov, rms):
    torch.manual_seed(2)
    g, m = torch.randn(96, 32), torch.randn(96, 32) * 0.1
    g0, m0 = g.clone(), m.clone()
    upd = muon_update(g, m, beta=0.9, nesterov=nesterov, rms_scale=rms)
    m_ref = m0 + (g0 - m0) * 0.1
    assert torch.allclose(m, m_ref, atol=1e-6)
    direction = g0 + (m_ref - g0) * 0.9 if nesterov else m_ref
    scale = 0.2 * 96 ** 0.5 if rms else (96 / 32) ** 0.5
    want = newton_schulz(direction).float() * scale
    assert torch.allclose(upd.float(), want, atol=1e-5)
    g4, m4 = torch.randn(8, 4, 3, 3), torch.zeros(8, 4, 3, 3)              # conv-style weights are flattened
    assert muon_update(g4, m4).shape == (8, 36)


def test_adam_update_matches_torch_adamw():
    torch.manual_seed(3)
    p = torch.nn.Parameter(torch.randn(10, 6))
    q = torch.nn.Parameter(p.detach().clone())
    ours = SingleDeviceMuonWithAuxAdam([dict(params=[p], use_muon=False, lr=1e-2, betas=(0.9, 0.95), eps=1e-10,
                                             weight_decay=0.1)])
    ref = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-10, weight_decay=0.1)
    for _ in range(3):
        g = torch.randn(10, 6)
        p.grad, q.grad = g.clone(), g.clone()
        ours.step()
        ref.step()
    assert torch.allclose(p, q, atol=1e-6)
    b1, b2 = torch.zeros(3), torch.zeros(3)
    u = adam_update(torch.ones(3), b1, b2, 1, (0.9, 0.95), 1e-10)
    assert torch.allclose(u, torch.ones(3), atol=1e-6)                       # bias-corrected first step


def test_single_device_muon_step_and_defaults():
    torch.manual_seed(4)
    w = torch.nn.Parameter(torch.randn(64, 32))
    b = torch.nn.Parameter(torch.randn(32))
    opt = SingleDeviceMuonWithAuxAdam([dict(params=[w], use_muon=True, lr=0.05, weight_decay=0.01),
                                       dict(params=[b], use_muon=False)])
    assert opt.param_groups[0]["momentum"] == 0.95 and opt.param_groups[1]["lr"] == 3e-4
    w0, g = w.detach().clone(), torch.randn(64, 32)
    w.grad, b.grad = g.clone(), torch.randn(32)
    loss = opt.step(lambda: torch.tensor(1.5))
    assert float(loss) == 1.5
    want = w0 * (1 - 0.05 * 0.01) - 0.05 * muon_update(g.clone(), torch.zeros(64, 32), beta=0.95)
    assert torch.allclose(w.detach(), want, atol=1e-5)
    with pytest.raises(AssertionError):
        SingleDeviceMuonWithAuxAdam([dict(params=[w])])


def test_sharded_muon_on_plain_tensors_equals_local_formula():
    """Without DTensor parameters the sharded class takes the single-device path (with its own defaults)."""
    torch.manual_seed(5)
    w = torch.nn.Parameter(torch.randn(32, 64))
    opt = Muon([dict(params=[w], use_muon=True, lr=0.02)])
    assert opt.param_groups[0]["rms_scale"] and opt.param_groups[0]["nesterov"]
    w0, g = w.detach().clone(), torch.randn(32, 64)
    w.grad = g.clone()
    opt.step()
    want = w0 - 0.02 * muon_update(g.clone(), torch.zeros(32, 64), 0.95, True, True)
    assert torch.allclose(w.detach(), want, atol=1e-5)


def test_sharded_muon_two_ranks_gloo():
    """dim-0 sharded DTensor parameters over 2 gloo ranks: same weights as the full-matrix update on one rank."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29647", os.path.join(HERE, "_gloo_muon_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, r.stdout[-2000:] + r.stderr[-4000:]
    for res in json.loads(lines[-1][7:]):
        assert res["max_diff"] < 1e-5, res
        assert res["moved"] > 1e-3, res
        assert res["aux_diff"] < 1e-6, res
        # sharded window engine with Muon: same master weights as one rank, up to bf16 rounding flips in Newton-Schulz
        assert res["engine_exact_frac"] > 0.9 and res["engine_max_diff"] < 2e-3, res
        assert res["engine_compute_diff"] < 2e-3 and res["engine_moved"] > 1e-3, res


@pytest.mark.gpu
def test_newton_schulz_on_own_gemm_matches_fp32_iterations():
    from templar_b200.ops import functional as OF

    torch.manual_seed(6)
    for shape in [(256, 256), (512, 256), (256, 1024)]:
        G = torch.randn(*shape, device="cuda")
        X = newton_schulz(G).float()
        ref = _ns_reference(G)
        assert float((X - ref).norm() / ref.norm()) < 4e-2
        sv = torch.linalg.svdvals(X)
        assert float(sv.max()) < 1.3 and 0.9 < float(sv.median()) < 1.1
    assert int(OF.status_word(torch.device("cuda")).item()) == 0


@pytest.mark.gpu
def test_one_triangle_products_match_full_products_and_fp32():
    """Lines 1 and 2 of the iteration as one-triangle products (tiles on or above the diagonal + mirror kernel)
    against the same kernel computing every tile, and against fp32 iterations; sizes with several 256-tiles per
    side, one that is not a multiple of 256, and both orientations."""
    import importlib

    from templar_b200.ops import functional as OF
    from templar_b200.ops import native

    ns = importlib.import_module("templar_b200.muon.newton_schulz")
    torch.manual_seed(8)
    # the triangle product and the mirror by themselves, bit for bit against the full product
    for M, K in ((1024, 512), (768, 2048), (520, 264)):
        x = (torch.randn(M, K, device="cuda") * 0.05).to(torch.bfloat16)
        full = OF.gemm(x, x)
        u = torch.full((M, M), float("nan"), dtype=torch.bfloat16, device="cuda")
        out = torch.empty_like(u)
        L, st = native.lib(), OF.status_word(torch.device("cuda")).data_ptr()
        native.check(L.tplr_gemm2_syrk(x.data_ptr(), u.data_ptr(), M, K, K, M, st, native.stream_ptr()), "syrk")
        native.check(L.tplr_sym_axpby(u.data_ptr(), M, M, 1.0, None, 0, 0.0, 0.0, out.data_ptr(), M, native.stream_ptr()), "sym")
        assert torch.equal(out.triu(256), full.triu(256))                 # tiles above the diagonal: the same numbers
        assert torch.equal(out, out.t()) and torch.isfinite(out.float()).all()
        assert (out.float() - full.float()).abs().max().item() <= 2 ** -7 * full.float().abs().max().item()
        aux = torch.randn_like(out)
        native.check(L.tplr_sym_axpby(u.data_ptr(), M, M, 0.5, aux.data_ptr(), M, -2.0, 3.0, out.data_ptr(), M,
                                      native.stream_ptr()), "sym")
        want = (0.5 * torch.where(torch.ones(M, M, device="cuda").triu().bool(), full.float(), full.float().t())
                - 2.0 * aux.float() + 3.0 * torch.eye(M, device="cuda"))
        assert (out.float() - want).abs().max().item() < 0.05 * max(want.abs().max().item(), 1.0)
    for shape in [(1024, 1024), (768, 2048), (2048, 512), (520, 1032)]:
        G = torch.randn(*shape, device="cuda")
        ns.SYMMETRIC_PRODUCTS = True
        X = newton_schulz(G).float()
        ns.SYMMETRIC_PRODUCTS = False
        try:
            F = newton_schulz(G).float()
        finally:
            ns.SYMMETRIC_PRODUCTS = True
        ref = _ns_reference(G)
        assert float((X - F).norm() / F.norm()) < 2e-2
        assert float((X - ref).norm() / ref.norm()) < 4e-2
        sv = torch.linalg.svdvals(X)
        assert float(sv.max()) < 1.3 and 0.9 < float(sv.median()) < 1.1
    assert int(OF.status_word(torch.device("cuda")).item()) == 0


def test_engine_muon_step_equals_single_device_muon_with_aux_adam():
    """The window engine's Muon inner step (flat fp32 state) against the optimizer class on the module tree,
    with the groups, LR scales and decays the trainer builds for ``optimizer.type == "muon"``."""
    from templar_b200.models.llama import ModelArgs, build_model
    from templar_b200.parallel.window_engine import EngineConfig, WindowEngine

    args = ModelArgs(dim=64, n_layers=2, n_heads=2, vocab_size=128, intermediate_size=128, max_seq_len=32)
    torch.manual_seed(0)
    toks = torch.randint(0, 128, (2, 2, 33))
    m1 = build_model(args, seed=3)
    eng = WindowEngine(m1, EngineConfig(inner_optimizer="muon", inner_lr=0.02, muon_momentum=0.9, muon_weight_decay=0.01,
                                        weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8, max_grad_norm=1.0))
    m2 = build_model(args, seed=3)
    groups = {"head": [], "embed": [], "scalar": [], "muon": []}
    for n, p in m2.named_parameters():
        groups[WindowEngine.muon_class(n, p.ndim)].append(p)
    assert groups["muon"] and groups["embed"] and groups["head"] and groups["scalar"]
    opt = SingleDeviceMuonWithAuxAdam(
        [dict(params=groups[k], lr=0.02 * sc, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8, use_muon=False)
         for k, sc in (("head", 0.5), ("embed", 0.5), ("scalar", 0.2))]
        + [dict(params=groups["muon"], lr=0.02, momentum=0.9, weight_decay=0.01, use_muon=True)])
    for step in range(2):
        t = toks[step]
        eng.micro_step(t[:, :-1], t[:, 1:], 1.0)
        eng.optimizer_step(lr=0.02)
        opt.zero_grad(set_to_none=True)
        m2.loss(t[:, :-1], t[:, 1:]).backward()
        torch.nn.utils.clip_grad_norm_(m2.parameters(), 1.0)
        opt.step()
    diffs = [float((p.detach() - dict(m1.named_parameters())[n].detach()).abs().max()) for n, p in m2.named_parameters()]
    # identical arithmetic; a last-bit difference in a gradient can flip a bf16 rounding inside Newton-Schulz,
    # which moves single entries of one matrix by about lr * 1e-2
    assert sum(d < 1e-6 for d in diffs) >= len(diffs) - 2 and max(diffs) < 1e-3, diffs
    assert float(eng.store.grad.abs().max()) == 0.0


def test_trainer_maps_muon_hparams_to_the_engine():
    from types import SimpleNamespace

    from neurons.trainer import Trainer

    t = Trainer.__new__(Trainer)
    t.hparams = SimpleNamespace(weight_decay=0.05)
    kw = t._muon_engine_args("muon", {"learning_rate": 0.03, "momentum": 0.9, "head_lr_scale": 0.4})
    assert kw["inner_optimizer"] == "muon" and kw["inner_lr"] == 0.03 and kw["muon_momentum"] == 0.9
    assert dict(kw["muon_aux_lr_scale"]) == {"head": 0.4, "embed": 0.5, "scalar": 0.2} and kw["weight_decay"] == 0.05
    assert t._muon_engine_args("adamw", {}) == {}
