"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""

import pytest
import torch
import torch.nn.functional as F

from templar_b200 import compress as C
from templar_b200.models.llama import ModelArgs, build_model
from templar_b200.ops import functional as OF
from templar_b200.ops import native
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine
from templar_b200.utils.synthetic import synthetic_payload

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _Bag(torch.nn.Module):
    """A module holding parameters of arbitrary shapes (drives the engine without a transformer)."""

    def __init__(self, shapes, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.ps = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(*s, generator=g) * 0.05) for s in shapes])


def _oracle_compress(e, delta, gamma, tr, comp, topk, use_dct):
    e = gamma * e + delta
    enc = tr.encode(e, use_dct=use_dct)
    idx, val, xshape, totalk = comp.compress(enc, topk)
    dec = tr.decode(comp.decompress(e, idx, val, xshape, totalk), use_dct=use_dct)
    return idx, val, xshape, totalk, e - dec, enc


@pytest.mark.parametrize("use_dct", [True, False])
@pytest.mark.parametrize("shapes,topk", [
    ([(128, 192), (256,), (64, 64)], 32),
    ([(96, 40), (192, 128), (130,)], 16),
    ([(64, 256), (48,), (320, 64)], 64),
])
def test_compress_kernel_matches_oracle(shapes, topk, use_dct):
    torch.manual_seed(1)
    model = _Bag(shapes).to(DEV)
    eng = WindowEngine(model, EngineConfig(topk=topk, use_dct=use_dct, momentum_decay=0.9), device=DEV,
                       compute_dtype=torch.float32)
    st = eng.store
    eng.snapshot()
    ef0 = torch.randn_like(eng.ef) * 0.01
    eng.ef.copy_(ef0)
    st.master_shard.add_(torch.randn_like(st.master_shard) * 0.02)   # theta after the inner steps
    theta0, theta = eng.theta0.clone(), st.master_shard.clone()
    eng.compress()
    torch.cuda.synchronize()
    assert eng.check_status() == 0
    tr = C.ChunkingTransformer(model, 64)
    comp = C.TopKCompressor()
    for s in eng.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        e = ef0[sl].view(s.shape).cpu().double()
        d = (theta0[sl] - theta[sl]).view(s.shape).cpu().double()
        tr64 = C.ChunkingTransformer(None, 64)
        tr64.register_shape(s.shape, dtype=torch.float64)
        idx_o, val_o, xshape, totalk, ef_o, enc = _oracle_compress(e, d, 0.9, tr64, comp, topk, use_dct)
        idx_k, val_k = eng.layout.payload_views(eng.own_idx, eng.own_val, s.name)
        k = s.topk(topk)
        assert tuple(val_k.shape) == tuple(val_o.shape)
        ik = C.unpack_12bit_indices(idx_k.cpu(), val_k.shape).reshape(-1, k)
        io = C.unpack_12bit_indices(idx_o, val_o.shape).reshape(-1, k)
        vk = val_k.cpu().double().reshape(-1, k)
        encf = enc.reshape(-1, s.totalk)
        # values are the coefficients at the reported indices
        assert torch.allclose(vk, torch.gather(encf, 1, ik), atol=2e-6, rtol=1e-4)
        # same selection up to ties at fp32 resolution: compare the selected magnitudes
        mk = vk.abs().sort(dim=1).values
        mo = val_o.reshape(-1, k).abs().sort(dim=1).values
        assert torch.allclose(mk, mo, atol=2e-6, rtol=1e-4)
        assert (ik.sort(dim=1).values[:, 1:] != ik.sort(dim=1).values[:, :-1]).all()   # distinct indices
        assert int(ik.max()) < s.totalk
        # error feedback residual
        ef_k = eng.ef[sl].view(s.shape).cpu().double()
        assert torch.allclose(ef_k, ef_o, atol=5e-6, rtol=1e-4), s.name
        _ = io


@pytest.mark.parametrize("use_dct", [True, False])
@pytest.mark.parametrize("update", ["sgd", "sign"])
def test_aggregate_kernel_matches_oracle(use_dct, update):
    shapes = [(128, 192), (256,), (96, 40), (64, 64)]
    n_peers, topk, lr = 5, 16, 0.3
    model = _Bag(shapes).to(DEV)
    eng = WindowEngine(model, EngineConfig(topk=topk, use_dct=use_dct, outer_lr=lr, outer_update=update,
                                           max_peers=n_peers), device=DEV, compute_dtype=torch.float32)
    eng.snapshot()
    theta0 = eng.theta0.clone()
    payloads = []
    for j in range(n_peers):
        idx, val = synthetic_payload(eng.layout, 10 + j, device=DEV, scale=1e-2 * (1 + 3 * j))
        payloads.append((idx, val))
        eng.load_peer_payload(j, (idx, val))
    eng.outer_step(n_peers, include_own=False)
    torch.cuda.synchronize()
    assert eng.check_status() == 0
    comp = C.TopKCompressor()
    for s in eng.layout.specs:
        tr = C.ChunkingTransformer(None, 64)
        tr.register_shape(s.shape, dtype=torch.float64)
        idxs, vals = [], []
        for idx, val in payloads:
            i, v = eng.layout.payload_views(idx, val, s.name)
            idxs.append(i.cpu()); vals.append(v.cpu().double())
        ref = torch.empty(s.shape, dtype=torch.float64)
        g = tr.decode(comp.batch_decompress(ref, idxs, vals, eng.layout.xshape(s.name), s.totalk, clip_norm=True),
                      use_dct=use_dct)
        sl = slice(s.offset, s.offset + s.numel)
        got = eng.store.master_shard[sl].view(s.shape).cpu().double()
        t0 = theta0[sl].view(s.shape).cpu().double()
        if update == "sgd":
            assert torch.allclose(got, t0 - lr * g, atol=3e-6, rtol=1e-5), s.name
        else:
            stable = g.abs() > 1e-7
            assert torch.allclose(got[stable], (t0 - lr * torch.sign(g))[stable], atol=1e-6), s.name


def test_rmsnorm_fwd_bwd():
    torch.manual_seed(0)
    for D in (256, 2048, 8192):
        x = torch.randn(3, 37, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
        y = OF.rmsnorm(x, w, 1e-5)
        dy = torch.randn_like(y)
        y.backward(dy)
        xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
        yr = F.rms_norm(xf, (D,), wf, 1e-5)
        yr.backward(dy.float())
        assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)
        assert torch.allclose(x.grad.float(), xf.grad, atol=2e-2, rtol=2e-2)
        assert torch.allclose(w.grad.float(), wf.grad, atol=0.15, rtol=3e-2)


def test_add_rmsnorm_fwd_bwd():
    """Residual add fused with RMSNorm (warp-per-row kernels) against fp32 autograd of the same math."""
    torch.manual_seed(1)
    # rows above 1024 elements take the bulk-copy-fed streaming backward: ragged last tile, many tiles per CTA
    for D, T in ((256, 37), (1024, 300), (2048, 2051), (776, 19), (1536, 999), (2048, 16385)):
        res = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        delta = torch.randn(T, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
        h, y = OF.add_rmsnorm(res, delta, w, 1e-5)
        dh, dy = torch.randn_like(h), torch.randn_like(y)
        torch.autograd.backward([h, y], [dh, dy])
        rf, df, wf = (t.detach().float().requires_grad_() for t in (res, delta, w))
        hr = (rf + df).detach().to(torch.bfloat16).float() + (rf + df - (rf + df).detach())   # bf16-rounded sum, identity gradient
        yr = F.rms_norm(hr, (D,), wf, 1e-5)
        torch.autograd.backward([hr, yr], [dh.float(), dy.float()])
        assert torch.equal(h, (res.detach().float() + delta.detach().float()).to(torch.bfloat16))
        assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
        assert torch.allclose(res.grad.float(), rf.grad, atol=4e-2, rtol=2e-2)
        assert torch.equal(res.grad, delta.grad)
        assert torch.allclose(w.grad.float(), wf.grad, atol=0.05 * T ** 0.5, rtol=3e-2)


def test_streaming_norm_backward_equals_the_warp_per_row_kernel():
    """Same arithmetic in the same order per row: dx bit-equal, dw equal up to the order of the atomic adds; with and
    without a residual gradient and without a weight-gradient target."""
    from templar_b200.ops import native

    L = native.lib()
    torch.manual_seed(3)
    for D, T, with_res in ((2048, 4099, True), (2048, 4096, False), (1280, 777, True)):
        dy, x = (torch.randn(T, D, device=DEV).to(torch.bfloat16) for _ in range(2))
        dres = torch.randn(T, D, device=DEV).to(torch.bfloat16) if with_res else None
        w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        outs = []
        for v2 in (False, True):
            dx = torch.full((T, D), float("nan"), device=DEV, dtype=torch.bfloat16)
            dw = torch.zeros(D, device=DEV)
            args = [dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if with_res else None,
                    dx.data_ptr(), dw.data_ptr(), T, D]
            if v2:
                native.check(L.tplr_add_rmsnorm_bwd_v2(*args, OF.status_word(DEV).data_ptr(), native.stream_ptr()), "bwd_v2")
            else:
                native.check(L.tplr_add_rmsnorm_bwd(*args, native.stream_ptr()), "bwd")
            outs.append((dx, dw))
        torch.cuda.synchronize()
        assert int(OF.status_word(DEV).item()) == 0
        assert torch.equal(outs[0][0], outs[1][0]), (D, T)
        assert torch.allclose(outs[0][1], outs[1][1], rtol=1e-4, atol=1e-3 * T ** 0.5), (D, T)
    # no weight-gradient target
    dx = torch.empty(T, D, device=DEV, dtype=torch.bfloat16)
    native.check(L.tplr_add_rmsnorm_bwd_v2(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), None,
                                           T, D, OF.status_word(DEV).data_ptr(), native.stream_ptr()), "bwd_v2")
    torch.cuda.synchronize()
    assert torch.isfinite(dx.float()).all() and int(OF.status_word(DEV).item()) == 0


def test_rope_matches_complex_multiply():
    B, S, H, KV, Dh = 2, 64, 4, 2, 128
    C_ = (H + 2 * KV) * Dh
    x = torch.randn(B, S, C_, device=DEV, dtype=torch.bfloat16)
    cos, sin = OF.rope_tables(S, Dh, 10000.0, DEV)
    xr = x.clone().requires_grad_()
    y = OF.rope(xr * 1.0, cos, sin, H + KV, Dh)
    fc = torch.complex(cos, sin)
    rot = torch.view_as_complex(x[..., :(H + KV) * Dh].float().reshape(B, S, H + KV, Dh // 2, 2))
    ref = torch.view_as_real(rot * fc.view(1, S, 1, Dh // 2)).reshape(B, S, (H + KV) * Dh)
    assert torch.allclose(y[..., :(H + KV) * Dh].float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(y[..., (H + KV) * Dh:], x[..., (H + KV) * Dh:])
    dy = torch.randn_like(y)
    y.backward(dy.clone())
    drot = torch.view_as_complex(dy[..., :(H + KV) * Dh].float().reshape(B, S, H + KV, Dh // 2, 2))
    dref = torch.view_as_real(drot * fc.conj().view(1, S, 1, Dh // 2)).reshape(B, S, (H + KV) * Dh)
    assert torch.allclose(xr.grad[..., :(H + KV) * Dh].float(), dref, atol=2e-2, rtol=2e-2)


def test_swiglu_fwd_bwd():
    h = torch.randn(5, 33, 2 * 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = OF.swiglu(h)
    dy = torch.randn_like(y)
    y.backward(dy)
    hf = h.detach().float().requires_grad_()
    yr = F.silu(hf[..., :512]) * hf[..., 512:]
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)
    assert torch.allclose(h.grad.float(), hf.grad, atol=3e-2, rtol=3e-2)


def test_cross_entropy_loss_and_grad():
    T, V = 300, 32000
    logits = (torch.randn(T, V, device=DEV) * 2).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    lf = logits.float().requires_grad_()
    ref = F.cross_entropy(lf, labels, ignore_index=-100)
    ref.backward()
    lg = logits.clone().requires_grad_()
    work = lg * 1.0
    loss = OF.cross_entropy(work, labels, 0.25)
    loss.backward()
    assert abs(float(loss) - float(ref)) < 2e-3
    assert torch.allclose(lg.grad.float(), 0.25 * lf.grad, atol=2e-5, rtol=2e-2)


def test_cross_entropy_out_of_range_labels_are_ignored_and_reported():
    """A label outside [0, V) is never used as an index: the row behaves like ignore_index and the status word
    carries the bad-index bit.  The oracle is PyTorch on labels masked on the host."""
    T, V = 64, 1000
    logits = (torch.randn(T, V, device=DEV) * 2).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[3], labels[10], labels[11] = V, -5, 2 ** 40
    labels[::9] = -100
    masked = torch.where((labels >= 0) & (labels < V), labels, torch.full_like(labels, -100))
    lf = logits.float().requires_grad_()
    ref = F.cross_entropy(lf, masked, ignore_index=-100)
    ref.backward()
    st = OF.status_word(DEV)
    st.zero_()
    lg = logits.clone().requires_grad_()
    loss = OF.cross_entropy(lg * 1.0, labels, 1.0)
    loss.backward()
    assert abs(float(loss) - float(ref)) < 2e-3
    assert torch.allclose(lg.grad.float(), lf.grad, atol=2e-5, rtol=2e-2)
    assert int(st.item()) & 1, "TPLR_ST_BAD_INDEX was not reported"
    st.zero_()


def test_embedding_fwd_bwd():
    V, D = 1000, 256
    table = torch.randn(V, D, device=DEV, dtype=torch.bfloat16)
    table.main_grad = torch.zeros(V, D, device=DEV)
    tok = torch.randint(0, V, (4, 50), device=DEV)
    t = table.clone().requires_grad_()
    out = OF.embedding(tok, t, table.main_grad)
    assert torch.equal(out, table[tok])
    dy = torch.randn_like(out)
    out.backward(dy)
    ref = torch.zeros(V, D, device=DEV).index_add_(0, tok.reshape(-1), dy.reshape(-1, D).float())
    assert torch.allclose(table.main_grad, ref, atol=1e-5)


def test_adamw_and_sumsq_match_torch():
    n = 4096 * 33
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 3
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    shadow = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    L = native.lib()
    scratch = torch.zeros(L.tplr_sumsq_blocks(), device=DEV)
    nsq = torch.zeros(1, device=DEV)
    for step in (1, 2, 3):
        gg = g * step
        ref_p.grad = gg.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        gk = gg.clone()
        native.check(L.tplr_sumsq(gk.data_ptr(), n, scratch.data_ptr(), nsq.data_ptr(), native.stream_ptr()), "sumsq")
        assert abs(float(nsq) - float((gg.double() ** 2).sum())) / float((gg.double() ** 2).sum()) < 1e-5
        native.check(L.tplr_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), gk.data_ptr(),
                                  native.ptr_array([shadow.data_ptr()]), 1, n, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0, 1.0,
                                  nsq.data_ptr(), 1, native.stream_ptr()), "adamw")
        assert torch.allclose(p, ref_p.detach(), atol=1e-5, rtol=1e-4)
        assert torch.equal(shadow, p.to(torch.bfloat16))
        assert float(gk.abs().max()) == 0.0


@pytest.mark.parametrize("backend", ["tcgen05_2sm", "tcgen05"])
def test_model_step_native_vs_torch_reference(backend):
    """One forward/backward of a small model: kernels (bf16) against the same model in fp32 PyTorch
    (fp32 operands never reach the own GEMM, so the reference side is torch.matmul)."""
    args = ModelArgs(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, intermediate_size=512, max_seq_len=128)
    prev = OF.gemm_backend()
    OF.set_gemm_backend(backend)
    try:
        ref = build_model(args, device=DEV, seed=3)           # fp32, autograd weight grads
        with torch.no_grad():
            for p in ref.parameters():                        # make the weights bf16-representable
                p.copy_(p.to(torch.bfloat16).float())
        model = build_model(args, device=DEV, dtype=torch.bfloat16, seed=None)
        model.load_state_dict(ref.state_dict())
        eng = WindowEngine(model, EngineConfig(topk=8), device=DEV)
        tok = torch.randint(0, 1024, (4, 129), device=DEV)
        loss = eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0)
        lr = ref.loss(tok[:, :-1], tok[:, 1:])
        lr.backward()
        assert abs(float(loss) - float(lr)) < 0.05
        for n, p in ref.named_parameters():
            g = dict(model.named_parameters())[n].main_grad
            rel = (g - p.grad).norm() / (p.grad.norm() + 1e-12)
            assert float(rel) < 0.08, (n, float(rel))
    finally:
        OF.set_gemm_backend(prev)


def test_sharded_parameter_engine_on_one_gpu_matches_plain_engine():
    """``shard_params`` with one rank: the whole machinery runs (weights gathered per block by the copy kernel on
    the side stream, weight gradients through the reduce-scatter GEMM epilogue, staged embedding / norm gradients,
    shard-addressed compress and outer step) and must give the plain engine's weights, error feedback and loss.
    The gradient of the plain engine is also checked against the shard tensor by tensor."""
    args = ModelArgs(dim=256, n_layers=3, n_heads=2, vocab_size=1024, intermediate_size=512, max_seq_len=256)
    tok = torch.randint(0, 1024, (2, 2, 4, 257), device=DEV)

    def run(shard, ckpt=False, buffers=2):
        model = build_model(args, device=DEV, dtype=torch.bfloat16, seed=3)
        model.activation_checkpointing = ckpt
        eng = WindowEngine(model, EngineConfig(topk=8, max_peers=2, inner_lr=1e-3, shard_params=shard,
                                               gather_buffers=buffers), device=DEV)
        eng.snapshot()
        grads = None
        for step in range(2):
            for mb in range(2):
                t = tok[step, mb]
                loss = eng.micro_step(t[:, :-1], t[:, 1:], 0.5)
            if step == 0:
                torch.cuda.synchronize()
                src = eng.store.grad_shard if shard else eng.store.grad
                grads = src.clone()
                if shard:                                     # staged tensors are reduced into the shard by the step
                    stage = eng.store.stage.clone()
                    for so, do, n in eng.store.stage_blocks(1 << 40):
                        grads[do: do + n] += stage[so: so + n]
            eng.optimizer_step()
        eng.compress()
        eng.load_peer_payload(1, synthetic_payload(eng.layout, 1, device=DEV))
        eng.outer_step(2)
        torch.cuda.synchronize()
        assert eng.check_status() == 0
        with torch.no_grad():
            final = float(model.loss(tok[0, 0][:, :-1], tok[0, 0][:, 1:]))
        return eng, grads, float(loss), final

    ref, g_ref, l_ref, f_ref = run(False)
    for kw in ({}, {"ckpt": True}, {"buffers": 8}):
        eng, g, l, f = run(True, **kw)
        assert eng.store.compute is None and eng.store.grad is None
        for s, a, b, la in eng.layout.segments(0):
            want = g_ref[a:b]
            rel = (g[la: la + (b - a)] - want).norm() / (want.norm() + 1e-12)
            assert float(rel) < 2e-3, (s.name, float(rel), kw)
        full = eng.full_master()
        assert (full - ref.store.master_shard).abs().max().item() < 1e-4 * max(ref.store.master_shard.abs().max().item(), 1.0)
        assert abs(l - l_ref) < 1e-3 and abs(f - f_ref) < 1e-2, (l, l_ref, f, f_ref)
        if kw.get("buffers"):
            assert eng.store.gather.gathers < 20      # every block stays gathered between the steps
    assert int(OF.status_word(DEV).item()) == 0


def test_payload_value_quantisation_matches_reference_format():
    """uint8 codes + per-tensor lookup produced by the kernels against the torch implementation of the
    reference's wire format, tensor by tensor."""
    from templar_b200 import compress as C

    args = ModelArgs(dim=256, n_layers=1, n_heads=2, vocab_size=512, intermediate_size=512, max_seq_len=128)
    model = build_model(args, device=DEV, dtype=torch.bfloat16, seed=1)
    eng = WindowEngine(model, EngineConfig(topk=8), device=DEV)
    eng.snapshot()
    eng.store.master_shard.add_(torch.randn_like(eng.store.master_shard) * 1e-3)
    eng.compress()
    plain = eng.own_payload()
    quant = eng.own_payload(quantize=True)
    comp = C.TopKCompressor(use_quantization=True, quantization_bins=256, quantization_range=6)
    for s in eng.layout.specs:
        val = plain[s.name + "vals"].float()
        q_ref, qp_ref = comp._quantize_values(val)
        q, qp = quant[s.name + "vals"], quant[s.name + "quant_params"]
        assert q.dtype == torch.uint8 and q.shape == val.shape
        assert torch.equal(plain[s.name + "idxs"], quant[s.name + "idxs"])
        assert abs(float(qp[0]) - float(qp_ref[0])) <= 1e-6 + 1e-4 * abs(float(qp_ref[0]))
        assert abs(qp[1] - qp_ref[1]) <= 1e-5 * qp_ref[1]
        assert qp[2] == qp_ref[2]
        mism = (q.int() - q_ref.int()).abs()
        assert int(mism.max()) <= 1 and float((mism > 0).float().mean()) < 0.01      # ties at bin edges only
        deq = comp._dequantize_values(q, qp)
        deq_ref = comp._dequantize_values(q_ref, qp_ref)
        assert float((deq.cpu() - deq_ref.cpu()).abs().max()) <= 2.0 * qp_ref[1]
        assert float((deq.cpu() - val.cpu()).abs().max()) <= 1.01 * qp_ref[1] * 256 / 2 + 1e-6


def test_index_overlap_kernel_matches_bitmap_count():
    """Pairwise shared (chunk, index) selections of staged peers: kernel over the packed payloads vs torch bitmaps."""
    from templar_b200.compress import unpack_12bit_indices

    args = ModelArgs(dim=256, n_layers=1, n_heads=2, vocab_size=512, intermediate_size=512, max_seq_len=128)
    model = build_model(args, device=DEV, dtype=torch.bfloat16, seed=1)
    eng = WindowEngine(model, EngineConfig(topk=8, max_peers=4), device=DEV)
    n = 4
    payloads = [synthetic_payload(eng.layout, 70 + j, device=DEV) for j in range(n)]
    payloads[2] = (payloads[0][0].clone(), payloads[2][1])          # peer 2 copies peer 0's indices: overlap 1.0
    for j, pl in enumerate(payloads):
        eng.load_peer_payload(j, pl)
    m = eng.index_overlap(n).cpu()
    assert abs(float(m[0, 2]) - 1.0) < 1e-12
    shared = torch.zeros(n, n, dtype=torch.float64)
    total = 0
    for s in eng.layout.specs:
        k = s.topk(eng.layout.topk)
        sets = []
        for j in range(n):
            ib, vb = eng.layout.payload_views(payloads[j][0], payloads[j][1], s.name)
            idx = unpack_12bit_indices(ib, vb.shape).reshape(-1, k)
            member = torch.zeros(idx.shape[0], 4096, dtype=torch.bool, device=idx.device)
            member.scatter_(-1, idx, True)
            sets.append(member)
        total += sets[0].shape[0] * k
        for i in range(n):
            for j in range(i + 1, n):
                shared[i, j] += float((sets[i] & sets[j]).sum())
    for i in range(n):
        for j in range(i + 1, n):
            assert abs(float(m[i, j]) - shared[i, j] / total) < 1e-9, (i, j)


def test_quantised_compress_keeps_quantisation_error_in_error_feedback():
    """Engine with ``quantize``: codes + tables from the kernels, dequantised values in the payload and
    ef_new + decode(payload) == momentum * ef_old + delta (the reference's residual under quantisation)."""
    import importlib.util
    import os

    spec = importlib.util.spec_from_file_location(
        "engine_cpu_cases", os.path.join(os.path.dirname(os.path.abspath(__file__)), "test_engine_cpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    quantised_window_identity = mod.quantised_window_identity

    eng = quantised_window_identity("cuda")
    assert eng.check_status() == 0


def test_encode_values_and_flat_quantised_staging():
    """encode_values -> (codes, tables); the 3-tuple staged from pinned host memory decodes to lookup[code] + shift,
    within half a bin of the original values where they were not clamped."""
    model = _Bag([(128, 192), (256,), (96, 40), (64, 64)]).to(DEV)
    eng = WindowEngine(model, EngineConfig(topk=16, max_peers=2, quant_bins=64), device=DEV, compute_dtype=torch.float32)
    idx, val = synthetic_payload(eng.layout, 3, device=DEV, scale=1e-2)
    codes, table = eng.encode_values(val)
    eng.load_peer_payload(1, (idx.cpu().pin_memory(), codes.cpu().pin_memory(), table.cpu().pin_memory()))
    torch.cuda.synchronize()
    assert torch.equal(eng.peer_idx[1][: idx.numel()], idx)
    for s in eng.layout.specs:
        _, c = eng.layout.payload_views(idx, codes, s.name)
        _, got = eng.layout.payload_views(idx, eng.peer_val[1], s.name)
        _, v = eng.layout.payload_views(idx, val, s.name)
        row = table[s.index]
        assert torch.equal(got, (row[:64][c.long()] + row[64]).reshape(got.shape))
        inner = (c > 0) & (c < 63)
        assert float((got - v).abs()[inner.reshape(got.shape)].max()) <= 1.01 * float(row[65])
        comp = C.TopKCompressor(use_quantization=True, quantization_bins=64, quantization_range=6)
        q, qp = comp._quantize_values(v.cpu().float())
        assert float((q.long() - c.cpu().long().reshape(q.shape)).abs().max()) <= 1     # same bins up to rounding ties
        assert abs(float(qp[1]) / float(row[65]) - 1) < 1e-4


def test_payloads_staged_on_the_side_stream_give_the_same_outer_step():
    """Peers' payloads copied from pinned host memory on a side stream (beside a busy compute stream) and joined by the
    outer step: the same weights as with copies on the compute stream, for two windows in a row (the second reuses the
    slots, which the side stream may only refill after the first outer step has read them)."""
    def run(asynchronous):
        torch.manual_seed(0)
        model = _Bag([(256, 192), (256,), (128, 64)]).to(DEV)
        eng = WindowEngine(model, EngineConfig(topk=16, max_peers=4, quant_bins=64), device=DEV, compute_dtype=torch.float32)
        busy = torch.randn(4096, 4096, device=DEV)
        out = []
        for w in range(2):
            eng.snapshot()
            eng.store.master_shard.add_(1e-3)
            eng.compress()
            items = []
            for j in range(1, 4):
                idx, val = synthetic_payload(eng.layout, 40 + 10 * w + j, device=DEV, scale=1e-2)
                if j == 2:                                     # one peer in the 8-bit wire format
                    codes, table = eng.encode_values(val)
                    items.append((j, (idx.cpu().pin_memory(), codes.cpu().pin_memory(), table.cpu().pin_memory())))
                else:
                    items.append((j, (idx.cpu().pin_memory(), val.cpu().pin_memory())))
            torch.cuda.synchronize()
            for _ in range(8):
                busy = busy @ busy * 1e-4                      # work in flight on the compute stream while the copies run
            if asynchronous:
                eng.load_peer_payloads_async(items)
            else:
                for slot, pl in items:
                    eng.load_peer_payload(slot, pl)
            eng.outer_step(4)
            out.append(eng.store.master_shard.clone())
        torch.cuda.synchronize()
        assert eng.check_status() == 0
        return out

    a, b = run(True), run(False)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert not torch.equal(a[0], a[1])


@pytest.mark.parametrize("quantize", [False, True])
def test_compress_and_aggregate_are_bitwise_repeatable(quantize):
    """The same inputs give the same bytes: payload, codes and tables, error feedback and updated weights.  The
    top-k compaction is ordered, the 8-bit encoder sums its bins in 64-bit fixed point, and the scatter-add of the
    gather uses shared-memory float atomics, which commute for the at most two contributions per coefficient of
    this case (own payload + one peer)."""
    args = ModelArgs(dim=256, n_layers=1, n_heads=2, vocab_size=512, intermediate_size=512, max_seq_len=128)
    runs = []
    for _ in range(2):
        model = build_model(args, device=DEV, dtype=torch.bfloat16, seed=4)
        eng = WindowEngine(model, EngineConfig(topk=16, max_peers=2, quantize=quantize), device=DEV)
        g = torch.Generator(device=DEV).manual_seed(11)
        eng.ef.copy_(torch.randn(eng.ef.shape, device=DEV, generator=g) * 1e-3)
        eng.snapshot()
        eng.store.master_shard.add_(torch.randn(eng.ef.shape, device=DEV, generator=g) * 1e-3)
        eng.compress()
        eng.load_peer_payload(1, synthetic_payload(eng.layout, 21, device=DEV))
        eng.outer_step(2)
        torch.cuda.synchronize()
        assert eng.check_status() == 0
        rec = {"idx": eng.own_idx.clone(), "val": eng.own_val.clone(), "ef": eng.ef.clone(),
               "master": eng.store.master_shard.clone(), "compute": eng.store.compute.clone()}
        if quantize:
            rec["codes"], rec["table"] = eng._q_codes.clone(), eng._q_table.clone()
        runs.append(rec)
    for name in runs[0]:
        assert torch.equal(runs[0][name], runs[1][name]), name
