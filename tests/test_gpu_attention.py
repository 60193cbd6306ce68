"""tcgen05 flash attention (forward and backward) against fp32 PyTorch attention on the same bf16 inputs."""

import math

import pytest
import torch

from templar_b200.ops import functional as OF

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference(qkv, H, KV, hd):
    """fp32 causal GQA attention of the packed tensor, plain matmul + softmax."""
    B, S, _ = qkv.shape
    x = qkv.float()
    q = x[..., :H * hd].view(B, S, H, hd).transpose(1, 2)
    k = x[..., H * hd:(H + KV) * hd].view(B, S, KV, hd).transpose(1, 2).repeat_interleave(H // KV, dim=1)
    v = x[..., (H + KV) * hd:].view(B, S, KV, hd).transpose(1, 2).repeat_interleave(H // KV, dim=1)
    s = q @ k.transpose(-1, -2) / math.sqrt(hd)
    mask = torch.ones(S, S, device=x.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, H * hd)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("B,S,H,KV", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 512, 2, 2), (2, 1024, 4, 1)])
def test_attention_forward_backward(B, S, H, KV, variant):
    """variant 1: 128 query rows per step; variant 2: pipelined transposed backward (64 query rows per step)."""
    from templar_b200.ops import native
    assert native.lib().tplr_attention_set_bwd_variant(variant) == 0
    try:
        _run_case(B, S, H, KV)
    finally:
        native.lib().tplr_attention_set_bwd_variant(1)


def _run_case(B, S, H, KV):
    hd = 128
    torch.manual_seed(S + H)
    qkv = torch.randn(B, S, (H + 2 * KV) * hd, device=DEV).to(torch.bfloat16).requires_grad_()
    OF.status_word(DEV).zero_()
    assert OF.attention_backend() == "tcgen05"
    out = OF.attention_packed(qkv, H, KV, hd)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    assert int(OF.status_word(DEV).item()) == 0, "a bounded wait expired inside the attention kernels"
    ref_in = qkv.detach().clone().requires_grad_()
    ref = _reference(ref_in, H, KV, hd)
    ref.backward(dout.float())
    assert (out.float() - ref).abs().max().item() < 2e-2
    g, gr = qkv.grad.float(), ref_in.grad.float()
    nq, nk = H * hd, KV * hd
    for name, sl in (("dq", slice(0, nq)), ("dk", slice(nq, nq + nk)), ("dv", slice(nq + nk, None))):
        err = (g[..., sl] - gr[..., sl]).abs().max().item()
        scale = gr[..., sl].abs().max().item()
        assert err < 2e-2 * max(scale, 1.0), (name, err, scale)


def test_attention_at_the_benchmark_shape():
    """B 8, S 2048, 16 query heads on 8 key/value heads (head_dim 128): the shape of the 1B benchmark's micro-batch,
    with grouped queries.  The fp32 oracle runs one batch element at a time to bound its memory."""
    B, S, H, KV, hd = 8, 2048, 16, 8, 128
    torch.manual_seed(7)
    qkv = torch.randn(B, S, (H + 2 * KV) * hd, device=DEV).to(torch.bfloat16).requires_grad_()
    OF.status_word(DEV).zero_()
    out = OF.attention_packed(qkv, H, KV, hd)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    assert int(OF.status_word(DEV).item()) == 0
    nq, nk = H * hd, KV * hd
    for b in range(B):
        ref_in = qkv.detach()[b:b + 1].clone().requires_grad_()
        ref = _reference(ref_in, H, KV, hd)
        ref.backward(dout[b:b + 1].float())
        assert (out[b:b + 1].float() - ref).abs().max().item() < 2e-2, b
        g, gr = qkv.grad[b:b + 1].float(), ref_in.grad.float()
        for name, sl in (("dq", slice(0, nq)), ("dk", slice(nq, nq + nk)), ("dv", slice(nq + nk, None))):
            err = (g[..., sl] - gr[..., sl]).abs().max().item()
            scale = gr[..., sl].abs().max().item()
            assert err < 2e-2 * max(scale, 1.0), (b, name, err, scale)


def test_attention_matches_sdpa_backend_in_model_block():
    """The packed path and the library path give the same block output (RoPE applied before both)."""
    B, S, H, KV, hd = 2, 256, 4, 2, 128
    qkv = torch.randn(B, S, (H + 2 * KV) * hd, device=DEV).to(torch.bfloat16)
    a = OF.attention_packed(qkv, H, KV, hd)
    OF.set_attention_backend("sdpa")
    try:
        b = OF.attention_packed(qkv, H, KV, hd)
    finally:
        OF.set_attention_backend("tcgen05")
    assert (a.float() - b.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("B,S,H,KV,K", [(2, 256, 4, 2, 512), (1, 384, 3, 1, 192), (8, 2048, 16, 8, 2048)])
def test_projection_rope_attention_as_one_node_matches_the_three_node_path(B, S, H, KV, K):
    """Rotary embedding in the projection's epilogue and its inverse in the attention backward's outputs, against the
    projection, the in-place rotation kernel and the attention as separate autograd nodes (which other tests pin to
    fp32 PyTorch), and against an fp32 PyTorch evaluation of the whole expression."""
    from templar_b200.ops import functional as OF

    hd = 128
    torch.manual_seed(B * S + H)
    x = (torch.randn(B, S, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hd, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    cos, sin = OF.rope_tables(S + 64, hd, 10000.0, "cuda")
    cos, sin = cos.contiguous(), sin.contiguous()
    dout = torch.randn(B, S, H * hd, device="cuda").to(torch.bfloat16)
    OF.status_word("cuda").zero_()

    def run(fused):
        xx, ww = x.clone().requires_grad_(), w.clone().requires_grad_()
        if fused:
            from templar_b200.ops import native
            n0 = native.launch_count
            out = OF.rope_attention_projection(xx, ww, cos, sin, H, KV, hd)
            assert native.launch_count - n0 == 2    # projection with the rotation, attention: no rotation pass
        else:
            out = OF.attention_packed(OF.rope(OF.linear(xx, ww), cos, sin, H + KV, hd), H, KV, hd)
        out.backward(dout)
        return out.float(), xx.grad.float(), ww.grad.float()

    o1, gx1, gw1 = run(True)
    o0, gx0, gw0 = run(False)
    torch.cuda.synchronize()
    assert int(OF.status_word("cuda").item()) == 0
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()      # noqa: E731
    # same arithmetic up to where the bf16 rounding of q and k happens (before the rotation there, after it here)
    assert rel(o1, o0) < 1.5e-2 and rel(gx1, gx0) < 2e-2 and rel(gw1, gw0) < 2e-2, (rel(o1, o0), rel(gx1, gx0), rel(gw1, gw0))
    if B * S <= 1024:
        xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
        qkv = OF._rope_torch(xf @ wf.t(), cos, sin, (H + KV) * hd, hd, False)
        q, k, v = OF._split_qkv(qkv, H, KV, hd)
        k, v = (t.repeat_interleave(H // KV, dim=2) for t in (k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                               is_causal=True).transpose(1, 2).reshape(B, S, H * hd)
        ref.backward(dout.float())
        e_fused = (rel(o1, ref), rel(gx1, xf.grad), rel(gw1, wf.grad))
        e_three = (rel(o0, ref), rel(gx0, xf.grad), rel(gw0, wf.grad))
        assert max(e_fused) < 3e-2, (e_fused, e_three)
        assert all(a < 1.5 * b + 2e-3 for a, b in zip(e_fused, e_three)), (e_fused, e_three)


@pytest.mark.parametrize("B,S,H,KV,K", [(2, 256, 4, 2, 512), (1, 384, 3, 1, 192), (8, 2048, 16, 8, 2048)])
def test_attention_block_with_delta_from_the_output_projection_epilogue(B, S, H, KV, K):
    """The whole block as one node: the output projection's data-gradient GEMM forms the attention backward's delta term
    (row sum of dO * O per head) in its epilogue.  Against the node-per-op path (separate delta kernel) and, for the small
    shapes, an fp32 PyTorch evaluation."""
    from templar_b200.ops import functional as OF, native

    hd = 128
    torch.manual_seed(B * S + H + 1)
    x = (torch.randn(B, S, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn((H + 2 * KV) * hd, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    wo = (torch.randn(K, H * hd, device="cuda") / (H * hd) ** 0.5).to(torch.bfloat16)
    cos, sin = OF.rope_tables(S, hd, 10000.0, "cuda")
    cos, sin = cos.contiguous(), sin.contiguous()
    dy = torch.randn(B, S, K, device="cuda").to(torch.bfloat16)
    OF.status_word("cuda").zero_()

    def run(fused):
        prev = OF.FUSED_PROJECTIONS
        OF.FUSED_PROJECTIONS = fused
        try:
            xx, ww, oo = (t.clone().requires_grad_() for t in (x, w, wo))
            n0 = native.launch_count
            y = OF.attention_block(xx, ww, oo, cos, sin, H, KV, hd)
            y.backward(dy)
            return y.float(), xx.grad.float(), ww.grad.float(), oo.grad.float(), native.launch_count - n0
        finally:
            OF.FUSED_PROJECTIONS = prev

    yf, *gf, n_f = run(True)
    ys, *gs, n_s = run(False)
    torch.cuda.synchronize()
    assert int(OF.status_word("cuda").item()) == 0
    assert n_f == 8 and n_s == 10          # no rotation pass in either direction (the delta pass is inside the attention launch count)
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()      # noqa: E731
    errs = [rel(yf, ys)] + [rel(a, b) for a, b in zip(gf, gs)]
    assert max(errs) < 2e-2, errs
    if B * S <= 1024:
        xf, wf, of = (t.float().requires_grad_() for t in (x, w, wo))
        qkv = OF._rope_torch(xf @ wf.t(), cos, sin, (H + KV) * hd, hd, False)
        q, k, v = OF._split_qkv(qkv, H, KV, hd)
        k, v = (t.repeat_interleave(H // KV, dim=2) for t in (k, v))
        att = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                               is_causal=True).transpose(1, 2).reshape(B, S, H * hd)
        ref = att @ of.t()
        ref.backward(dy.float())
        e_f = [rel(yf, ref)] + [rel(a, b.grad) for a, b in zip(gf, (xf, wf, of))]
        e_s = [rel(ys, ref)] + [rel(a, b.grad) for a, b in zip(gs, (xf, wf, of))]
        assert max(e_f) < 3e-2, (e_f, e_s)
        assert all(a < 1.5 * b + 2e-3 for a, b in zip(e_f, e_s)), (e_f, e_s)
