"""The composite ops of ``ops/functional.py`` on the CPU path: each equals the node-per-op composition it stands for
(on CUDA the same entry points run the GEMM-epilogue kernels; the GPU tier compares those against fp32 PyTorch)."""

import torch

from templar_b200.ops import functional as OF


def _grads(out, *tensors):
    out.sum().backward()
    g = [t.grad.clone() for t in tensors]
    for t in tensors:
        t.grad = None
    return g


def test_feed_forward_equals_projection_activation_projection():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 16, requires_grad=True)
    w13 = torch.randn(24, 16, requires_grad=True)
    w2 = torch.randn(16, 12, requires_grad=True)
    y = OF.feed_forward(x, w13, w2)
    g = _grads(y, x, w13, w2)
    y2 = OF.linear(OF.swiglu(OF.linear(x, w13)), w2)
    g2 = _grads(y2, x, w13, w2)
    ref = (torch.nn.functional.silu(x @ w13[:12].t()) * (x @ w13[12:].t())) @ w2.t()
    assert torch.equal(y, y2) and torch.allclose(y, ref, atol=1e-5)
    assert all(torch.equal(a, b) for a, b in zip(g, g2))


def test_feed_forward_accumulates_into_main_grad_buffers():
    torch.manual_seed(1)
    x = torch.randn(4, 16, requires_grad=True)
    w13, w2 = torch.randn(24, 16, requires_grad=True), torch.randn(16, 12, requires_grad=True)
    w13.main_grad, w2.main_grad = torch.ones(24, 16), torch.ones(16, 12)
    OF.feed_forward(x, w13, w2).sum().backward()
    a, b = w13.main_grad.clone(), w2.main_grad.clone()
    w13.main_grad, w2.main_grad = None, None
    del w13.main_grad, w2.main_grad
    x.grad = None
    OF.feed_forward(x, w13, w2).sum().backward()
    assert torch.allclose(a, w13.grad + 1, atol=1e-5) and torch.allclose(b, w2.grad + 1, atol=1e-5)


def test_rope_attention_projection_equals_its_three_steps():
    torch.manual_seed(2)
    B, S, H, KV, hd, K = 2, 8, 2, 1, 16, 32
    x = torch.randn(B, S, K, requires_grad=True)
    w = torch.randn((H + 2 * KV) * hd, K, requires_grad=True)
    cos, sin = OF.rope_tables(S, hd)
    o = OF.rope_attention_projection(x, w, cos, sin, H, KV, hd)
    g = _grads(o, x, w)
    o2 = OF.attention_packed(OF.rope(OF.linear(x, w), cos, sin, H + KV, hd), H, KV, hd)
    g2 = _grads(o2, x, w)
    assert torch.equal(o, o2) and all(torch.equal(a, b) for a, b in zip(g, g2))
    # against the textbook formula: rotate q and k, causal softmax per head with grouped keys
    qkv = x @ w.t()
    q, k, v = OF._split_qkv(OF._rope_torch(qkv, cos, sin, (H + KV) * hd, hd, False), H, KV, hd)
    k, v = (t.repeat_interleave(H // KV, dim=2) for t in (k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                           is_causal=True).transpose(1, 2).reshape(B, S, H * hd)
    assert torch.allclose(o, ref, atol=1e-5)


def test_linear_swiglu_equals_projection_then_activation():
    torch.manual_seed(3)
    x, w = torch.randn(6, 16, requires_grad=True), torch.randn(24, 16, requires_grad=True)
    h = OF.linear_swiglu(x, w)
    g = _grads(h, x, w)
    h2 = OF.swiglu(OF.linear(x, w))
    g2 = _grads(h2, x, w)
    assert torch.equal(h, h2) and all(torch.equal(a, b) for a, b in zip(g, g2))


def test_attention_block_equals_projection_rotation_attention_projection():
    torch.manual_seed(4)
    B, S, H, KV, hd, K = 1, 8, 2, 1, 16, 32
    x = torch.randn(B, S, K, requires_grad=True)
    w = torch.randn((H + 2 * KV) * hd, K, requires_grad=True)
    wo = torch.randn(K, H * hd, requires_grad=True)
    cos, sin = OF.rope_tables(S, hd)
    o = OF.attention_block(x, w, wo, cos, sin, H, KV, hd)
    g = _grads(o, x, w, wo)
    o2 = OF.linear(OF.attention_packed(OF.rope(OF.linear(x, w), cos, sin, H + KV, hd), H, KV, hd), wo)
    g2 = _grads(o2, x, w, wo)
    assert torch.equal(o, o2) and all(torch.equal(a, b) for a, b in zip(g, g2))
