"""LLaMA-architecture decoder with the parameter names of the reference's model.

State-dict keys match the torchtitan ``Transformer`` the reference trains
(models/llama3/model/model.py:20-436): ``tok_embeddings.weight``,
``layers.{i}.attention.{wq,wk,wv,wo}.weight``, ``layers.{i}.feed_forward.{w1,w2,w3}.weight``,
``layers.{i}.{attention_norm,ffn_norm}.weight``, ``norm.weight``, ``output.weight`` and the
persistent complex buffer ``freqs_cis`` — so DCP checkpoints are interchangeable.

Execution differs from the reference: Q/K/V are one GEMM against the packed
``[wq; wk; wv]`` rows and gate/up one GEMM against ``[w1; w3]`` (the flat parameter store
lays those tensors out adjacently, so the packed matrices are views, not copies), RoPE is
applied in place on the packed projection, SwiGLU reads the packed projection, and the
loss kernel emits the logit gradient during the forward pass.  All of these go through
:mod:`templar_b200.ops.functional`, i.e. hand-written kernels on a B200 and PyTorch on CPU.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import functional as OF


@dataclass
class ModelArgs:
    dim: int = 2048
    n_layers: int = 16
    n_heads: int = 16
    n_kv_heads: int | None = None
    vocab_size: int = 32000
    intermediate_size: int | None = None
    multiple_of: int = 256
    ffn_dim_multiplier: float | None = None
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 2048
    depth_init: bool = True
    tie_embeddings: bool = False

    @property
    def kv_heads(self) -> int:
        return self.n_kv_heads or self.n_heads

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def ffn_hidden(self) -> int:
        if self.intermediate_size is not None:
            return int(self.intermediate_size)
        hidden = int(2 * (4 * self.dim) / 3)
        if self.ffn_dim_multiplier is not None:
            hidden = int(self.ffn_dim_multiplier * hidden)
        return self.multiple_of * ((hidden + self.multiple_of - 1) // self.multiple_of)

    def num_params(self) -> int:
        d, f, v, kv = self.dim, self.ffn_hidden, self.vocab_size, self.kv_heads * self.head_dim
        per_layer = 2 * d * d + 2 * kv * d + 3 * d * f + 2 * d
        return self.n_layers * per_layer + v * d * (1 if self.tie_embeddings else 2) + d

    def flops_per_token(self, seq_len: int) -> float:
        """Forward+backward model FLOPs per token (6 N for the matmuls + causal attention)."""
        d, f, v, kv = self.dim, self.ffn_hidden, self.vocab_size, self.kv_heads * self.head_dim
        mm = self.n_layers * (2 * d * d + 2 * kv * d + 3 * d * f) + v * d
        attn = self.n_layers * 2 * seq_len * d / 2  # QK^T and PV, causal half
        return 6.0 * mm + 6.0 * attn


# Named presets.  "150M" and "1B" are the benchmark configurations; the llama3 sizes follow the
# public architecture tables.
PRESETS: dict[str, ModelArgs] = {
    "tiny": ModelArgs(dim=128, n_layers=2, n_heads=4, vocab_size=512, intermediate_size=256, max_seq_len=128),
    "150M": ModelArgs(dim=768, n_layers=12, n_heads=12, vocab_size=32000, intermediate_size=3072),
    "1B": ModelArgs(dim=2048, n_layers=16, n_heads=16, vocab_size=32000, intermediate_size=8192),
    "8B": ModelArgs(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256, intermediate_size=14336,
                    rope_theta=500000.0),
    "18B-tp": ModelArgs(dim=8192, n_layers=16, n_heads=64, n_kv_heads=8, vocab_size=128256,
                        intermediate_size=28672, rope_theta=500000.0),
    "34B": ModelArgs(dim=8192, n_layers=32, n_heads=64, n_kv_heads=8, vocab_size=128256, intermediate_size=28672,
                     rope_theta=500000.0),
    "70B": ModelArgs(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, vocab_size=128256, intermediate_size=28672,
                     rope_theta=500000.0),
}


class _Weight(nn.Module):
    """A bias-free linear layer's parameter holder (keeps the ``.weight`` FQN)."""

    def __init__(self, out_features: int, in_features: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def forward(self, x):
        return OF.linear(x, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return OF.rmsnorm(x, self.weight, self.eps)


class Attention(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.n_heads, self.n_kv, self.hd = args.n_heads, args.kv_heads, args.head_dim
        self.wq = _Weight(args.n_heads * self.hd, args.dim)
        self.wk = _Weight(self.n_kv * self.hd, args.dim)
        self.wv = _Weight(self.n_kv * self.hd, args.dim)
        self.wo = _Weight(args.dim, args.n_heads * self.hd)
        self.packed = None  # (weight view, main_grad view) of [wq; wk; wv] set by the flat store

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        if self.packed is not None:          # projections, rotary embedding and attention as one node on the own kernels
            return OF.attention_block(x, self.packed[0], self.wo.weight, cos, sin, self.n_heads, self.n_kv, self.hd,
                                      self.packed[1], getattr(self.wo.weight, "main_grad", None))
        qkv = OF.linear(x, torch.cat((self.wq.weight, self.wk.weight, self.wv.weight), dim=0))
        qkv = OF.rope(qkv, cos, sin, self.n_heads + self.n_kv, self.hd)
        return self.wo(OF.attention_packed(qkv, self.n_heads, self.n_kv, self.hd))


class FeedForward(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.w1 = _Weight(args.ffn_hidden, args.dim)
        self.w2 = _Weight(args.dim, args.ffn_hidden)
        self.w3 = _Weight(args.ffn_hidden, args.dim)
        self.packed = None  # [w1; w3]

    def forward(self, x):
        if self.packed is not None:      # the activation and its backward run in the epilogues of the two projections
            return OF.feed_forward(x, self.packed[0], self.w2.weight, self.packed[1], getattr(self.w2.weight, "main_grad", None))
        h = OF.linear(x, torch.cat((self.w1.weight, self.w3.weight), dim=0))
        return self.w2(OF.swiglu(h))


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, args: ModelArgs):
        super().__init__()
        self.attention = Attention(args)
        self.feed_forward = FeedForward(args)
        self.attention_norm = RMSNorm(args.dim, args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, args.norm_eps)
        self.layer_id = layer_id
        self.weight_init_std = (0.02 / (2 * (layer_id + 1)) ** 0.5 if args.depth_init
                                else 0.02 / (2 * args.n_layers) ** 0.5)

    def forward(self, x, cos, sin):
        h = x + self.attention(self.attention_norm(x), cos, sin)
        return h + self.feed_forward(self.ffn_norm(h))

    def forward_fused(self, res, delta, cos, sin):
        """Same block on a split residual stream: the hidden state is ``res + delta`` and the sum is
        formed inside the norm kernels (``delta`` None: ``res`` alone).  Returns the next ``(res, delta)``.

        With ``recompute_ops`` (per-op selective activation checkpointing) the normalised activations and the
        SwiGLU output are not stored: each is recomputed in the backward pass for the weight gradient of the
        GEMM that consumed it, while every GEMM and attention output is kept."""
        att, ff = self.attention, self.feed_forward
        if getattr(self, "recompute_ops", False) and att.packed is not None and ff.packed is not None:
            nw, eps = self.attention_norm, self.attention_norm.eps
            if delta is None:
                qkv = OF.norm_linear(res, None, nw.weight, eps, att.packed[0], att.packed[1])
            else:
                res, qkv = OF.norm_linear(res, delta, nw.weight, eps, att.packed[0], att.packed[1])
            qkv = OF.rope(qkv, cos, sin, att.n_heads + att.n_kv, att.hd)
            a = att.wo(OF.attention_packed(qkv, att.n_heads, att.n_kv, att.hd))
            res, h13 = OF.norm_linear(res, a, self.ffn_norm.weight, self.ffn_norm.eps, ff.packed[0], ff.packed[1])
            return res, OF.swiglu_linear(h13, ff.w2.weight)
        if delta is None:
            y = self.attention_norm(res)
        else:
            res, y = OF.add_rmsnorm(res, delta, self.attention_norm.weight, self.attention_norm.eps)
        a = self.attention(y, cos, sin)
        res, y = OF.add_rmsnorm(res, a, self.ffn_norm.weight, self.ffn_norm.eps)
        return res, self.feed_forward(y)

    def init_weights(self, generator=None):
        for norm in (self.attention_norm, self.ffn_norm):
            nn.init.ones_(norm.weight)
        for lin in (self.attention.wq, self.attention.wk, self.attention.wv, self.feed_forward.w1):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=0.02, generator=generator)
        for lin in (self.attention.wo, self.feed_forward.w2, self.feed_forward.w3):
            nn.init.trunc_normal_(lin.weight, mean=0.0, std=self.weight_init_std, generator=generator)


class LlamaModel(nn.Module):
    """``forward(tokens, labels=None)`` returns logits; :meth:`loss` returns the mean CE."""

    def __init__(self, args: ModelArgs):
        super().__init__()
        self.args = args
        self.model_args = args  # name used by torchtitan-style callers
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.layers = nn.ModuleDict({str(i): TransformerBlock(i, args) for i in range(args.n_layers)})
        self.norm = RMSNorm(args.dim, args.norm_eps)
        self.output = _Weight(args.vocab_size, args.dim)
        if args.tie_embeddings:
            self.output.weight = self.tok_embeddings.weight
        self.register_buffer("freqs_cis", self._freqs_cis(), persistent=True)
        self._rope_cache: dict = {}
        # False / True (every block recomputed), or the reference's modes (hparams torchtitan.activation_checkpoint):
        # "none", "full", "selective" with ``ac_option`` = "op" (per-op policy: GEMM and attention outputs kept,
        # norms and activations recomputed) or an integer N (every N-th block recomputed whole)
        self.activation_checkpointing = False
        self.ac_option = "op"

    # -- rotary tables --------------------------------------------------------------------
    def _freqs_cis(self) -> torch.Tensor:
        cos, sin = OF.rope_tables(self.args.max_seq_len, self.args.head_dim, self.args.rope_theta)
        return torch.complex(cos, sin)

    def _rope(self, device):
        key = str(device)
        if key not in self._rope_cache:
            cos, sin = OF.rope_tables(self.args.max_seq_len, self.args.head_dim, self.args.rope_theta, device)
            self._rope_cache[key] = (cos.contiguous(), sin.contiguous())
        return self._rope_cache[key]

    # -- init ------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int | None = None, buffer_device=None):
        gen = None
        dev = self.tok_embeddings.weight.device
        if seed is not None:
            gen = torch.Generator(device=dev)
            gen.manual_seed(seed)
        self.tok_embeddings.weight.normal_(generator=gen)
        for layer in self.layers.values():
            layer.init_weights(gen)
        nn.init.ones_(self.norm.weight)
        if not self.args.tie_embeddings:
            std = self.args.dim ** -0.5
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=gen)
        self.freqs_cis = self._freqs_cis().to(buffer_device or self.freqs_cis.device)

    def materialize_param(self, name: str, device, dtype=None, seed: int = 0) -> torch.Tensor:
        """One parameter's initial value, created on ``device`` on its own (the distributions of
        :meth:`init_weights`, seeded per tensor).  Lets a model that was built on the meta device be initialised
        tensor by tensor straight into sharded storage, so that a model too large for one GPU never exists whole."""
        shape = dict(self.named_parameters())[name].shape
        gen = torch.Generator(device=device)
        index = [n for n, _ in self.named_parameters()].index(name)
        gen.manual_seed(int(seed) * 1_000_003 + index)
        t = torch.empty(shape, dtype=torch.float32, device=device)
        if name.endswith("norm.weight"):
            t.fill_(1.0)
        elif name == "tok_embeddings.weight":
            t.normal_(generator=gen)
        elif name == "output.weight":
            std = self.args.dim ** -0.5
            nn.init.trunc_normal_(t, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=gen)
        else:
            layer = self.layers[name.split(".")[1]]
            scaled = any(k in name for k in ("attention.wo.", "feed_forward.w2.", "feed_forward.w3."))
            nn.init.trunc_normal_(t, mean=0.0, std=layer.weight_init_std if scaled else 0.02, generator=gen)
        return t if dtype is None else t.to(dtype)

    # -- forward ---------------------------------------------------------------------------
    def hidden_states(self, tokens: torch.Tensor) -> torch.Tensor:
        cos, sin = self._rope(tokens.device)
        # With sharded parameters (parallel/fsdp.py) the weights of a block are only present while the block runs:
        # `pg` brings them in ahead of the block in both directions of the pass.
        pg = getattr(self, "_param_gather", None)
        if pg is not None:
            pg.begin_forward()
        h = OF.embedding(tokens, self.tok_embeddings.weight)
        delta = None
        mode = self.activation_checkpointing
        mode = {True: "full", False: "none", None: "none"}.get(mode, mode)
        per_op = mode == "selective" and str(self.ac_option) == "op"
        every = int(self.ac_option) if mode == "selective" and str(self.ac_option).isdigit() else (1 if mode == "full" else 0)
        for count, (key, layer) in enumerate(self.layers.items(), start=1):
            layer.recompute_ops = per_op and torch.is_grad_enabled()
            fn = layer.forward_fused
            if pg is not None:
                fn = self._gated_block(pg, f"layers.{key}", layer)
            if every and count % every == 0 and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                h, delta = checkpoint(fn, h, delta, cos, sin, use_reentrant=False)
            else:
                h, delta = fn(h, delta, cos, sin)
            if pg is not None:
                h, delta = pg.leave(f"layers.{key}", h, delta)
        if pg is not None:
            pg.acquire("post")
        if delta is None:
            return self.norm(h)
        return OF.add_rmsnorm(h, delta, self.norm.weight, self.norm.eps)[1]

    @staticmethod
    def _gated_block(pg, group: str, layer):
        def run(h, delta, cos, sin):
            if delta is None:
                h = pg.enter(group, h)
            else:
                h, delta = pg.enter(group, h, delta)
            return layer.forward_fused(h, delta, cos, sin)
        return run

    def forward(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        return self.output(self.hidden_states(tokens))

    def loss(self, tokens: torch.Tensor, labels: torch.Tensor, grad_scale: float = 1.0,
             ignore_index: int = -100) -> torch.Tensor:
        """Mean cross entropy over ``labels != ignore_index``.  The gradient that flows back is
        ``grad_scale`` times the gradient of this mean (see ``ops.functional.cross_entropy``)."""
        logits = self.forward(tokens)
        return OF.cross_entropy(logits, labels, grad_scale, ignore_index)


def build_model(args: ModelArgs | str, device=None, dtype=None, seed: int | None = 42) -> LlamaModel:
    if isinstance(args, str):
        args = PRESETS[args]
    with torch.device(device or "cpu"):
        model = LlamaModel(args)
    if dtype is not None:
        # floating-point tensors only: the complex rotary buffer keeps its dtype (checkpoint compatibility)
        model = model._apply(lambda t: t.to(dtype) if t.is_floating_point() else t)
    if seed is not None:
        model.init_weights(seed)
    return model
