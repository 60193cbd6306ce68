"""Tensor-parallel LLaMA on the fused all-gather->GEMM / GEMM->reduce-scatter kernels.

Same module tree and parameter names as :class:`templar_b200.models.llama.LlamaModel`, but every
rank holds only its shard of the projection weights (the reference's plan, torchtitan
models/llama3/infra/parallelize.py:151-219): wq/wk/wv and w1/w3 by output feature (whole heads),
wo and w2 by input feature, tok_embeddings and output by vocabulary row; norm weights are
replicated.  Activations between sub-layers are sharded by token ([T/world, D], sequence
parallel), so the norms and the residual stream cost 1/world per rank.

Because shard boundaries are multiples of 64 in both dimensions, the 64x64 compression chunks of a
rank's shards are exactly a subset of the chunks of the full tensors: compressing the shards is the
same per-chunk top-k as compressing the logical tensors, which is what the protocol requires.

The embedding's reduce-scatter and the vocabulary-parallel loss statistics ride on NCCL (once per
micro-batch each); the projections, which carry the traffic, use the fused kernels.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as OF
from ..parallel.tensor_parallel import (TensorParallel, all_gather_rows, column_parallel_linear,
                                        reduce_scatter_rows, row_parallel_linear)
from .llama import Attention, FeedForward, LlamaModel, ModelArgs, RMSNorm, TransformerBlock, _Weight


def _mg(w):
    return getattr(w, "main_grad", None)


class TPAttention(Attention):
    def __init__(self, args: ModelArgs, world: int):
        nn.Module.__init__(self)
        assert args.n_heads % world == 0 and args.kv_heads % world == 0, "heads must divide by the TP degree"
        self.n_heads, self.n_kv, self.hd = args.n_heads // world, args.kv_heads // world, args.head_dim
        self.wq = _Weight(self.n_heads * self.hd, args.dim)
        self.wk = _Weight(self.n_kv * self.hd, args.dim)
        self.wv = _Weight(self.n_kv * self.hd, args.dim)
        self.wo = _Weight(args.dim, self.n_heads * self.hd)
        self.packed = None
        self.tp: TensorParallel | None = None

    def forward(self, x_shard, cos, sin, B, S):
        if self.packed is not None:
            w, mg = self.packed
        else:
            w, mg = torch.cat((self.wq.weight, self.wk.weight, self.wv.weight), dim=0), None
        qkv = column_parallel_linear(x_shard, w, self.tp, mg).view(B, S, -1)
        qkv = OF.rope(qkv, cos, sin, self.n_heads + self.n_kv, self.hd)
        o = OF.attention_packed(qkv, self.n_heads, self.n_kv, self.hd)
        return row_parallel_linear(o.view(B * S, -1), self.wo.weight, self.tp, _mg(self.wo.weight))


class TPFeedForward(FeedForward):
    def __init__(self, args: ModelArgs, world: int):
        nn.Module.__init__(self)
        assert args.ffn_hidden % (64 * world) == 0, "hidden width must divide by 64 * TP degree"
        f = args.ffn_hidden // world
        self.w1 = _Weight(f, args.dim)
        self.w2 = _Weight(args.dim, f)
        self.w3 = _Weight(f, args.dim)
        self.packed = None
        self.tp: TensorParallel | None = None

    def forward(self, x_shard):
        if self.packed is not None:
            w, mg = self.packed
        else:
            w, mg = torch.cat((self.w1.weight, self.w3.weight), dim=0), None
        h = column_parallel_linear(x_shard, w, self.tp, mg)
        return row_parallel_linear(OF.swiglu(h), self.w2.weight, self.tp, _mg(self.w2.weight))


class TPTransformerBlock(TransformerBlock):
    def __init__(self, layer_id: int, args: ModelArgs, world: int):
        nn.Module.__init__(self)
        self.attention = TPAttention(args, world)
        self.feed_forward = TPFeedForward(args, world)
        self.attention_norm = RMSNorm(args.dim, args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, args.norm_eps)
        self.layer_id = layer_id
        self.weight_init_std = (0.02 / (2 * (layer_id + 1)) ** 0.5 if args.depth_init
                                else 0.02 / (2 * args.n_layers) ** 0.5)

    def forward_tp(self, res, delta, cos, sin, B, S):
        """Token-sharded residual stream ``res + delta`` in, next ``(res, delta)`` out."""
        if delta is None:
            y = self.attention_norm(res)
        else:
            res, y = OF.add_rmsnorm(res, delta, self.attention_norm.weight, self.attention_norm.eps)
        a = self.attention(y, cos, sin, B, S)
        res, y = OF.add_rmsnorm(res, a, self.ffn_norm.weight, self.ffn_norm.eps)
        return res, self.feed_forward(y)


class _VocabParallelEmbedding(torch.autograd.Function):
    """Rows of the table are split by vocabulary; output is the token shard of the summed lookup."""

    @staticmethod
    def forward(ctx, tokens, weight, rank, world, group, main_grad):
        vl = weight.shape[0]
        ids = tokens.reshape(-1) - rank * vl
        mask = (ids >= 0) & (ids < vl)
        part = weight[ids.clamp(0, vl - 1)] * mask.unsqueeze(-1).to(weight.dtype)
        out = reduce_scatter_rows(part, rank, world, group)
        ctx.save_for_backward(ids, mask)
        ctx.meta = (world, group, main_grad, weight.shape, weight.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        ids, mask = ctx.saved_tensors
        world, group, mg, shape, dtype = ctx.meta
        full = all_gather_rows(dout, world, group)
        sel = mask.nonzero(as_tuple=True)[0]
        if mg is not None:
            mg.index_add_(0, ids[sel], full[sel].to(mg.dtype))
            return None, None, None, None, None, None
        dw = torch.zeros(shape, dtype=torch.float32, device=dout.device)
        dw.index_add_(0, ids[sel], full[sel].float())
        return None, dw.to(dtype), None, None, None, None


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross entropy over labels != ignore_index with the vocabulary split over ranks.  As in the
    single-GPU loss, the logit gradient (times ``grad_scale``) is produced in the forward."""

    @staticmethod
    def forward(ctx, logits, labels, rank, group, grad_scale, ignore_index, vocab):
        vl = logits.shape[-1]
        lf = logits.float()
        n_real = min(max(vocab - rank * vl, 0), vl)         # columns of this rank that are real vocabulary entries
        if n_real < vl:
            lf[:, n_real:] = float("-inf")
        m = lf.max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m.unsqueeze(-1))
        s = e.sum(-1)
        dist.all_reduce(s, group=group)
        lab = labels.reshape(-1)
        valid = lab != ignore_index
        ids = lab - rank * vl
        mine = valid & (ids >= 0) & (ids < vl)
        tgt = torch.where(mine, lf.gather(-1, ids.clamp(0, vl - 1).unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
        dist.all_reduce(tgt, group=group)
        n = valid.sum().clamp_min(1)
        loss = ((m + torch.log(s) - tgt) * valid).sum() / n
        g = e / s.unsqueeze(-1)
        g[mine.nonzero(as_tuple=True)[0], ids[mine]] -= 1.0
        g *= (valid.to(g.dtype) * (grad_scale / n)).unsqueeze(-1)
        ctx.save_for_backward(g.to(logits.dtype))
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return g, None, None, None, None, None, None


class TPLlamaModel(LlamaModel):
    """Holds rank ``tp.rank``'s shard of a LLaMA; ``loss()`` is the training entry point."""

    def __init__(self, args: ModelArgs, tp_rank: int, tp_world: int):
        nn.Module.__init__(self)
        self.args = self.model_args = args
        self.tp_rank, self.tp_world = tp_rank, tp_world
        # the vocabulary is padded so that every rank's rows are whole 64-row chunks; padded rows are zero,
        # never indexed by a token and masked out of the softmax
        step = 64 * tp_world
        self.vocab_padded = -(-args.vocab_size // step) * step
        self.tok_embeddings = nn.Embedding(self.vocab_padded // tp_world, args.dim)
        self.layers = nn.ModuleDict({str(i): TPTransformerBlock(i, args, tp_world) for i in range(args.n_layers)})
        self.norm = RMSNorm(args.dim, args.norm_eps)
        self.output = _Weight(self.vocab_padded // tp_world, args.dim)
        self.register_buffer("freqs_cis", self._freqs_cis(), persistent=True)
        self._rope_cache: dict = {}
        self.activation_checkpointing = False
        self.tp: TensorParallel | None = None
        self.group = None

    def attach(self, tp: TensorParallel, group=None) -> None:
        """Give every parallel layer its workspace (one per model: buffers are reused layer after layer)."""
        self.tp, self.group = tp, group
        for layer in self.layers.values():
            layer.attention.tp = tp
            layer.feed_forward.tp = tp

    def replicated_parameters(self):
        """Parameters whose gradient each rank computes from its token shard only (sum over ranks needed)."""
        for name, p in self.named_parameters():
            if name.endswith("norm.weight"):
                yield name, p

    def reduce_replicated_grads(self) -> None:
        for _, p in self.replicated_parameters():
            g = getattr(p, "main_grad", None)
            if g is None:
                g = p.grad
            if g is not None:
                dist.all_reduce(g, group=self.group)

    @torch.no_grad()
    def load_from_full(self, full: LlamaModel) -> None:
        """Copy this rank's shards out of an unsharded model with the same arguments."""
        r, w = self.tp_rank, self.tp_world
        sd = full.state_dict()

        def rows(t):
            n = t.shape[0] // w
            return t[r * n:(r + 1) * n]

        def vocab_rows(t):
            n = self.vocab_padded // w
            out = torch.zeros(n, t.shape[1], dtype=t.dtype, device=t.device)
            lo, hi = r * n, min((r + 1) * n, t.shape[0])
            if hi > lo:
                out[: hi - lo] = t[lo:hi]
            return out

        def cols(t):
            n = t.shape[1] // w
            return t[:, r * n:(r + 1) * n]

        for name, p in self.named_parameters():
            src = sd[name]
            if name in ("tok_embeddings.weight", "output.weight"):
                p.copy_(vocab_rows(src))
            elif name.endswith(("wq.weight", "wk.weight", "wv.weight", "w1.weight", "w3.weight")):
                p.copy_(rows(src))
            elif name.endswith(("wo.weight", "w2.weight")):
                p.copy_(cols(src))
            else:
                p.copy_(src)

    def hidden_states(self, tokens: torch.Tensor) -> torch.Tensor:
        B, S = tokens.shape
        cos, sin = self._rope(tokens.device)
        mg = _mg(self.tok_embeddings.weight)
        h = _VocabParallelEmbedding.apply(tokens, self.tok_embeddings.weight, self.tp_rank, self.tp_world, self.group, mg)
        delta = None
        for layer in self.layers.values():
            if self.activation_checkpointing and torch.is_grad_enabled() and delta is not None:
                # the block is re-run in the backward pass, collectives included (every rank recomputes the same block)
                from torch.utils.checkpoint import checkpoint
                h, delta = checkpoint(layer.forward_tp, h, delta, cos, sin, B, S, use_reentrant=False)
            else:
                h, delta = layer.forward_tp(h, delta, cos, sin, B, S)
        return OF.add_rmsnorm(h, delta, self.norm.weight, self.norm.eps)[1]

    def forward(self, tokens: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        """Local slice [B*S, V/world] of the logits."""
        return column_parallel_linear(self.hidden_states(tokens), self.output.weight, self.tp, _mg(self.output.weight))

    def loss(self, tokens: torch.Tensor, labels: torch.Tensor, grad_scale: float = 1.0,
             ignore_index: int = -100) -> torch.Tensor:
        return _VocabParallelCE.apply(self.forward(tokens), labels, self.tp_rank, self.group, grad_scale, ignore_index,
                                      self.args.vocab_size)
