"""Differentiable model ops with a hand-written sm_100a kernel behind each on CUDA.

Each op is a ``torch.autograd.Function`` whose forward/backward call the native kernels
for bf16 CUDA tensors and an equivalent plain-PyTorch expression otherwise (CPU, fp32),
so the same model code trains on a B200 and runs the CPU/gloo test tier.

Weight gradients: when a weight tensor carries a ``main_grad`` attribute (an fp32 view
into the flat gradient buffer of :class:`templar_b200.parallel.flat.FlatParamStore`) the
backward accumulates straight into it and returns ``None`` to autograd; otherwise the
gradient is returned as usual.

Reference ops replaced (torchtitan LLaMA used by the reference, models/llama3/model/model.py):
RMSNorm :276-277, RoPE :69-95, attention :185-198, SwiGLU :236-237, output + CE :351 and
components/loss.py:18-22.
"""

from __future__ import annotations


import torch
import torch.nn.functional as F

from . import native

# "tcgen05": own GEMM kernel, one CTA per tile; "tcgen05_2sm": own GEMM kernel on CTA pairs
# (cta_group::2); "cublas": torch.matmul (library).  Switched by templar_b200.ops.set_gemm_backend().
_GEMM_BACKEND = "tcgen05_2sm"
# Element-wise work folded into the projections' GEMM epilogues (SwiGLU of [w1; w3], rotary embedding of q and k).
# TPLR_FUSED_PROJECTIONS=0 runs the projection and the element-wise kernel as separate launches (comparison runs).
FUSED_PROJECTIONS = __import__("os").environ.get("TPLR_FUSED_PROJECTIONS", "1") == "1"
_status_words: dict[int, torch.Tensor] = {}


def set_gemm_backend(name: str) -> None:
    global _GEMM_BACKEND
    if name not in ("tcgen05", "tcgen05_2sm", "cublas"):
        raise ValueError(name)
    _GEMM_BACKEND = name


def gemm_backend() -> str:
    return _GEMM_BACKEND


def status_word(device) -> torch.Tensor:
    """Per-device uint32 status word the kernels OR error bits into (0 = healthy)."""
    idx = torch.device(device).index or 0
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = t
    return t


def _native_ok(*ts) -> bool:
    return all(t.is_cuda for t in ts) and all(t.dtype == torch.bfloat16 for t in ts if t.is_floating_point())


# --------------------------------------------------------------------------- #
# GEMM
# --------------------------------------------------------------------------- #
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, accumulate: bool = False,
         out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``C = op(A) op(B)^T`` with ``A``: [M,K] (or [K,M] when ``a_mn``), ``B``: [N,K] (or [K,N] when ``b_mn``).

    bf16 CUDA operands go to the tcgen05 kernel (fp32 accumulation in TMEM); ``accumulate``
    adds into an fp32 ``out``.  Rows may be strided (leading dimension), columns contiguous.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    if K != Kb:
        raise ValueError(f"gemm inner dimensions differ: {K} vs {Kb}")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else a.dtype
    use_native = (_GEMM_BACKEND != "cublas" and a.is_cuda and a.dtype == torch.bfloat16
                  and b.dtype == torch.bfloat16 and a.stride(-1) == 1 and b.stride(-1) == 1
                  and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0
                  and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
                  and out_dtype in (torch.bfloat16, torch.float32))
    if use_native:
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
            accumulate = False
        native.require(out.stride(-1) == 1 and out.shape == (M, N), "gemm: bad out")
        if accumulate and out.dtype != torch.float32:
            raise ValueError("gemm: accumulate needs an fp32 out")
        epi = 0 if out.dtype == torch.bfloat16 else (1 if accumulate else 2)
        L = native.lib()
        fn = L.tplr_gemm2_bf16 if _GEMM_BACKEND == "tcgen05_2sm" else L.tplr_gemm_bf16
        err = fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                 a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), epi,
                 status_word(a.device).data_ptr(), 0, native.stream_ptr())
        native.check(err, "tplr_gemm_bf16")
        return out
    if a.is_cuda and a.dtype == torch.bfloat16 and _GEMM_BACKEND != "cublas":
        _library_gemm_fallback(a, b)
    A = a.t() if a_mn else a
    Bt = b if b_mn else b.t()
    c = A @ Bt
    if out is None:
        return c.to(out_dtype)
    if accumulate:
        out.add_(c.to(out.dtype))
    else:
        out.copy_(c)
    return out


library_gemm_fallbacks = 0        # bf16 CUDA products that left the own kernels (reported by bench.py)
_gemm_fallback_seen: set = set()


def _library_gemm_fallback(a: torch.Tensor, b: torch.Tensor) -> None:
    """A bf16 CUDA product whose operands the own kernels cannot take (a row stride that is not a multiple of
    8 elements, a base that is not 16-byte aligned, columns not contiguous) goes to the library.  It is counted,
    said once per operand layout, and an error under ``TPLR_STRICT_NATIVE=1``: library time must not enter a
    measurement unnoticed."""
    global library_gemm_fallbacks
    import os
    import warnings

    library_gemm_fallbacks += 1
    why = (f"strides {tuple(a.stride())} / {tuple(b.stride())}, alignment {a.data_ptr() % 16} / {b.data_ptr() % 16}, "
           f"dtypes {a.dtype} / {b.dtype}")
    if os.environ.get("TPLR_STRICT_NATIVE") == "1":
        raise RuntimeError("gemm: operands outside the own tcgen05 kernels (" + why + ")")
    key = (tuple(a.stride()), tuple(b.stride()), a.data_ptr() % 16, b.data_ptr() % 16, b.dtype)
    if key not in _gemm_fallback_seen:
        _gemm_fallback_seen.add(key)
        warnings.warn("gemm: operands outside the own tcgen05 kernels (" + why + "); using torch.matmul for them",
                      stacklevel=3)


class _Linear(torch.autograd.Function):
    """y = x W^T for W [N, K]; dW goes to ``main_grad`` when given."""

    @staticmethod
    def forward(ctx, x, w, main_grad):
        ctx.save_for_backward(x, w)
        ctx.main_grad = main_grad
        x2 = x.reshape(-1, x.shape[-1])
        # the output is allocated in its final shape (not returned as a view) so that in-place
        # consumers such as RoPE may mark it dirty
        y = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        gemm(x2, w, out=y.view(-1, w.shape[0]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view_as(x)
        if ctx.main_grad is not None and not torch.is_tensor(ctx.main_grad):
            ctx.main_grad.accumulate(dy2, x2)        # sharded parameters: reduce-add into the owners' gradient shards
        elif ctx.main_grad is not None:
            gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.main_grad, accumulate=True)
        elif ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, main_grad: torch.Tensor | None = None) -> torch.Tensor:
    if main_grad is None:
        main_grad = getattr(w, "main_grad", None)
    return _Linear.apply(x, w, main_grad)


# --------------------------------------------------------------------------- #
# RMSNorm
# --------------------------------------------------------------------------- #
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, main_grad):
        ctx.eps = eps
        ctx.main_grad = main_grad
        if _native_ok(x, w) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
            xc = x.contiguous()
            T = xc.numel() // xc.shape[-1]
            y = torch.empty_like(xc)
            rstd = torch.empty(T, dtype=torch.float32, device=x.device)
            if xc.shape[-1] <= 2048:
                # rows of up to 2048 elements: the warp-per-row kernel (eight rows in flight per CTA, no block barrier)
                # with no residual to add; measured 1.6x the CTA-per-row kernel's rate at D = 2048
                native.check(native.lib().tplr_add_rmsnorm_fwd(xc.data_ptr(), None, w.data_ptr(), None, y.data_ptr(),
                                                               rstd.data_ptr(), T, xc.shape[-1], eps, native.stream_ptr()),
                             "rmsnorm_fwd")
            else:
                native.check(native.lib().tplr_rmsnorm_fwd(xc.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                                                           T, xc.shape[-1], eps, native.stream_ptr()), "rmsnorm_fwd")
            ctx.native = True
            ctx.save_for_backward(xc, w, rstd)
            return y
        ctx.native = False
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        ctx.save_for_backward(x, w, rstd)
        return (xf * rstd * w.float()).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        mg = ctx.main_grad
        if ctx.native:
            dyc = dy.contiguous()
            T, D = x.numel() // x.shape[-1], x.shape[-1]
            dx = torch.empty_like(x)
            dw_buf = mg if mg is not None else torch.zeros(D, dtype=torch.float32, device=x.device)
            if D <= 2048:
                native.check(native.lib().tplr_add_rmsnorm_bwd_v2(dyc.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None,
                                                                  dx.data_ptr(), dw_buf.data_ptr(), T, D,
                                                                  status_word(x.device).data_ptr(), native.stream_ptr()),
                             "rmsnorm_bwd")
            else:
                native.check(native.lib().tplr_rmsnorm_bwd(dyc.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                                           dx.data_ptr(), dw_buf.data_ptr(), T, D, native.stream_ptr()),
                             "rmsnorm_bwd")
            return dx, (None if mg is not None else dw_buf.to(w.dtype)), None, None
        xf, g = x.float(), dy.float()
        xh = xf * rstd
        gw = g * w.float()
        dx = rstd * (gw - xh * (gw * xh).mean(-1, keepdim=True))
        dw = (g * xh).reshape(-1, x.shape[-1]).sum(0)
        if mg is not None:
            mg.add_(dw.to(mg.dtype))
            dw = None
        else:
            dw = dw.to(w.dtype)
        return dx.to(x.dtype), dw, None, None


def rmsnorm(x, w, eps: float = 1e-5, main_grad=None):
    if main_grad is None:
        main_grad = getattr(w, "main_grad", None)
    return _RMSNorm.apply(x, w, eps, main_grad)


class _AddRMSNorm(torch.autograd.Function):
    """(h, y) = (res + delta, rmsnorm(res + delta) * w) in one kernel; the backward folds the
    residual gradient into the norm's input gradient, which serves ``res`` and ``delta`` alike."""

    @staticmethod
    def forward(ctx, res, delta, w, eps, main_grad):
        ctx.eps, ctx.main_grad = eps, main_grad
        D = res.shape[-1]
        if _native_ok(res, delta, w) and D % 8 == 0 and D <= 2048 and res.is_contiguous() and delta.is_contiguous():
            T = res.numel() // D
            h = torch.empty_like(res)
            y = torch.empty_like(res)
            rstd = torch.empty(T, dtype=torch.float32, device=res.device)
            native.check(native.lib().tplr_add_rmsnorm_fwd(res.data_ptr(), delta.data_ptr(), w.data_ptr(), h.data_ptr(),
                                                           y.data_ptr(), rstd.data_ptr(), T, D, eps, native.stream_ptr()),
                         "add_rmsnorm_fwd")
            ctx.native = 1
        elif _native_ok(res, delta, w) and D % 8 == 0 and D <= 8192:
            # wide rows: eager add, then the one-CTA-per-row norm kernels
            h = res + delta
            T = h.numel() // D
            y = torch.empty_like(h)
            rstd = torch.empty(T, dtype=torch.float32, device=res.device)
            native.check(native.lib().tplr_rmsnorm_fwd(h.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                                                       T, D, eps, native.stream_ptr()), "rmsnorm_fwd")
            ctx.native = 2
        else:
            h = res + delta
            hf = h.float()
            rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
            y = (hf * rstd * w.float()).to(res.dtype)
            ctx.native = 0
        ctx.save_for_backward(h, w, rstd)
        return h, y

    @staticmethod
    def backward(ctx, dh, dy):
        h, w, rstd = ctx.saved_tensors
        mg = ctx.main_grad
        D = h.shape[-1]
        if ctx.native == 2:
            T = h.numel() // D
            dyc = dy.contiguous()
            dx = torch.empty_like(h)
            dw_buf = mg if mg is not None else torch.zeros(D, dtype=torch.float32, device=h.device)
            native.check(native.lib().tplr_rmsnorm_bwd(dyc.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                                       dx.data_ptr(), dw_buf.data_ptr(), T, D, native.stream_ptr()),
                         "rmsnorm_bwd")
            if dh is not None:
                dx += dh
            return dx, dx, (None if mg is not None else dw_buf.to(w.dtype)), None, None
        if ctx.native:
            T = h.numel() // D
            dyc = dy.contiguous()
            dhc = dh.contiguous() if dh is not None else None
            dx = torch.empty_like(h)
            dw_buf = mg if mg is not None else torch.zeros(D, dtype=torch.float32, device=h.device)
            native.check(native.lib().tplr_add_rmsnorm_bwd_v2(dyc.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                                              dhc.data_ptr() if dhc is not None else None, dx.data_ptr(),
                                                              dw_buf.data_ptr(), T, D, status_word(h.device).data_ptr(),
                                                              native.stream_ptr()), "add_rmsnorm_bwd")
            return dx, dx, (None if mg is not None else dw_buf.to(w.dtype)), None, None
        hf, g = h.float(), dy.float()
        xh = hf * rstd
        gw = g * w.float()
        dx = rstd * (gw - xh * (gw * xh).mean(-1, keepdim=True))
        if dh is not None:
            dx = dx + dh.float()
        dw = (g * xh).reshape(-1, D).sum(0)
        if mg is not None:
            mg.add_(dw.to(mg.dtype))
            dw = None
        else:
            dw = dw.to(w.dtype)
        dx = dx.to(h.dtype)
        return dx, dx, dw, None, None


def add_rmsnorm(res, delta, w, eps: float = 1e-5, main_grad=None):
    """Returns ``(res + delta, rmsnorm(res + delta) * w)``."""
    if main_grad is None:
        main_grad = getattr(w, "main_grad", None)
    return _AddRMSNorm.apply(res, delta, w, eps, main_grad)


# --------------------------------------------------------------------------- #
# RoPE (interleaved pairs), applied to the leading rotary heads of a packed projection
# --------------------------------------------------------------------------- #
def rope_tables(seq_len: int, head_dim: int, theta: float = 10000.0, device=None):
    """cos/sin tables [S, head_dim/2] (fp32) of the angles ``pos * theta^(-2i/head_dim)``."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32)[: head_dim // 2] / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32), inv)
    return torch.cos(ang).to(device), torch.sin(ang).to(device)


def _rope_torch(x, cos, sin, n_rot_cols, head_dim, inverse):
    # x: [B, S, C]; rotate the first n_rot_cols columns head by head
    B, S, _ = x.shape
    rot = x[..., :n_rot_cols].float().reshape(B, S, n_rot_cols // head_dim, head_dim // 2, 2)
    c = cos[:S].view(1, S, 1, head_dim // 2)
    s = sin[:S].view(1, S, 1, head_dim // 2)
    if inverse:
        s = -s
    a, b = rot[..., 0], rot[..., 1]
    out = torch.stack((a * c - b * s, a * s + b * c), dim=-1).reshape(B, S, n_rot_cols)
    return torch.cat((out.to(x.dtype), x[..., n_rot_cols:]), dim=-1)


class _Rope(torch.autograd.Function):
    """On CUDA bf16 the rotation is done in place (the input is the private output of the QKV
    projection, which its producer does not need again); the backward rotates the incoming
    gradient by the opposite angle, also in place."""

    @staticmethod
    def forward(ctx, x, cos, sin, n_rot_heads, head_dim):
        ctx.save_for_backward(cos, sin)
        ctx.cfg = (n_rot_heads, head_dim)
        B, S, C = x.shape
        if _native_ok(x) and head_dim % 8 == 0 and C % 8 == 0 and x.is_contiguous():
            native.check(native.lib().tplr_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * S, S, n_rot_heads,
                                                head_dim, C, 0, native.stream_ptr()), "rope")
            ctx.mark_dirty(x)
            return x
        return _rope_torch(x, cos, sin, n_rot_heads * head_dim, head_dim, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        n_rot_heads, head_dim = ctx.cfg
        B, S, C = dy.shape
        if _native_ok(dy) and head_dim % 8 == 0 and C % 8 == 0:
            dx = dy if dy.is_contiguous() else dy.contiguous()
            native.check(native.lib().tplr_rope(dx.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * S, S, n_rot_heads,
                                                head_dim, C, 1, native.stream_ptr()), "rope_bwd")
            return dx, None, None, None, None
        return _rope_torch(dy, cos, sin, n_rot_heads * head_dim, head_dim, True), None, None, None, None


def rope(x, cos, sin, n_rot_heads: int, head_dim: int):
    """Rotate the first ``n_rot_heads`` heads of ``x`` [B, S, C] (heads laid out along C)."""
    return _Rope.apply(x, cos, sin, n_rot_heads, head_dim)


# --------------------------------------------------------------------------- #
# SwiGLU on a packed [.., 2F] projection
# --------------------------------------------------------------------------- #
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h):
        F2 = h.shape[-1]
        Fd = F2 // 2
        ctx.save_for_backward(h)
        if _native_ok(h) and Fd % 8 == 0 and h.is_contiguous():
            T = h.numel() // F2
            y = torch.empty(*h.shape[:-1], Fd, dtype=h.dtype, device=h.device)
            native.check(native.lib().tplr_swiglu_fwd(h.data_ptr(), y.data_ptr(), T, Fd, native.stream_ptr()), "swiglu_fwd")
            return y
        a, b = h[..., :Fd].float(), h[..., Fd:].float()
        return (F.silu(a) * b).to(h.dtype)

    @staticmethod
    def backward(ctx, dy):
        (h,) = ctx.saved_tensors
        F2 = h.shape[-1]
        Fd = F2 // 2
        if _native_ok(h, dy) and Fd % 8 == 0 and h.is_contiguous():
            dyc = dy.contiguous()
            dh = torch.empty_like(h)
            native.check(native.lib().tplr_swiglu_bwd(h.data_ptr(), dyc.data_ptr(), dh.data_ptr(), h.numel() // F2, Fd,
                                                      native.stream_ptr()), "swiglu_bwd")
            return dh
        a, b, g = h[..., :Fd].float(), h[..., Fd:].float(), dy.float()
        sg = torch.sigmoid(a)
        silu = a * sg
        return torch.cat((g * b * (sg + silu * (1 - sg)), g * silu), dim=-1).to(h.dtype)


def swiglu(h):
    return _SwiGLU.apply(h)


class _LinearSwiGLU(torch.autograd.Function):
    """``swiglu(x W^T)`` for the packed weight ``W = [w1; w3]``.  On the own GEMM the activation is computed in
    the projection's epilogue from the fp32 accumulators (``tplr_gemm2_swiglu``): the packed projection ``gu`` is
    still written, because the backward pass needs it, but it is not read back by a separate activation pass.
    The backward pass is the one of :class:`_SwiGLU` followed by the one of :class:`_Linear`."""

    @staticmethod
    def forward(ctx, x, w, main_grad):
        ctx.main_grad = main_grad
        F2, Fd = w.shape[0], w.shape[0] // 2
        x2 = x.reshape(-1, x.shape[-1])
        gu = torch.empty(*x.shape[:-1], F2, dtype=x.dtype, device=x.device)
        h = None
        if (FUSED_PROJECTIONS and _native_ok(x2, w) and _GEMM_BACKEND == "tcgen05_2sm" and x.dtype == torch.bfloat16 and Fd % 128 == 0
                and x2.is_contiguous() and w.stride(1) == 1 and w.stride(0) % 8 == 0 and x2.shape[1] % 8 == 0):
            h = torch.empty(*x.shape[:-1], Fd, dtype=x.dtype, device=x.device)
            rc = native.lib().tplr_gemm2_swiglu(x2.data_ptr(), w.data_ptr(), gu.data_ptr(), h.data_ptr(), x2.shape[0], Fd,
                                                x2.shape[1], x2.stride(0), w.stride(0), F2, Fd, status_word(x.device).data_ptr(),
                                                native.stream_ptr())
            if rc == -111:                      # shapes or alignment the fused entry does not take
                h = None
            else:
                native.check(rc, "gemm2_swiglu")
        if h is None:
            gemm(x2, w, out=gu.view(-1, F2))
            h = _swiglu_raw(gu)
        ctx.save_for_backward(x, w, gu)
        return h

    @staticmethod
    def backward(ctx, dh):
        x, w, gu = ctx.saved_tensors
        sw = _NoCtx()
        sw.saved_tensors = (gu,)
        with torch.no_grad():
            dgu = _SwiGLU.backward(sw, dh)
        dgu2 = dgu.reshape(-1, dgu.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = gemm(dgu2, w, b_mn=True).view_as(x) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(ctx.main_grad, dgu2, x2, w, ctx.needs_input_grad[1])
        return dx, dw, None


class _FeedForward(torch.autograd.Function):
    """``swiglu(x W13^T) W2^T`` (``W13 = [w1; w3]``) as one autograd node on the own GEMM: the activation is formed in
    the epilogue of the first projection (``tplr_gemm2_swiglu``) and its backward in the epilogue of the second
    projection's data gradient (``tplr_gemm2_swiglu_bwd``), so neither direction runs an element-wise pass over the
    [T, 2F] projection.  Saved for the backward pass: x, the packed projection and the activation (as the separate
    nodes save them)."""

    @staticmethod
    def forward(ctx, x, w13, w2, mg13, mg2):
        F2, Fd = w13.shape[0], w13.shape[0] // 2
        x2 = x.reshape(-1, x.shape[-1])
        T = x2.shape[0]
        st = status_word(x.device).data_ptr()
        gu = torch.empty(T, F2, dtype=x.dtype, device=x.device)
        h = torch.empty(T, Fd, dtype=x.dtype, device=x.device)
        native.check(native.lib().tplr_gemm2_swiglu(x2.data_ptr(), w13.data_ptr(), gu.data_ptr(), h.data_ptr(), T, Fd,
                                                    x2.shape[1], x2.stride(0), w13.stride(0), F2, Fd, st, native.stream_ptr()),
                     "gemm2_swiglu")
        y = torch.empty(*x.shape[:-1], w2.shape[0], dtype=x.dtype, device=x.device)
        gemm(h, w2, out=y.view(-1, w2.shape[0]))
        ctx.save_for_backward(x, w13, w2, gu, h)
        ctx.mg = (mg13, mg2)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w13, w2, gu, h = ctx.saved_tensors
        mg13, mg2 = ctx.mg
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        T, Fd = gu.shape[0], gu.shape[1] // 2
        dgu = torch.empty_like(gu)
        native.check(native.lib().tplr_gemm2_swiglu_bwd(dy2.data_ptr(), w2.data_ptr(), gu.data_ptr(), dgu.data_ptr(), T, Fd,
                                                        dy2.shape[1], dy2.stride(0), w2.stride(0), gu.stride(0), dgu.stride(0),
                                                        status_word(x.device).data_ptr(), native.stream_ptr()),
                     "gemm2_swiglu_bwd")
        dw2 = _weight_grad(mg2, dy2, h, w2, ctx.needs_input_grad[2])
        dx = gemm(dgu, w13, b_mn=True).view_as(x) if ctx.needs_input_grad[0] else None
        dw13 = _weight_grad(mg13, dgu, x2, w13, ctx.needs_input_grad[1])
        return dx, dw13, dw2, None, None


def feed_forward(x, w13, w2, main_grad13=None, main_grad2=None):
    """``(silu(x w1^T) * (x w3^T)) w2^T`` for the packed ``w13 = [w1; w3]`` ([2F, D]) and ``w2`` [D, F]."""
    if main_grad13 is None:
        main_grad13 = getattr(w13, "main_grad", None)
    if main_grad2 is None:
        main_grad2 = getattr(w2, "main_grad", None)
    Fd = w13.shape[0] // 2
    x2 = x.reshape(-1, x.shape[-1])
    if (FUSED_PROJECTIONS and _GEMM_BACKEND == "tcgen05_2sm" and _native_ok(x2, w13, w2) and x.dtype == torch.bfloat16
            and Fd % 128 == 0 and x2.is_contiguous() and w13.stride(1) == 1 and w2.stride(1) == 1 and w13.stride(0) % 8 == 0
            and w2.stride(0) % 8 == 0 and x2.shape[1] % 8 == 0 and w2.shape[0] % 8 == 0
            and all(t.data_ptr() % 16 == 0 for t in (x2, w13, w2))):
        return _FeedForward.apply(x, w13, w2, main_grad13, main_grad2)
    return _Linear.apply(linear_swiglu(x, w13, main_grad13), w2, main_grad2)


def linear_swiglu(x, w, main_grad=None):
    """``silu(x w1^T) * (x w3^T)`` for the packed ``w = [w1; w3]`` ([2F, K]); one GEMM launch on CUDA."""
    if main_grad is None:
        main_grad = getattr(w, "main_grad", None)
    return _LinearSwiGLU.apply(x, w, main_grad)


# --------------------------------------------------------------------------- #
# Per-op selective activation checkpointing: the outputs of GEMMs and of attention are kept, the
# cheap element-wise producers of a GEMM's input (SwiGLU, RMSNorm) are recomputed in the backward
# pass instead of being stored.  The reference gets the same policy from torchtitan's selective
# "op" mode, which saves matmul / attention results and recomputes the rest
# (models/llama3/infra/parallelize.py:234-322, hparams torchtitan.activation_checkpoint).
# --------------------------------------------------------------------------- #
def _swiglu_raw(h: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return _SwiGLU.forward(_NoCtx(), h)


def _weight_grad(main_grad, dy2, x2, w, needs_grad: bool):
    """dW of ``y = x W^T`` routed like :class:`_Linear` does: into ``main_grad`` (fp32 buffer or gradient
    scatter target) when there is one, else returned."""
    if main_grad is not None and not torch.is_tensor(main_grad):
        main_grad.accumulate(dy2, x2)
        return None
    if main_grad is not None:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype) if needs_grad else None


class _NoCtx:
    """Stand-in context for calling a Function's forward as a plain computation."""

    needs_input_grad = (False,) * 8

    def save_for_backward(self, *a):
        self.saved = a

    def mark_dirty(self, *a):
        pass


class _SwiGLULinear(torch.autograd.Function):
    """``y = swiglu(h) W^T`` that stores ``h`` only: the activation ``swiglu(h)`` (a third of a block's stored
    activations) is recomputed for the weight gradient."""

    @staticmethod
    def forward(ctx, h, w, main_grad):
        ctx.save_for_backward(h, w)
        ctx.main_grad = main_grad
        s = _swiglu_raw(h)
        y = torch.empty(*s.shape[:-1], w.shape[0], dtype=s.dtype, device=s.device)
        gemm(s.reshape(-1, s.shape[-1]), w, out=y.view(-1, w.shape[0]))
        return y

    @staticmethod
    def backward(ctx, dy):
        h, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        s = _swiglu_raw(h)
        s2 = s.reshape(-1, s.shape[-1])
        ds = gemm(dy2, w, b_mn=True).view_as(s)
        dw = _weight_grad(ctx.main_grad, dy2, s2, w, ctx.needs_input_grad[1])
        del s, s2
        sw = _NoCtx()
        sw.saved_tensors = (h,)
        with torch.no_grad():
            dh = _SwiGLU.backward(sw, ds)
        return dh, dw, None


def swiglu_linear(h, w, main_grad=None):
    """``swiglu(h) @ w.T`` with the activation recomputed in the backward pass."""
    if main_grad is None:
        main_grad = getattr(w, "main_grad", None)
    return _SwiGLULinear.apply(h, w, main_grad)


class _NormLinear(torch.autograd.Function):
    """``(hsum, y)`` with ``hsum = res + delta`` (``delta`` may be None) and ``y = rmsnorm(hsum) W^T``; stores
    ``hsum`` (needed by the residual stream anyway) and the row statistics, not the normalised activations."""

    @staticmethod
    def forward(ctx, res, delta, wn, eps, main_grad_n, w, main_grad_w):
        nctx = _NoCtx()
        with torch.no_grad():
            if delta is None:
                xn = _RMSNorm.forward(nctx, res, wn, eps, None)
                hsum = res
            else:
                hsum, xn = _AddRMSNorm.forward(nctx, res, delta, wn, eps, None)
        ctx.kind = "plain" if delta is None else "add"
        ctx.native = nctx.native
        ctx.eps, ctx.main_grad_n, ctx.main_grad_w = eps, main_grad_n, main_grad_w
        ctx.save_for_backward(*nctx.saved, w)              # (x or h, wn, rstd, w)
        y = torch.empty(*xn.shape[:-1], w.shape[0], dtype=xn.dtype, device=xn.device)
        gemm(xn.reshape(-1, xn.shape[-1]), w, out=y.view(-1, w.shape[0]))
        if delta is None:
            return y
        return hsum, y

    @staticmethod
    def backward(ctx, *grads):
        x, wn, rstd, w = ctx.saved_tensors
        dh, dy = (None, grads[0]) if ctx.kind == "plain" else grads
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        # the normalised activations again (one pass over x), for the weight gradient only
        with torch.no_grad():
            if ctx.native and x.is_contiguous() and x.shape[-1] <= 8192:
                xn = torch.empty_like(x)
                T = x.numel() // x.shape[-1]
                native.check(native.lib().tplr_rmsnorm_fwd(x.data_ptr(), wn.data_ptr(), xn.data_ptr(), rstd.data_ptr(), T,
                                                           x.shape[-1], ctx.eps, native.stream_ptr()), "rmsnorm_fwd")
            else:
                xn = (x.float() * rstd.reshape(*x.shape[:-1], 1) * wn.float()).to(x.dtype)
        dw = _weight_grad(ctx.main_grad_w, dy2, xn.reshape(-1, xn.shape[-1]), w, ctx.needs_input_grad[5])
        del xn
        dxn = gemm(dy2, w, b_mn=True).view_as(x)
        nctx = _NoCtx()
        nctx.saved_tensors, nctx.main_grad, nctx.native, nctx.eps = (x, wn, rstd), ctx.main_grad_n, ctx.native, ctx.eps
        with torch.no_grad():
            if ctx.kind == "plain":
                dx, dwn, _, _ = _RMSNorm.backward(nctx, dxn)
                return dx, None, dwn, None, None, dw, None
            dx, _, dwn, _, _ = _AddRMSNorm.backward(nctx, dh, dxn)
        return dx, dx, dwn, None, None, dw, None


def norm_linear(res, delta, wn, eps, w, main_grad_w=None):
    """``rmsnorm(res + delta) @ w.T`` (and the sum, when ``delta`` is given) with the normalised activations
    recomputed in the backward pass."""
    if main_grad_w is None:
        main_grad_w = getattr(w, "main_grad", None)
    return _NormLinear.apply(res, delta, wn, eps, getattr(wn, "main_grad", None), w, main_grad_w)


# --------------------------------------------------------------------------- #
# Embedding
# --------------------------------------------------------------------------- #
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, table, main_grad):
        ctx.save_for_backward(tokens)
        ctx.main_grad = main_grad
        ctx.tshape = table.shape
        ctx.tdtype = table.dtype
        if _native_ok(table) and table.shape[1] % 8 == 0 and table.is_contiguous():
            tok = tokens.contiguous().to(torch.int64)
            out = torch.empty(*tokens.shape, table.shape[1], dtype=table.dtype, device=table.device)
            native.check(native.lib().tplr_embedding_fwd(tok.data_ptr(), table.data_ptr(), out.data_ptr(), tok.numel(),
                                                         table.shape[1], table.shape[0], native.stream_ptr()), "embedding_fwd")
            return out
        return F.embedding(tokens, table)

    @staticmethod
    def backward(ctx, dy):
        (tokens,) = ctx.saved_tensors
        V, D = ctx.tshape
        mg = ctx.main_grad
        if mg is not None and dy.is_cuda and dy.dtype == torch.bfloat16 and D % 8 == 0:
            dyc = dy.contiguous()
            tok = tokens.contiguous().to(torch.int64)
            native.check(native.lib().tplr_embedding_bwd(tok.data_ptr(), dyc.data_ptr(), mg.data_ptr(), tok.numel(), D, V,
                                                         native.stream_ptr()), "embedding_bwd")
            return None, None, None
        grad = torch.zeros(V, D, dtype=torch.float32, device=dy.device)
        grad.index_add_(0, tokens.reshape(-1), dy.reshape(-1, D).float())
        if mg is not None:
            mg.add_(grad.to(mg.dtype))
            return None, None, None
        return None, grad.to(ctx.tdtype), None


def embedding(tokens, table, main_grad=None):
    if main_grad is None:
        main_grad = getattr(table, "main_grad", None)
    return _Embedding.apply(tokens, table, main_grad)


# --------------------------------------------------------------------------- #
# Attention (causal, GQA)
# --------------------------------------------------------------------------- #
def attention(q, k, v):
    """Causal attention on [B, S, H, Dh] / [B, S, KV, Dh] tensors (strided views allowed)."""
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    gqa = kh.shape[1] != qh.shape[1]
    if gqa and not q.is_cuda:
        rep = qh.shape[1] // kh.shape[1]
        kh = kh.repeat_interleave(rep, dim=1)
        vh = vh.repeat_interleave(rep, dim=1)
        gqa = False
    o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=gqa)
    return o.transpose(1, 2)


_ATTN_BACKEND = "tcgen05"      # "tcgen05": own flash-attention kernels; "sdpa": torch SDPA (library)


def set_attention_backend(name: str) -> None:
    global _ATTN_BACKEND
    if name not in ("tcgen05", "sdpa"):
        raise ValueError(name)
    _ATTN_BACKEND = name


def attention_backend() -> str:
    return _ATTN_BACKEND


def _split_qkv(qkv, n_heads, n_kv, hd):
    B, S, _ = qkv.shape
    nq, nk = n_heads * hd, n_kv * hd
    return (qkv[..., :nq].view(B, S, n_heads, hd), qkv[..., nq:nq + nk].view(B, S, n_kv, hd),
            qkv[..., nq + nk:].view(B, S, n_kv, hd))


class _AttentionPacked(torch.autograd.Function):
    """Causal GQA attention on the packed projection output [B, S, (H + 2 KV) * 128]; the backward
    returns the gradient in the same packed layout, so nothing splits or concatenates q, k and v."""

    @staticmethod
    def forward(ctx, qkv, n_heads, n_kv, hd):
        B, S, C = qkv.shape
        out = torch.empty(B, S, n_heads * hd, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(B, n_heads, S, dtype=torch.float32, device=qkv.device)
        native.check(native.lib().tplr_attention_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, n_heads, n_kv,
                                                     qkv.stride(1), out.stride(1), hd ** -0.5,
                                                     status_word(qkv.device).data_ptr(), native.stream_ptr()),
                     "attention_fwd")
        ctx.save_for_backward(qkv, out, lse)
        ctx.dims = (n_heads, n_kv, hd)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        n_heads, n_kv, hd = ctx.dims
        B, S, C = qkv.shape
        do = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dq32 = torch.zeros(B, S, n_heads * hd, dtype=torch.float32, device=qkv.device)
        delta = torch.empty(B, n_heads, S, dtype=torch.float32, device=qkv.device)
        native.check(native.lib().tplr_attention_bwd(qkv.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                                     delta.data_ptr(), dq32.data_ptr(), dqkv.data_ptr(), B, S, n_heads, n_kv,
                                                     qkv.stride(1), out.stride(1), hd ** -0.5,
                                                     status_word(qkv.device).data_ptr(), native.stream_ptr()),
                     "attention_bwd")
        return dqkv, None, None, None


class _QKVRopeAttention(torch.autograd.Function):
    """``attention(rope(x W^T))`` for the packed ``W = [wq; wk; wv]`` as one autograd node on the own kernels:
    the rotary embedding is applied to the q and k columns in the projection's epilogue (``tplr_gemm2_rope``) and
    undone for dq and dk where the attention backward writes them (``tplr_attention_bwd_unrope``), so neither
    pass runs a separate rotation over the projection or its gradient.  One node, because the gradient that
    leaves the attention backward is already the one of the un-rotated projection."""

    @staticmethod
    def forward(ctx, x, w, main_grad, cos, sin, n_heads, n_kv, hd):
        B, S, _ = x.shape
        C = w.shape[0]
        x2 = x.reshape(-1, x.shape[-1])
        qkv = torch.empty(B, S, C, dtype=x.dtype, device=x.device)
        st = status_word(x.device).data_ptr()
        L = native.lib()
        native.check(L.tplr_gemm2_rope(x2.data_ptr(), w.data_ptr(), qkv.data_ptr(), x2.shape[0], C, x2.shape[1], x2.stride(0),
                                       w.stride(0), C, cos.data_ptr(), sin.data_ptr(), S, (n_heads + n_kv) * hd, hd, st,
                                       native.stream_ptr()), "gemm2_rope")
        out = torch.empty(B, S, n_heads * hd, dtype=x.dtype, device=x.device)
        lse = torch.empty(B, n_heads, S, dtype=torch.float32, device=x.device)
        native.check(L.tplr_attention_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, n_heads, n_kv, qkv.stride(1),
                                          out.stride(1), hd ** -0.5, st, native.stream_ptr()), "attention_fwd")
        ctx.save_for_backward(x, w, qkv, out, lse, cos, sin)
        ctx.main_grad, ctx.dims = main_grad, (n_heads, n_kv, hd)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w, qkv, out, lse, cos, sin = ctx.saved_tensors
        n_heads, n_kv, hd = ctx.dims
        B, S, C = qkv.shape
        do = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dq32 = torch.zeros(B, S, n_heads * hd, dtype=torch.float32, device=qkv.device)
        delta = torch.empty(B, n_heads, S, dtype=torch.float32, device=qkv.device)
        native.check(native.lib().tplr_attention_bwd_unrope(
            qkv.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq32.data_ptr(), dqkv.data_ptr(),
            B, S, n_heads, n_kv, qkv.stride(1), out.stride(1), hd ** -0.5, cos.data_ptr(), sin.data_ptr(),
            status_word(qkv.device).data_ptr(), native.stream_ptr()), "attention_bwd_unrope")
        del dq32, delta
        d2 = dqkv.view(-1, C)
        x2 = x.reshape(-1, x.shape[-1])
        dx = gemm(d2, w, b_mn=True).view_as(x) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(ctx.main_grad, d2, x2, w, ctx.needs_input_grad[1])
        return dx, dw, None, None, None, None, None, None


class _AttentionBlock(torch.autograd.Function):
    """``attention(rope(x Wqkv^T)) Wo^T`` as one autograd node on the own kernels.  Beyond :class:`_QKVRopeAttention`
    (rotation in the projection's epilogue, inverse rotation in the attention backward's outputs) the output projection
    belongs to the node, so that its data gradient ``dO = dY Wo`` can form the attention backward's ``delta`` term (the
    row sum of dO * O per head) in its epilogue (``tplr_gemm2_attn_dout``) instead of a separate pass over dO and O."""

    @staticmethod
    def forward(ctx, x, wqkv, wo, mg_qkv, mg_wo, cos, sin, n_heads, n_kv, hd):
        B, S, _ = x.shape
        C = wqkv.shape[0]
        x2 = x.reshape(-1, x.shape[-1])
        st = status_word(x.device).data_ptr()
        L = native.lib()
        qkv = torch.empty(B, S, C, dtype=x.dtype, device=x.device)
        native.check(L.tplr_gemm2_rope(x2.data_ptr(), wqkv.data_ptr(), qkv.data_ptr(), x2.shape[0], C, x2.shape[1], x2.stride(0),
                                       wqkv.stride(0), C, cos.data_ptr(), sin.data_ptr(), S, (n_heads + n_kv) * hd, hd, st,
                                       native.stream_ptr()), "gemm2_rope")
        out = torch.empty(B, S, n_heads * hd, dtype=x.dtype, device=x.device)
        lse = torch.empty(B, n_heads, S, dtype=torch.float32, device=x.device)
        native.check(L.tplr_attention_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, n_heads, n_kv, qkv.stride(1),
                                          out.stride(1), hd ** -0.5, st, native.stream_ptr()), "attention_fwd")
        y = torch.empty(B, S, wo.shape[0], dtype=x.dtype, device=x.device)
        gemm(out.view(-1, n_heads * hd), wo, out=y.view(-1, wo.shape[0]))
        ctx.save_for_backward(x, wqkv, wo, qkv, out, lse, cos, sin)
        ctx.mg, ctx.dims = (mg_qkv, mg_wo), (n_heads, n_kv, hd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wqkv, wo, qkv, out, lse, cos, sin = ctx.saved_tensors
        mg_qkv, mg_wo = ctx.mg
        n_heads, n_kv, hd = ctx.dims
        B, S, C = qkv.shape
        T, N = B * S, n_heads * hd
        L = native.lib()
        st = status_word(qkv.device).data_ptr()
        dy2 = dy.reshape(T, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        out2 = out.view(T, N)
        do = torch.empty(T, N, dtype=qkv.dtype, device=qkv.device)
        delta = torch.empty(B, n_heads, S, dtype=torch.float32, device=qkv.device)
        native.check(L.tplr_gemm2_attn_dout(dy2.data_ptr(), wo.data_ptr(), out2.data_ptr(), do.data_ptr(), delta.data_ptr(), T, N,
                                            dy2.shape[1], S, dy2.stride(0), wo.stride(0), out2.stride(0), do.stride(0), st,
                                            native.stream_ptr()), "gemm2_attn_dout")
        dwo = _weight_grad(mg_wo, dy2, out2, wo, ctx.needs_input_grad[2])
        dqkv = torch.empty_like(qkv)
        dq32 = torch.zeros(B, S, N, dtype=torch.float32, device=qkv.device)
        native.check(L.tplr_attention_bwd_unrope_delta(
            qkv.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq32.data_ptr(), dqkv.data_ptr(),
            B, S, n_heads, n_kv, qkv.stride(1), out.stride(1), hd ** -0.5, cos.data_ptr(), sin.data_ptr(), st,
            native.stream_ptr()), "attention_bwd_unrope_delta")
        del dq32, delta, do
        d2 = dqkv.view(T, C)
        x2 = x.reshape(T, x.shape[-1])
        dx = gemm(d2, wqkv, b_mn=True).view_as(x) if ctx.needs_input_grad[0] else None
        dwqkv = _weight_grad(mg_qkv, d2, x2, wqkv, ctx.needs_input_grad[1])
        return dx, dwqkv, dwo, None, None, None, None, None, None, None


def attention_block(x, wqkv, wo, cos, sin, n_heads: int, n_kv: int, hd: int, main_grad_qkv=None, main_grad_wo=None):
    """Causal attention block without its norm and residual: ``attention(rope(x @ wqkv.T)) @ wo.T`` for the packed
    ``wqkv = [wq; wk; wv]``.  One autograd node on the own kernels, three elsewhere."""
    if main_grad_qkv is None:
        main_grad_qkv = getattr(wqkv, "main_grad", None)
    if main_grad_wo is None:
        main_grad_wo = getattr(wo, "main_grad", None)
    B, S, K = x.shape
    if (FUSED_PROJECTIONS and _ATTN_BACKEND == "tcgen05" and _GEMM_BACKEND == "tcgen05_2sm" and _native_ok(x, wqkv, wo)
            and x.dtype == torch.bfloat16 and hd == 128 and S % 128 == 0 and n_heads % n_kv == 0 and x.is_contiguous()
            and wqkv.stride(1) == 1 and wo.stride(1) == 1 and wqkv.stride(0) % 8 == 0 and wo.stride(0) % 8 == 0 and K % 8 == 0
            and wo.shape[0] % 8 == 0 and wo.shape[1] == n_heads * hd and cos.is_cuda and cos.dtype == torch.float32
            and cos.is_contiguous() and sin.is_contiguous() and cos.shape[0] >= S and cos.shape[1] == hd // 2
            and all(t.data_ptr() % 16 == 0 for t in (x, wqkv, wo, cos, sin))):
        return _AttentionBlock.apply(x, wqkv, wo, main_grad_qkv, main_grad_wo, cos, sin, n_heads, n_kv, hd)
    return _Linear.apply(rope_attention_projection(x, wqkv, cos, sin, n_heads, n_kv, hd, main_grad_qkv), wo, main_grad_wo)


def rope_attention_projection(x, w, cos, sin, n_heads: int, n_kv: int, hd: int, main_grad=None):
    """Causal attention of the rotary-embedded packed projection ``x @ w.T`` (``w = [wq; wk; wv]``); returns
    [B, S, H * hd].  On the own kernels this is one autograd node with the rotation inside the GEMM and attention
    kernels; elsewhere the projection, the rotation and the attention are three."""
    if main_grad is None:
        main_grad = getattr(w, "main_grad", None)
    B, S, K = x.shape
    if (FUSED_PROJECTIONS and _ATTN_BACKEND == "tcgen05" and _GEMM_BACKEND == "tcgen05_2sm" and _native_ok(x, w) and x.dtype == torch.bfloat16
            and hd == 128 and S % 128 == 0 and n_heads % n_kv == 0 and x.is_contiguous() and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and K % 8 == 0 and w.shape[0] % 8 == 0 and cos.is_cuda and cos.dtype == torch.float32
            and cos.is_contiguous() and sin.is_contiguous() and cos.shape[0] >= S and cos.shape[1] == hd // 2
            and cos.data_ptr() % 16 == 0 and sin.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return _QKVRopeAttention.apply(x, w, main_grad, cos, sin, n_heads, n_kv, hd)
    qkv = rope(_Linear.apply(x, w, main_grad), cos, sin, n_heads + n_kv, hd)
    return attention_packed(qkv, n_heads, n_kv, hd)


_attn_fallback_seen: set = set()


def attention_packed(qkv, n_heads: int, n_kv: int, hd: int):
    """Causal attention of ``qkv`` [B, S, (H + 2 KV) * hd] (q heads, k heads, v heads); returns [B, S, H * hd]."""
    B, S, C = qkv.shape
    if (_ATTN_BACKEND == "tcgen05" and qkv.is_cuda and qkv.dtype == torch.bfloat16 and hd == 128 and S % 128 == 0
            and n_heads % n_kv == 0 and qkv.stride(2) == 1 and qkv.stride(0) == S * qkv.stride(1)
            and qkv.stride(1) % 8 == 0 and qkv.data_ptr() % 16 == 0):
        return _AttentionPacked.apply(qkv, n_heads, n_kv, hd)
    if _ATTN_BACKEND == "tcgen05" and qkv.is_cuda and (hd, S % 128) not in _attn_fallback_seen:
        # said once per shape class: a GPU run that silently uses the library kernel would misreport what ran
        _attn_fallback_seen.add((hd, S % 128))
        import warnings

        warnings.warn(f"attention_packed: head_dim {hd}, sequence {S}, dtype {qkv.dtype} is outside the own flash-attention "
                      f"kernels (bf16, head_dim 128, sequence a multiple of 128); using torch SDPA for it", stacklevel=2)
    q, k, v = _split_qkv(qkv, n_heads, n_kv, hd)
    return attention(q, k, v).reshape(B, S, n_heads * hd)


# --------------------------------------------------------------------------- #
# Cross entropy with the logit gradient produced in the forward pass
# --------------------------------------------------------------------------- #
class _CrossEntropy(torch.autograd.Function):
    """Mean CE over labels != ignore_index.  The backward assumes the loss is the root of the
    graph: the gradient ``(softmax - onehot) * grad_scale / n_valid`` is computed in the
    forward kernel, in place in the logits buffer, and ``grad_scale`` replaces the incoming
    ``grad_output`` (no extra pass over the logits, no host sync)."""

    @staticmethod
    def forward(ctx, logits, labels, grad_scale, ignore_index):
        T = labels.numel()
        V = logits.shape[-1]
        lg = logits.reshape(T, V)
        if (_native_ok(lg) and lg.stride(-1) == 1 and lg.stride(0) % 8 == 0 and lg.stride(0) >= V
                and lg.data_ptr() % 16 == 0):
            lab = labels.reshape(-1).contiguous().to(torch.int64)
            losses = torch.empty(T, dtype=torch.float32, device=lg.device)
            nvalid = torch.empty(1, dtype=torch.int32, device=lg.device)
            loss = torch.empty((), dtype=torch.float32, device=lg.device)
            want_grad = ctx.needs_input_grad[0]
            native.check(native.lib().tplr_cross_entropy(lg.data_ptr(), lab.data_ptr(), losses.data_ptr(), nvalid.data_ptr(),
                                                         loss.data_ptr(), float(grad_scale), T, V, lg.stride(0),
                                                         int(ignore_index), int(want_grad),
                                                         status_word(lg.device).data_ptr(), native.stream_ptr()),
                         "cross_entropy")
            # the logits buffer now holds d(loss)/d(logits); it is handed to autograd in backward
            ctx.inplace = True
            ctx.shape = logits.shape
            ctx.dlogits = lg
            return loss
        ctx.inplace = False
        ctx.grad_scale = grad_scale
        ctx.ignore_index = ignore_index
        ctx.shape = logits.shape
        ctx.save_for_backward(lg, labels.reshape(-1))
        return F.cross_entropy(lg.float(), labels.reshape(-1), ignore_index=ignore_index)

    @staticmethod
    def backward(ctx, dloss):
        if ctx.inplace:
            return ctx.dlogits.view(ctx.shape), None, None, None
        lg, labels = ctx.saved_tensors
        lf = lg.float()
        valid = labels != ctx.ignore_index
        n = valid.sum().clamp(min=1)
        p = torch.softmax(lf, dim=-1)
        p[valid, labels[valid]] -= 1.0
        p[~valid] = 0
        return (p * (ctx.grad_scale / n)).to(lg.dtype).view(ctx.shape), None, None, None


def cross_entropy(logits, labels, grad_scale: float = 1.0, ignore_index: int = -100):
    return _CrossEntropy.apply(logits, labels, grad_scale, ignore_index)
