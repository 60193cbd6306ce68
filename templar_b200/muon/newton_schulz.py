"""Newton–Schulz orthogonalisation for Muon on the tcgen05 GEMM.

Five quintic iterations with per-iteration coefficients (the schedule of the reference's
src/tplr/muon/newton_schulz_triton.py:336-374):

    A = X X^T                    "line 1"  -> ``gemm(X, X)``          (both operands K-major: one tensor, two roles)
    B = b A + c A A              "line 2"  -> ``gemm(A, A)`` + axpby  (A is symmetric, so A A = A A^T)
    X = a X + B X                "line 3"  -> ``gemm(B, X, b_mn=True)`` + axpby

bf16 operands, fp32 accumulation in TMEM.  The reference runs lines 1-2 as Triton kernels that compute one triangle
of the symmetric results and mirror it on the store, and line 3 through cuBLAS; here all three are the same
hand-written tcgen05 kernel, lines 1-2 in its one-triangle mode (``_ns_2d_symmetric``), and no transposed copy is
made.  ``python -m templar_b200.muon.bench`` times the variants and the reference's kernels.
Batched inputs (leading dimensions) are processed matrix by matrix.
"""

from __future__ import annotations

import torch

from ..ops import functional as OF

NS_CONSTS = [(4.0848, -6.8946, 2.9270), (3.9505, -6.3029, 2.6377), (3.7418, -5.5913, 2.3037),
             (2.8769, -3.1427, 1.2046), (2.8366, -3.0525, 1.2012)]


def _one_triangle_ok(X: torch.Tensor) -> bool:
    return (X.is_cuda and X.dtype == torch.bfloat16 and OF.gemm_backend() == "tcgen05_2sm" and X.shape[0] >= 512
            and X.shape[0] % 8 == 0 and X.shape[1] % 8 == 0 and SYMMETRIC_PRODUCTS)


SYMMETRIC_PRODUCTS = True        # lines 1 and 2 as one-triangle products (module switch, for the comparison benchmark)


class _SymmetricChain:
    """The five iterations for one matrix shape on static buffers, captured once in a CUDA graph and replayed:
    25 launches (per iteration: one-triangle X X^T, mirror, one-triangle A A, mirror with the line's scalars and the
    identity term, full product) with no host work between them.

    Lines 1 and 2 compute only the 256 x 256 tiles on or above the diagonal of their symmetric results
    (``tplr_gemm2_syrk``: half the tensor-core work) and ``tplr_sym_axpby`` mirrors the triangle while it applies
    the line's scalars.  Line 3, ``a X + B X``, is one product ``(B + a I) X``: the mirror kernel of line 2 adds
    ``a`` on the diagonal, so no element-wise pass over X remains."""

    def __init__(self, M: int, K: int, device):
        from ..ops import native

        self.M, self.K, self.native = M, K, native
        z = lambda *shape: torch.empty(*shape, dtype=torch.bfloat16, device=device)       # noqa: E731
        self.x = [z(M, K), z(M, K)]
        self.U, self.A, self.B = z(M, M), z(M, M), z(M, M)
        self.status = OF.status_word(device)
        self.graph = None
        self._run()                                    # warm-up outside the capture (first-use set-up of the kernels)
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._run()
        self.graph = g

    def _run(self) -> None:
        native, L, M, K = self.native, self.native.lib(), self.M, self.K
        st = self.status.data_ptr()
        src, dst = self.x
        for a, b, c in NS_CONSTS:
            s = native.stream_ptr()
            native.check(L.tplr_gemm2_syrk(src.data_ptr(), self.U.data_ptr(), M, K, K, M, st, s), "syrk")
            native.check(L.tplr_sym_axpby(self.U.data_ptr(), M, M, 1.0, None, 0, 0.0, 0.0, self.A.data_ptr(), M, s), "sym_axpby")
            native.check(L.tplr_gemm2_syrk(self.A.data_ptr(), self.U.data_ptr(), M, M, M, M, st, s), "syrk")   # A A = A A^T
            native.check(L.tplr_sym_axpby(self.U.data_ptr(), M, M, c, self.A.data_ptr(), M, b, a, self.B.data_ptr(), M, s),
                         "sym_axpby")
            OF.gemm(self.B, src, b_mn=True, out=dst)                                      # (B + a I) X
            src, dst = dst, src
        self.result = src

    def __call__(self, X: torch.Tensor) -> torch.Tensor:
        self.x[0].copy_(X)
        self.graph.replay()
        return self.result.clone()


_chains: dict = {}


def _ns_2d_symmetric(X: torch.Tensor) -> torch.Tensor:
    key = (X.shape[0], X.shape[1], X.device.index, torch.cuda.current_stream(X.device).cuda_stream)
    chain = _chains.get(key)
    if chain is None:
        if len(_chains) >= 32:                          # a model has a handful of matrix shapes; bound the cache anyway
            _chains.clear()
        chain = _chains[key] = _SymmetricChain(X.shape[0], X.shape[1], X.device)
    return chain(X)


def _ns_2d(G: torch.Tensor, epsilon: float) -> torch.Tensor:
    X = G.to(torch.bfloat16)
    transposed = G.size(-2) > G.size(-1)
    if transposed:
        X = X.mT
    X = (X / (X.float().norm() + epsilon).to(X.dtype)).contiguous()
    if _one_triangle_ok(X):
        X = _ns_2d_symmetric(X)
        return X.mT if transposed else X
    for a, b, c in NS_CONSTS:
        A = OF.gemm(X, X)                       # X X^T
        AA = OF.gemm(A, A)                      # A A^T = A A
        B = (b * A + c * AA).contiguous()
        X = (a * X + OF.gemm(B, X, b_mn=True)).contiguous()
    return X.mT if transposed else X


@torch.no_grad()
def newton_schulz(G: torch.Tensor, epsilon: float = 1e-7) -> torch.Tensor:
    """Approximate ``U V^T`` of ``G = U S V^T`` (singular values pushed towards 1)."""
    if G.ndim < 2:
        raise ValueError("newton_schulz needs a matrix")
    if G.ndim == 2:
        return _ns_2d(G, epsilon)
    flat = G.reshape(-1, G.size(-2), G.size(-1))
    return torch.stack([_ns_2d(g, epsilon) for g in flat]).reshape(G.shape)


def zeropower_via_newtonschulz5(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Fixed-coefficient variant ``(3.4445, -4.7750, 2.0315)`` (plain PyTorch; kept for comparison)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.bfloat16() if G.is_cuda else G.float()
    t = G.size(-2) > G.size(-1)
    if t:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.mT
        X = a * X + (b * A + c * A @ A) @ X
    return X.mT if t else X


newton_schulz_triton = newton_schulz     # the name used by callers written against the reference
