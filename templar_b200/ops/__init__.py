"""Kernels of the framework: ``functional`` (autograd ops with a CPU path), ``native``
(ctypes bindings of the sm_100a library) and ``build`` (in-tree nvcc build)."""

from .functional import (add_rmsnorm, attention, cross_entropy, embedding, gemm, gemm_backend, linear, rmsnorm, rope,
                         rope_tables, set_gemm_backend, swiglu)

__all__ = ["add_rmsnorm", "attention", "cross_entropy", "embedding", "gemm", "gemm_backend", "linear", "rmsnorm", "rope",
           "rope_tables", "set_gemm_backend", "swiglu"]
