"""ctypes bindings of ``libtplr_b200.so`` (the sm_100a kernels and the C++ runtime).

Every function takes torch CUDA tensors, checks dtype / contiguity / alignment in Python,
and launches on the current CUDA stream.  Nothing here falls back to PyTorch: callers that
want a CPU path use :mod:`templar_b200.ops.functional`, which dispatches on the device.
If a CUDA device is present but the library is missing and cannot be built, importing a
kernel raises — a silent eager fallback on a GPU box would hide that the native path is
not the one running.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build as _build

_lock = threading.Lock()
_lib = None
launch_count = 0          # number of kernel-launching native calls made by this process


class NativeError(RuntimeError):
    pass


def available() -> bool:
    """True when the shared library exists (or can be built) — says nothing about a GPU."""
    try:
        lib()
        return True
    except Exception:
        return False


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.lib_path()
            if not path.exists():
                _build.build()
            _lib = ctypes.CDLL(str(path))
            _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    vp, i, ll, f = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "tplr_param_desc_size": [],
        "tplr_compress_chunks": [vp, i, i, vp, vp, vp, vp, vp, vp, vp, f, i, i, i, i, i, vp],
        "tplr_peer_sumsq": [vp, i, i, i, vp, i, vp, i, vp, vp],
        "tplr_clip_factors": [vp, i, i, vp, vp, vp, vp, vp, vp],
        "tplr_aggregate_apply": [vp, i, i, vp, i, vp, vp, i, vp, i, i, vp, vp, vp, vp, vp, vp, f, f, i, i, i, vp, vp],
        "tplr_index_overlap": [vp, i, i, i, vp, vp, vp],
        "tplr_quantize_values": [vp, i, vp, vp, vp, vp, i, i, f, vp],
        "tplr_dequantize_values": [vp, i, vp, vp, vp, i, vp],
        "tplr_requant_residual": [vp, i, i, vp, vp, vp, vp, vp, vp, i, i, i, vp],
        "tplr_compress_chunks_tc": [vp, i, i, vp, vp, vp, vp, vp, vp, vp, f, i, i, i, vp],
        "tplr_aggregate_apply_tc": [vp, i, i, vp, i, vp, vp, i, vp, i, i, vp, vp, vp, vp, vp, vp, f, f, i, vp, vp],
        "tplr_rmsnorm_fwd": [vp, vp, vp, vp, ll, i, f, vp],
        "tplr_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, ll, i, vp],
        "tplr_add_rmsnorm_fwd": [vp, vp, vp, vp, vp, vp, ll, i, f, vp],
        "tplr_add_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, ll, i, vp],
        "tplr_add_rmsnorm_bwd_v2": [vp, vp, vp, vp, vp, vp, vp, ll, i, vp, vp],
        "tplr_rope": [vp, vp, vp, ll, i, i, i, ll, i, vp],
        "tplr_swiglu_fwd": [vp, vp, ll, i, vp],
        "tplr_swiglu_bwd": [vp, vp, vp, ll, i, vp],
        "tplr_cross_entropy": [vp, vp, vp, vp, vp, f, ll, i, ll, ll, i, vp, vp],
        "tplr_cross_entropy_noalloc": [vp, vp, vp, f, ll, i, ll, ll, i, vp],
        "tplr_embedding_fwd": [vp, vp, vp, ll, i, i, vp],
        "tplr_embedding_bwd": [vp, vp, vp, ll, i, i, vp],
        "tplr_sumsq_blocks": [],
        "tplr_sumsq": [vp, ll, vp, vp, vp],
        "tplr_adamw": [vp, vp, vp, vp, vp, i, ll, f, f, f, f, f, i, f, f, vp, i, vp],
        "tplr_cast_bf16": [vp, vp, ll, vp],
        "tplr_attention_set_bwd_variant": [i],
        "tplr_compress_set_variant": [i],
        "tplr_gemm2_swiglu": [vp, vp, vp, vp, i, i, i, ll, ll, ll, ll, vp, vp],
        "tplr_gemm2_rope": [vp, vp, vp, i, i, i, ll, ll, ll, vp, vp, i, i, i, vp, vp],
        "tplr_gemm2_swiglu_bwd": [vp, vp, vp, vp, i, i, i, ll, ll, ll, ll, vp, vp],
        "tplr_gemm2_attn_dout": [vp, vp, vp, vp, vp, i, i, i, i, ll, ll, ll, ll, vp, vp],
        "tplr_attention_bwd_unrope_delta": [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, ll, ll, f, vp, vp, vp, vp],
        "tplr_attention_bwd_unrope": [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, ll, ll, f, vp, vp, vp, vp],
        "tplr_attention_fwd": [vp, vp, vp, i, i, i, i, ll, ll, f, vp, vp],
        "tplr_attention_bwd": [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, ll, ll, f, vp, vp],
        "tplr_gemm_bf16": [vp, vp, vp, i, i, i, ll, ll, ll, i, i, i, vp, i, vp],
        "tplr_gemm2_bf16": [vp, vp, vp, i, i, i, ll, ll, ll, i, i, i, vp, i, vp],
        "tplr_gemm2_gather": [vp, vp, vp, i, i, i, ll, ll, ll, i, i, i, i, i, i, i, vp, vp, ctypes.c_uint, i, vp, vp],
        "tplr_gemm2_scatter": [vp, vp, i, i, i, ll, ll, i, i, i, i, i, vp, ll, i, vp, vp],
        "tplr_gemm2_syrk": [vp, vp, i, i, ll, ll, vp, vp],
        "tplr_sym_axpby": [vp, ll, i, f, vp, ll, f, f, vp, ll, vp],
        "tplr_gemm2_scatter_v": [vp, vp, i, i, i, ll, ll, i, i, i, i, ctypes.POINTER(c_int), vp, vp, vp],
        "tplr_copy_blocks": [vp, i, i, vp],
        "tplr_store_i64": [vp, ll, vp],
        "tplr_reduce_blocks": [vp, i, vp, i, vp, vp],
        "tplr_heap_alloc": [ctypes.c_ulonglong, ctypes.POINTER(c_void_p)],
        "tplr_heap_free": [vp],
        "tplr_ipc_handle_size": [],
        "tplr_ipc_get": [vp, ctypes.c_char_p],
        "tplr_ipc_open": [ctypes.c_char_p, ctypes.POINTER(c_void_p)],
        "tplr_ipc_close": [vp],
        "tplr_barrier": [vp, i, i, ctypes.c_ulonglong, ctypes.c_ulonglong, vp, vp],
        "tplr_reduce_shards": [vp, i, i, ll, ll, vp],
        "tplr_push_copy": [vp, vp, i, ll, vp],
    }
    for name, args in sigs.items():
        fn = getattr(L, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(err: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if err != 0:
        raise NativeError(f"{what} failed with CUDA error {err}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def ptr_array(ptrs: list[int]):
    arr = (c_void_p * len(ptrs))(*ptrs)
    return arr


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)
