"""The allocation-free cross-entropy entry point, called through its exported C symbol.

Some embedders of the native library cannot allocate device memory at call time (all memory
belongs to another runtime's arena, or the calling thread must stay clear of cudaMalloc/cudaFree
because they synchronise the device).  For them ``tplr_cross_entropy_noalloc`` keeps its scratch
in a fixed array inside the library.  This file checks that it computes what the regular entry
point computes, twice in a row (the second call finds the first call's leftovers in the shared
array), and that it refuses shapes beyond its capacity.  It is named to be collected last, so a
run that stops at the first failure has already executed every other test.
"""

import ctypes

import pytest
import torch

from templar_b200.ops import native

pytestmark = pytest.mark.gpu


def _symbols():
    L = native.lib()
    fn = L.tplr_cross_entropy_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_longlong, ctypes.c_int,
                   ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    cap = L.tplr_cross_entropy_noalloc_max_rows
    cap.argtypes, cap.restype = [], ctypes.c_longlong
    return L, fn, cap


def _reference_call(L, logits, labels, grad_scale, write_grad):
    """The existing entry point, which takes its scratch (per-row losses, counter) from the caller."""
    T, V = logits.shape
    losses = torch.empty(T, dtype=torch.float32, device=logits.device)
    n_valid = torch.empty(1, dtype=torch.int32, device=logits.device)
    loss = torch.empty((), dtype=torch.float32, device=logits.device)
    native.check(L.tplr_cross_entropy(logits.data_ptr(), labels.data_ptr(), losses.data_ptr(), n_valid.data_ptr(),
                                      loss.data_ptr(), grad_scale, T, V, logits.stride(0), -100, int(write_grad),
                                      None, native.stream_ptr()), "cross_entropy")
    return loss


@pytest.mark.parametrize("rows,vocab", [(300, 32000), (64, 1000)])
def test_noalloc_matches_regular_entry_point_twice(rows, vocab):
    L, fn, cap = _symbols()
    assert cap() >= rows
    dev = torch.device("cuda", 0)
    for call in range(2):                       # second call reuses the array the first one wrote
        torch.manual_seed(100 + call)
        logits = (torch.randn(rows - call * 7, vocab, device=dev) * 2).to(torch.bfloat16)
        labels = torch.randint(0, vocab, (logits.shape[0],), device=dev)
        labels[::5] = -100
        if call == 1:                           # labels outside [0, vocab) behave like ignore_index, never as an index
            labels[1], labels[2] = vocab + 5, -7
        want_grad = logits.clone()
        want_loss = _reference_call(L, want_grad, labels, 0.5, True)
        got_grad = logits.clone()
        got_loss = torch.full((), float("nan"), dtype=torch.float32, device=dev)
        rc = fn(got_grad.data_ptr(), labels.data_ptr(), got_loss.data_ptr(), 0.5, logits.shape[0], vocab,
                got_grad.stride(0), -100, 1, native.stream_ptr())
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert abs(float(got_loss) - float(want_loss)) < 2e-3
        assert torch.allclose(got_grad.float(), want_grad.float(), atol=2e-5, rtol=2e-2)
        # and against the plain fp32 PyTorch loss, with the out-of-range labels masked on the host
        masked = torch.where((labels >= 0) & (labels < vocab), labels, torch.full_like(labels, -100))
        torch_loss = torch.nn.functional.cross_entropy(logits.float(), masked, ignore_index=-100)
        assert abs(float(got_loss) - float(torch_loss)) < 2e-3
        # loss-only mode leaves the logits alone
        keep = logits.clone()
        rc = fn(keep.data_ptr(), labels.data_ptr(), got_loss.data_ptr(), 1.0, logits.shape[0], vocab, keep.stride(0),
                -100, 0, native.stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(keep, logits)
        assert abs(float(got_loss) - float(want_loss)) < 2e-3


def test_noalloc_rejects_shapes_beyond_capacity():
    _, fn, cap = _symbols()
    dev = torch.device("cuda", 0)
    tiny = torch.zeros(8, 8, dtype=torch.bfloat16, device=dev)
    labels = torch.zeros(8, dtype=torch.int64, device=dev)
    out = torch.zeros((), dtype=torch.float32, device=dev)
    rc = fn(tiny.data_ptr(), labels.data_ptr(), out.data_ptr(), 1.0, cap() + 1, 8, 8, -100, 0, native.stream_ptr())
    assert rc == -201                       # TPLR_ERR_NOALLOC_TOO_LARGE, nothing launched
    rc = fn(tiny.data_ptr(), labels.data_ptr(), out.data_ptr(), 1.0, 8, 8, 7, -100, 0, native.stream_ptr())
    assert rc == -202                       # row stride must be a multiple of 8 elements
    rc = fn(tiny.data_ptr(), labels.data_ptr(), out.data_ptr(), 1.0, 8, 16, 8, -100, 0, native.stream_ptr())
    assert rc == -202                       # a row stride below the vocabulary would make rows overlap
    rc = fn(tiny.data_ptr() + 2, labels.data_ptr(), out.data_ptr(), 1.0, 4, 8, 8, -100, 0, native.stream_ptr())
    assert rc == -202                       # rows are accessed as 16-byte vectors: the base must be aligned
    torch.cuda.synchronize()
