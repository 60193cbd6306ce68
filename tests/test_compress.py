"""CPU tests of the compression spec: 12-bit packing, chunk geometry, DCT, top-k, quantisation,
batch decompress.  Mirrors the cases of the reference's tests/unit/test_compress.py."""

import math

import pytest
import torch

from templar_b200 import compress as C


class _M(torch.nn.Module):
    def __init__(self, shapes):
        super().__init__()
        self.ps = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(*s)) for s in shapes])


def test_pack_unpack_roundtrip_and_size():
    idx = torch.randint(0, 4096, (7, 5, 32))
    packed = C.pack_12bit_indices(idx)
    assert packed.dtype == torch.uint8 and packed.numel() == idx.numel() * 3 // 2
    assert torch.equal(C.unpack_12bit_indices(packed, idx.shape), idx)
    assert packed.numel() * 1 == int(idx.numel() * 2 * 0.75)      # 25 % smaller than int16


def test_pack_bit_layout():
    packed = C.pack_12bit_indices(torch.tensor([0xABC, 0x123]))
    assert packed.tolist() == [0xBC, 0xA | (0x3 << 4), 0x12]


def test_pack_rejects_odd_and_large():
    with pytest.raises(ValueError):
        C.pack_12bit_indices(torch.tensor([1, 2, 3]))
    with pytest.raises(ValueError):
        C.pack_12bit_indices(torch.tensor([1, 4096]))
    with pytest.raises(ValueError):
        C.unpack_12bit_indices(torch.zeros(3, dtype=torch.uint8), (3,))


def test_pack_empty_and_device():
    assert C.pack_12bit_indices(torch.zeros(0, dtype=torch.int64)).numel() == 0
    assert C.unpack_12bit_indices(torch.zeros(0, dtype=torch.uint8), (0, 4)).shape == (0, 4)


@pytest.mark.parametrize("n,target,want", [(64, 64, 64), (2048, 64, 64), (96, 64, 48), (100, 64, 50), (7, 64, 7),
                                           (127, 64, 1), (32000, 64, 64), (28672, 64, 64), (130, 64, 26)])
def test_chunk_size(n, target, want):
    assert C.chunk_size_for(n, target) == want
    assert C._get_smaller_split(n, target) == want


@pytest.mark.parametrize("n", [1, 2, 8, 48, 64])
def test_dct_basis_is_orthonormal_and_matches_scipy_definition(n):
    f = C.dct_basis(n, dtype=torch.float64)
    assert torch.allclose(f @ f.T, torch.eye(n, dtype=torch.float64), atol=1e-12)
    x = torch.randn(3, n, dtype=torch.float64)
    y = C._dct(x, norm="ortho")
    k = torch.arange(n, dtype=torch.float64)
    ref = torch.stack([(x * torch.cos(math.pi * (2 * k + 1) * kk / (2 * n))).sum(-1) * math.sqrt(2 / n) *
                       (math.sqrt(0.5) if kk == 0 else 1.0) for kk in range(n)], dim=-1)
    assert torch.allclose(y, ref, atol=1e-10)
    assert torch.allclose(C._idct(y, norm="ortho"), x, atol=1e-10)
    assert torch.allclose(C._idct(C._dct(x)), x, atol=1e-9)      # unnormalised pair is also inverse


@pytest.mark.parametrize("shape", [(128, 192), (96, 40), (256,), (130,)])
@pytest.mark.parametrize("use_dct", [False, True])
def test_encode_decode_roundtrip(shape, use_dct):
    m = _M([shape])
    tr = C.ChunkingTransformer(m, 64)
    x = torch.randn(*shape)
    enc = tr.encode(x, use_dct=use_dct)
    if len(shape) == 2:
        assert enc.shape == (shape[0] // tr.shape_dict[shape[0]], shape[1] // tr.shape_dict[shape[1]],
                             tr.shape_dict[shape[0]], tr.shape_dict[shape[1]])
    assert torch.allclose(tr.decode(enc, use_dct=use_dct), x, atol=1e-5)
    if use_dct:      # energy preserving
        assert torch.allclose(enc.pow(2).sum(), x.pow(2).sum(), rtol=1e-4)


def test_compress_contract_and_decompress():
    m = _M([(128, 128), (64,)])
    tr = C.ChunkingTransformer(m, 64)
    comp = C.TopKCompressor()
    x = torch.randn(128, 128)
    enc = tr.encode(x, use_dct=True)
    idx, val, xshape, totalk = comp.compress(enc, 32)
    assert idx.dtype == torch.uint8 and val.shape == (2, 2, 32) and totalk == 4096 and tuple(xshape) == (2, 2, 64, 64)
    dense = comp.decompress(x, idx, val, xshape, totalk)
    assert dense.shape == enc.shape
    flat = enc.reshape(2, 2, -1)
    thr = flat.abs().topk(32, dim=-1).values[..., -1:]
    assert torch.equal(dense.reshape(2, 2, -1) != 0, flat.abs() >= thr)
    assert torch.allclose(dense.reshape(2, 2, -1)[dense.reshape(2, 2, -1) != 0], flat[flat.abs() >= thr])
    # 1-D: k clamps to the chunk size, stays even, at least 2
    e1 = tr.encode(torch.randn(64), use_dct=False)
    i1, v1, xs1, tk1 = comp.compress(e1, 100)
    assert v1.shape == (1, 64) and tk1 == 64
    assert comp._clamp_topk(torch.zeros(4, 7), 5) == 4 and comp._clamp_topk(torch.zeros(4, 7), 1) == 2


def test_quantised_compress_is_a_5_tuple_and_dequantises():
    comp = C.TopKCompressor(use_quantization=True, quantization_bins=256, quantization_range=6)
    x = torch.randn(4, 4, 4096)
    idx, q, xshape, totalk, qp = comp.compress(x.reshape(4, 4, 64, 64), 32)
    assert q.dtype == torch.uint8 and len(qp) == 5 and qp[2] == 128 and qp[3].shape == (256,)
    deq = comp._dequantize_values(q, qp)
    vals = torch.gather(x, -1, C.unpack_12bit_indices(idx, q.shape))
    assert (deq - vals).abs().max() < 6 * vals.std() / 256 * 2
    assert comp.maybe_dequantize_values([q, q], [qp, qp], "cpu")[1].dtype == torch.float32
    with pytest.raises(IndexError):
        comp.maybe_dequantize_values([q, q], [qp, None], "cpu")


def test_batch_decompress_mean_over_contributors_and_clip():
    comp = C.TopKCompressor()
    p = torch.zeros(1, 8)
    idx_a, idx_b = torch.tensor([[0, 1]]), torch.tensor([[1, 2]])
    va, vb = torch.tensor([[2.0, 4.0]]), torch.tensor([[8.0, 6.0]])
    out = comp.batch_decompress(p, [C.pack_12bit_indices(idx_a), C.pack_12bit_indices(idx_b)], [va, vb], (1, 8), 8,
                                clip_norm=False)
    assert out.tolist() == [[2.0, 6.0, 6.0, 0, 0, 0, 0, 0]]
    # clip to the (lower) median norm: b is scaled down to a's norm
    out = comp.batch_decompress(p, [C.pack_12bit_indices(idx_a), C.pack_12bit_indices(idx_b)], [va, vb], (1, 8), 8,
                                clip_norm=True)
    s = va.norm() / vb.norm()
    assert torch.allclose(out, torch.tensor([[2.0, (4 + 8 * s) / 2, 6 * s, 0, 0, 0, 0, 0]]), atol=1e-6)
    out = comp.batch_decompress(p, [C.pack_12bit_indices(idx_a)], [va], (1, 8), 8, normalise=True)
    assert torch.allclose(out[0, :2], va[0] / va.norm(), atol=1e-6)
    with pytest.raises(ValueError):
        comp.batch_decompress(p, [idx_a], [va], (1, 8), 8)
