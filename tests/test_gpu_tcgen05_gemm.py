"""tcgen05/TMEM GEMM against torch.matmul in fp32 for every operand layout and epilogue."""

import pytest
import torch

from templar_b200.ops import functional as OF

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=["tcgen05", "tcgen05_2sm"], autouse=True)
def backend(request):
    """Every test runs on the one-CTA-per-tile kernel and on the CTA-pair (cta_group::2) kernel."""
    prev = OF.gemm_backend()
    OF.set_gemm_backend(request.param)
    yield request.param
    OF.set_gemm_backend(prev)


def _check(M, N, K, a_mn, b_mn, epi):
    torch.manual_seed(M + N + K)
    A = torch.randn((K, M) if a_mn else (M, K), device=DEV).to(torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), device=DEV).to(torch.bfloat16)
    Af = (A.t() if a_mn else A).float()
    Bf = (B if b_mn else B.t()).float()
    ref = Af @ Bf
    OF.status_word(DEV).zero_()
    if epi == "bf16":
        out = OF.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
        tol = 2e-2 * (K ** 0.5)
    elif epi == "f32":
        out = OF.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
        tol = 1e-3 * (K ** 0.5)
    else:
        base = torch.randn(M, N, device=DEV)
        out = OF.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=base.clone(), accumulate=True)
        ref = ref + base
        tol = 1e-3 * (K ** 0.5)
    torch.cuda.synchronize()
    assert int(OF.status_word(DEV).item()) == 0, "bounded wait expired inside the GEMM kernel"
    err = (out.float() - ref).abs().max().item()
    assert err < tol, (M, N, K, a_mn, b_mn, epi, err)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("epi", ["bf16", "f32", "acc"])
def test_gemm_layouts(a_mn, b_mn, epi):
    _check(256, 512, 320, a_mn, b_mn, epi)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 256, 2048), (2048, 2048, 2048), (1000, 776, 136),
                                   (4096, 32000, 512), (130, 264, 72), (8, 8, 8), (257, 513, 4104)])
def test_gemm_shapes(M, N, K):
    _check(M, N, K, False, False, "bf16")


def test_linear_backward_matches_autograd():
    x = torch.randn(3, 100, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    y = OF.linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xf @ wf.t()).backward(dy.float())
    assert torch.allclose(x.grad.float(), xf.grad, atol=0.1, rtol=3e-2)
    assert torch.allclose(w.grad.float(), wf.grad, atol=0.5, rtol=3e-2)


def test_gemm_from_a_fresh_thread():
    """The tensor-map encode is a driver call; a thread that has not touched CUDA yet (like an
    autograd worker) must still be able to launch the GEMM."""
    import threading

    A = torch.randn(256, 128, device=DEV).to(torch.bfloat16)
    B = torch.randn(512, 128, device=DEV).to(torch.bfloat16)
    box = {}

    def work():
        try:
            box["out"] = OF.gemm(A, B)
        except Exception as e:  # noqa: BLE001
            box["err"] = e

    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert "err" not in box, box.get("err")
    assert (box["out"].float() - A.float() @ B.float().t()).abs().max().item() < 0.5
