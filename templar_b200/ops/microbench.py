"""Per-kernel microbenchmarks with CUDA-event timing and roofline fractions.

    python -m templar_b200.ops.microbench gemm      [--m 16384 --n 8192 --k 2048] [--layout nt|nn|tn] [--compare]
    python -m templar_b200.ops.microbench compress  [--model 1B] [--topk 32]
    python -m templar_b200.ops.microbench aggregate [--model 1B] [--peers 8] [--topk 32]
    python -m templar_b200.ops.microbench elementwise

Each case warms up, flushes L2 between timed iterations (a 256 MB write), times with CUDA
events on the launching stream and prints one JSON line with the achieved bandwidth / FLOP
rate and its fraction of the measured peaks (``MEASURED_PEAKS.json`` beside the repo root when
present, otherwise the stated fallback).  ``--small`` shrinks a case for profiler captures.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import functional as OF

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return dict(FALLBACK_PEAKS)


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_ms(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_gemm(a):
    M, N, K = a.m, a.n, a.k
    a_mn, b_mn = {"nt": (False, False), "nn": (False, True), "tn": (True, True)}[a.layout]
    A = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
    out_dtype = torch.float32 if a.layout == "tn" else torch.bfloat16
    out = torch.zeros(M, N, device="cuda", dtype=out_dtype)
    OF.set_gemm_backend(a.backend)
    med, best = time_ms(lambda: OF.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=(a.layout == "tn")), a.iters)
    pk = peaks()
    fl = 2.0 * M * N * K
    rec = {"case": "gemm", "backend": a.backend, "layout": a.layout, "M": M, "N": N, "K": K, "ms_median": med, "ms_best": best,
           "tflops": fl / med / 1e9, "frac_of_peak": fl / med / 1e9 / pk["bf16_tflops"], "peaks": pk["source"],
           "status": int(OF.status_word("cuda").item())}
    if a.compare:
        Am = A.t() if a_mn else A
        Bm = B if b_mn else B.t()
        med_c, _ = time_ms(lambda: torch.matmul(Am, Bm), a.iters)
        rec["cublas_ms"] = med_c
        rec["vs_cublas"] = med_c / med
    if a.sustain > 0:
        # back-to-back launches for a.sustain seconds (what a training step sees: the board sits at its power cap);
        # SM clock and board power are READ through NVML while the loop runs
        lib_out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        Am, Bm = (A.t() if a_mn else A), (B if b_mn else B.t())
        rec["sustained_own"] = sustained(lambda: OF.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=(a.layout == "tn")),
                                         fl, a.sustain)
        rec["sustained_library_bf16_out"] = sustained(lambda: torch.matmul(Am, Bm, out=lib_out), fl, a.sustain)
    print(json.dumps(rec))


def sustained(fn, flops: float, seconds: float) -> dict:
    """ms per launch and TFLOP/s over ``seconds`` of back-to-back launches, with the median SM clock and the mean board
    power of the second half of the loop (NVML reads from a sampling thread; absent NVML: timing only)."""
    import threading
    import time

    samples, stop = [], threading.Event()
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())

        def sample():
            while not stop.is_set():
                samples.append((pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM),
                                pynvml.nvmlDeviceGetPowerUsage(handle) / 1e3))
                time.sleep(0.1)
    except Exception:  # noqa: BLE001
        sample = None
    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    th = threading.Thread(target=sample) if sample else None
    if th:
        th.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.time()
    e0.record()
    while time.time() - t0 < seconds:
        for _ in range(50):
            fn()
        n += 50
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    stop.set()
    if th:
        th.join()
    ms = e0.elapsed_time(e1) / n
    out = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "launches": n}
    tail = samples[len(samples) // 2:]
    if tail:
        out["sm_mhz_median"] = sorted(c for c, _ in tail)[len(tail) // 2]
        out["watts_mean"] = round(sum(p for _, p in tail) / len(tail), 1)
    return out


def bench_fused(a):
    """The projections whose element-wise consumers run in the GEMM epilogue, against the same work as separate launches:
    [w1; w3] projection + SwiGLU (forward), and packed q/k/v projection + rotary embedding + attention (forward, and
    forward + backward, where the inverse rotation is folded into the attention backward's outputs)."""
    T, D, Fd = a.m, a.k, a.n // 2
    B, S, H, KV, hd = a.batch, a.seq, a.heads, a.kv_heads, 128
    x = (torch.randn(T, D, device="cuda") * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(2 * Fd, D, device="cuda") / D ** 0.5).to(torch.bfloat16)
    rec = {"case": "fused_projections", "T": T, "D": D, "F": Fd, "B": B, "S": S, "H": H, "KV": KV}
    with torch.no_grad():
        for name, flag in (("fused", True), ("separate", False)):
            OF.FUSED_PROJECTIONS = flag
            rec[f"swiglu_projection_{name}_ms"], _ = time_ms(lambda: OF.linear_swiglu(x, w13), a.iters)
    # the whole feed-forward, forward + backward (the backward of the SwiGLU runs in the down projection's dgrad epilogue)
    w2 = (torch.randn(D, Fd, device="cuda") / Fd ** 0.5).to(torch.bfloat16).requires_grad_()
    w13g = w13.clone().requires_grad_()
    w2.main_grad, w13g.main_grad = torch.zeros(w2.shape, device="cuda"), torch.zeros(w13.shape, device="cuda")
    xg = x.clone().requires_grad_()
    dyf = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    for name, flag in (("fused", True), ("separate", False)):
        OF.FUSED_PROJECTIONS = flag

        def ffn():
            xg.grad = None
            OF.feed_forward(xg, w13g, w2).backward(dyf)
        rec[f"feed_forward_fwdbwd_{name}_ms"], _ = time_ms(ffn, a.iters)
    xq = (torch.randn(B, S, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    wq = (torch.randn((H + 2 * KV) * hd, D, device="cuda") / D ** 0.5).to(torch.bfloat16).requires_grad_()
    wq.main_grad = torch.zeros(wq.shape, device="cuda")
    cos, sin = OF.rope_tables(S, hd, 10000.0, "cuda")
    cos, sin = cos.contiguous(), sin.contiguous()
    dout = torch.randn(B, S, H * hd, device="cuda").to(torch.bfloat16)
    for name, flag in (("fused", True), ("separate", False)):
        OF.FUSED_PROJECTIONS = flag
        with torch.no_grad():
            rec[f"qkv_rope_attention_fwd_{name}_ms"], _ = time_ms(
                lambda: OF.rope_attention_projection(xq, wq, cos, sin, H, KV, hd), a.iters)

        def fb():
            xq.grad = None
            OF.rope_attention_projection(xq, wq, cos, sin, H, KV, hd).backward(dout)
        rec[f"qkv_rope_attention_fwdbwd_{name}_ms"], _ = time_ms(fb, a.iters)
    OF.FUSED_PROJECTIONS = True
    rec["status"] = int(OF.status_word("cuda").item())
    print(json.dumps(rec))


def bench_attention(a):
    """Own flash attention (forward, forward+backward) vs torch SDPA on the packed layout of one layer."""
    B, S, H, KV, hd = a.batch, a.seq, a.heads, a.kv_heads, 128
    qkv = torch.randn(B, S, (H + 2 * KV) * hd, device="cuda").to(torch.bfloat16).requires_grad_()
    dout = torch.randn(B, S, H * hd, device="cuda").to(torch.bfloat16)
    fl_fwd = 4.0 * B * H * S * S * hd / 2
    rec = {"case": "attention", "B": B, "S": S, "H": H, "KV": KV, "status": 0}
    for be in ("tcgen05", "sdpa"):
        OF.set_attention_backend(be)
        with torch.no_grad():
            med_f, _ = time_ms(lambda: OF.attention_packed(qkv, H, KV, hd), a.iters)

        def fb():
            qkv.grad = None
            OF.attention_packed(qkv, H, KV, hd).backward(dout)
        med_fb, _ = time_ms(fb, a.iters)
        rec[f"{be}_fwd_ms"], rec[f"{be}_fwd_tflops"] = med_f, fl_fwd / med_f / 1e9
        rec[f"{be}_fwdbwd_ms"], rec[f"{be}_fwdbwd_tflops"] = med_fb, 3.5 * fl_fwd / med_fb / 1e9
    OF.set_attention_backend("tcgen05")
    rec["status"] = int(OF.status_word("cuda").item())
    print(json.dumps(rec))


def _engine(model_name, topk, peers):
    from ..models.llama import PRESETS, build_model
    from ..parallel.window_engine import EngineConfig, WindowEngine

    model = build_model(PRESETS[model_name], device="cuda", dtype=torch.bfloat16, seed=0)
    return WindowEngine(model, EngineConfig(topk=topk, max_peers=peers), device="cuda")


def bench_compress(a):
    eng = _engine(a.model, a.topk, 1)
    eng.snapshot()
    eng.store.master_shard.add_(torch.randn_like(eng.store.master_shard) * 1e-3)
    med, best = time_ms(lambda: eng.compress(), a.iters)
    n = eng.layout.total
    byts = n * 4 * 4  # theta0 + theta + e read, e written
    pk = peaks()
    print(json.dumps({"case": "compress", "model": a.model, "topk": a.topk, "elements": n, "ms_median": med,
                      "ms_best": best, "gbs": byts / med / 1e6, "frac_of_hbm": byts / med / 1e6 / pk["hbm_gbs"],
                      "peaks": pk["source"], "status": eng.check_status()}))


def bench_quantize(a):
    """The two steps that the 8-bit payload mode adds after compress: encode (codes + tables) and the
    error-feedback correction with the dequantised values written back."""
    eng = _engine(a.model, a.topk, 1)
    eng.snapshot()
    eng.store.master_shard.add_(torch.randn_like(eng.store.master_shard) * 1e-3)
    eng.compress()
    exact = eng.own_val.clone()
    eng.cfg.quantize = True

    def both():
        eng.own_val.copy_(exact)
        eng._quantize_own(on_rank0=False)

    copy_med, _ = time_ms(lambda: eng.own_val.copy_(exact), a.iters)
    med, best = time_ms(both, a.iters)
    enc_med, _ = time_ms(lambda: eng.encode_values(exact), a.iters)
    n = eng.layout.total
    byts = n * 4 * 2                      # error feedback read and written
    pk = peaks()
    print(json.dumps({"case": "quantize", "model": a.model, "topk": a.topk, "values": int(eng.layout.val_elems),
                      "ms_median": med - copy_med, "ms_best": best - copy_med, "encode_ms": enc_med,
                      "gbs": byts / (med - copy_med) / 1e6, "frac_of_hbm": byts / (med - copy_med) / 1e6 / pk["hbm_gbs"],
                      "peaks": pk["source"], "status": eng.check_status()}))


def bench_aggregate(a):
    from ..utils.synthetic import synthetic_payload

    eng = _engine(a.model, a.topk, a.peers)
    eng.snapshot()
    for j in range(a.peers):
        eng.load_peer_payload(j, synthetic_payload(eng.layout, 7 + j, device="cuda"))
    med, best = time_ms(lambda: eng.outer_step(a.peers, include_own=False), a.iters)
    n = eng.layout.total
    byts = n * (4 + 4 + 2) + a.peers * (eng.layout.idx_bytes + eng.layout.val_elems * 4) * 2
    pk = peaks()
    print(json.dumps({"case": "aggregate", "model": a.model, "peers": a.peers, "topk": a.topk, "ms_median": med,
                      "ms_best": best, "gbs": byts / med / 1e6, "frac_of_hbm": byts / med / 1e6 / pk["hbm_gbs"],
                      "peaks": pk["source"], "status": eng.check_status()}))


def bench_overlap(a):
    """Pairwise index overlap of the staged peers' packed payloads (the validator's copy check), one kernel."""
    from ..utils.synthetic import synthetic_payload

    eng = _engine(a.model, a.topk, a.peers)
    for j in range(a.peers):
        eng.load_peer_payload(j, synthetic_payload(eng.layout, 7 + j, device="cuda"))
    med, best = time_ms(lambda: eng.index_overlap(a.peers), a.iters)
    byts = a.peers * eng.layout.idx_bytes
    pk = peaks()
    print(json.dumps({"case": "index_overlap", "model": a.model, "peers": a.peers, "topk": a.topk, "ms_median": med,
                      "ms_best": best, "index_bytes": byts, "gbs": byts / med / 1e6, "frac_of_hbm": byts / med / 1e6 / pk["hbm_gbs"],
                      "peaks": pk["source"], "status": eng.check_status()}))


def bench_elementwise(a):
    pk = peaks()
    T, D, F, V = (2048, 2048, 8192, 32000) if a.small else (16384, 2048, 8192, 32000)
    x = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    h = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, V, device="cuda").to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device="cuda")
    res = torch.randn(T, D, device="cuda").to(torch.bfloat16).requires_grad_()
    delta = torch.randn(T, D, device="cuda").to(torch.bfloat16).requires_grad_()
    wn = torch.ones(D, device="cuda", dtype=torch.bfloat16).requires_grad_()
    wn.main_grad = torch.zeros(D, device="cuda")
    hg = h.clone().requires_grad_()
    dyh = torch.randn(T, F, device="cuda").to(torch.bfloat16)
    H, hd = D // 128, 128
    qkv = torch.randn(1, T, 3 * D, device="cuda").to(torch.bfloat16)
    cos, sin = OF.rope_tables(T, hd, 10000.0, "cuda")

    def add_norm_fwd_bwd():
        hh, y = OF.add_rmsnorm(res, delta, wn)
        torch.autograd.backward([hh, y], [x, x])

    def swiglu_fwd_bwd():
        hg.grad = None
        OF.swiglu(hg).backward(dyh)

    cases = {
        "rmsnorm_fwd": (lambda: OF.rmsnorm(x, w), T * D * 2 * 2),
        "add_rmsnorm_fwd_bwd": (add_norm_fwd_bwd, T * D * 2 * (4 + 4)),
        "rope_inplace": (lambda: OF.rope(qkv, cos, sin, 2 * H, hd), T * 2 * D * 2 * 2),
        "swiglu_fwd": (lambda: OF.swiglu(h), T * F * 2 * 3),
        "swiglu_fwd_bwd": (swiglu_fwd_bwd, T * F * 2 * (3 + 5)),
        "cross_entropy_fwd_bwd": (lambda: OF.cross_entropy(logits.requires_grad_(), labels), T * V * 2 * 3),
    }
    # fused AdamW on a flat shard: fp32 master / moments / gradient in, master / moments / bf16 copy out
    from . import native
    n = (8 if a.small else 64) * 1024 * 1024
    master, m1, m2 = (torch.zeros(n, device="cuda") for _ in range(3))
    grad = torch.randn(n, device="cuda") * 1e-3
    shadow = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    gsq = (grad * grad).sum().reshape(1)

    def adamw():
        native.check(native.lib().tplr_adamw(master.data_ptr(), m1.data_ptr(), m2.data_ptr(), grad.data_ptr(),
                                             native.ptr_array([shadow.data_ptr()]), 1, n, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1,
                                             1.0, 1.0, gsq.data_ptr(), 1, native.stream_ptr()), "adamw")

    cases["adamw"] = (adamw, n * (4 * 4 + 4 * 3 + 4 + 2))      # the gradient is zeroed in the same pass
    # the backward kernel of add+RMSNorm alone (three distinct bf16 inputs, one output, fp32 weight gradient)
    b_dy, b_x, b_dres = (torch.randn(T, D, device="cuda").to(torch.bfloat16) for _ in range(3))
    b_dx = torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
    b_dw = torch.zeros(D, device="cuda")
    b_rstd = torch.rsqrt(b_x.float().pow(2).mean(-1) + 1e-5).contiguous()

    def norm_bwd():
        native.check(native.lib().tplr_add_rmsnorm_bwd_v2(b_dy.data_ptr(), b_x.data_ptr(), w.data_ptr(), b_rstd.data_ptr(),
                                                          b_dres.data_ptr(), b_dx.data_ptr(), b_dw.data_ptr(), T, D,
                                                          OF.status_word("cuda").data_ptr(), native.stream_ptr()), "norm_bwd")

    cases["add_rmsnorm_bwd_kernel"] = (norm_bwd, T * D * 2 * 4)
    # --compare: the same operations as the reference's stack runs them (PyTorch eager ops on the same tensors:
    # torchtitan's RMSNorm / SwiGLU / cross entropy modules and torch.optim.AdamW(fused=True) + clip_grad_norm_)
    library = {}
    if a.compare:
        import torch.nn.functional as TF

        xr, dr = res.detach().clone().requires_grad_(), delta.detach().clone().requires_grad_()
        wr = wn.detach().clone().requires_grad_()
        hr = h.clone().requires_grad_()
        lr_ = logits.clone().requires_grad_()
        pm = torch.nn.Parameter(master.clone())
        opt = torch.optim.AdamW([pm], lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)

        def lib_norm():
            xr.grad = dr.grad = wr.grad = None
            hh = xr + dr
            y = TF.rms_norm(hh, (D,), wr, 1e-5)
            torch.autograd.backward([hh, y], [x, x])

        def lib_swiglu():
            hr.grad = None
            (TF.silu(hr[:, :F]) * hr[:, F:]).backward(dyh)

        def lib_ce():
            lr_.grad = None
            TF.cross_entropy(lr_.float(), labels).backward()

        def lib_adamw():
            pm.grad = grad
            torch.nn.utils.clip_grad_norm_([pm], 1.0)
            opt.step()

        library = {"rmsnorm_fwd": lambda: TF.rms_norm(x, (D,), w, 1e-5), "add_rmsnorm_fwd_bwd": lib_norm,
                   "swiglu_fwd": lambda: TF.silu(h[:, :F]) * h[:, F:], "swiglu_fwd_bwd": lib_swiglu,
                   "cross_entropy_fwd_bwd": lib_ce, "adamw": lib_adamw}
    for name, (fn, byts) in cases.items():
        med, best = time_ms(fn, a.iters)
        rec = {"case": name, "ms_median": med, "gbs": byts / med / 1e6, "frac_of_hbm": byts / med / 1e6 / pk["hbm_gbs"],
               "peaks": pk["source"]}
        if name in library:
            rec["torch_ms"], _ = time_ms(library[name], a.iters)
            rec["vs_torch"] = rec["torch_ms"] / med
        print(json.dumps(rec))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "compress", "quantize", "aggregate", "overlap", "elementwise", "attention", "fused"])
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--sustain", type=float, default=0.0,
                    help="gemm: also run back-to-back launches for this many seconds (own kernel, then the library) and "
                         "report the rate with the SM clock and board power read through NVML")
    ap.add_argument("--backend", default="tcgen05_2sm", choices=["tcgen05", "tcgen05_2sm"])
    ap.add_argument("--model", default="1B")
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--peers", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--variant", type=int, default=None,
                    help="compress / aggregate: switches of the tensor-core kernels (tplr_compress_set_variant)")
    a = ap.parse_args()
    if a.variant is not None:
        from . import native
        native.lib().tplr_compress_set_variant(a.variant)
    {"gemm": bench_gemm, "compress": bench_compress, "quantize": bench_quantize, "aggregate": bench_aggregate,
     "elementwise": bench_elementwise, "attention": bench_attention, "fused": bench_fused, "overlap": bench_overlap}[a.case](a)


if __name__ == "__main__":
    main()
