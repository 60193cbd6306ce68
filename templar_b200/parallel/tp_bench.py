"""Microbenchmark of the fused tensor-parallel kernels against NCCL + cuBLAS.

Run under torchrun, one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
        -m templar_b200.parallel.tp_bench --tokens 8192 --dim 8192 --ffn 28672

Cases (shapes of the 18B tensor-parallel preset by default):
  ag_gemm   y[T, F/w]   = all_gather(x)[T, D] W1^T     vs  all_gather_into_tensor + matmul
  gemm_rs   y[T/w, D]   = reduce_scatter(h[T, F/w] W2^T) vs matmul + reduce_scatter_tensor
  fsdp_ag_gemm y[T, D]  = x[T, D] all_gather(W)[D, D]^T   vs all_gather_into_tensor + matmul (row-sharded weight)
Times are CUDA-event times on the launching stream, max over ranks, median over iterations; a
buffer larger than L2 is rewritten between iterations.  Prints one JSON line per case with the
roofline: the slower of FLOPs / measured GEMM peak and NVLink bytes / 770 GB/s.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops.microbench import peaks
from .symmetric import SymmetricHeap
from .tensor_parallel import GatheredWeight, TensorParallel

NVLINK_GBS = 770.0   # measured peer-copy bandwidth per direction per GPU


def _time(fn, iters, flush, world):
    ts = []
    for i in range(iters + 3):
        flush.add_(1.0)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if i >= 3:
            ts.append(float(t.item()))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--comm-pairs", type=int, default=0, help="CTA pairs for the collective (0: chosen per call)")
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    OF.set_gemm_backend("tcgen05_2sm")
    heap = SymmetricHeap.create(dev, rank, world, timeout_s=20.0)
    T, D, F = a.tokens, a.dim, a.ffn
    fl, tr = F // world, T // world
    tp = TensorParallel(heap, rows=T, width=D, n_comm_pairs=a.comm_pairs or None)
    flush = torch.zeros(64 * 1024 * 1024, device=dev)           # 256 MB > L2
    x_shard = (torch.randn(tr, D, device=dev) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(fl, D, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(D, fl, device=dev) * 0.02).to(torch.bfloat16)
    h = (torch.randn(T, fl, device=dev) * 0.5).to(torch.bfloat16)
    y1 = torch.empty(T, fl, dtype=torch.bfloat16, device=dev)
    y2 = torch.empty(tr, D, dtype=torch.bfloat16, device=dev)
    xg = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    part = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    pk = peaks()

    def fused_ag():
        slot, _, own = tp.gather_buffer(D)
        own.copy_(x_shard)
        tp.ag_gemm(slot, D, w1, out=y1)

    def lib_ag():
        dist.all_gather_into_tensor(xg, x_shard)
        torch.matmul(xg, w1.t(), out=y1)

    def fused_rs():
        tp.gemm_rs(h, w2, out=y2)

    def lib_rs():
        torch.matmul(h, w2.t(), out=part)
        dist.reduce_scatter_tensor(y2, part)

    gw = GatheredWeight(heap, D, D, n_comm_pairs=a.comm_pairs or None)
    w_shard = (torch.randn(D // world, D, device=dev) * 0.02).to(torch.bfloat16)
    gw.own.copy_(w_shard)
    xfull = (torch.randn(T, D, device=dev) * 0.5).to(torch.bfloat16)
    wg = torch.empty(D, D, dtype=torch.bfloat16, device=dev)
    y3 = torch.empty(T, D, dtype=torch.bfloat16, device=dev)

    def fused_fsdp():
        gw.linear(xfull, out=y3)

    def lib_fsdp():
        dist.all_gather_into_tensor(wg, w_shard)
        torch.matmul(xfull, wg.t(), out=y3)

    rows = []
    for name, fused, lib, flops, link_bytes in (
            ("fsdp_ag_gemm", fused_fsdp, lib_fsdp, 2.0 * T * D * D, (world - 1) * (D // world) * D * 2),
            ("ag_gemm", fused_ag, lib_ag, 2.0 * T * fl * D, (world - 1) * tr * D * 2),
            ("gemm_rs", fused_rs, lib_rs, 2.0 * T * D * fl, (world - 1) * tr * D * 2)):
        # correctness of the fused result against the library path on the same inputs
        lib()
        buf = {"ag_gemm": y1, "gemm_rs": y2, "fsdp_ag_gemm": y3}[name]
        ref = buf.float().clone()
        buf.zero_()
        fused()
        torch.cuda.synchronize()
        got = buf.float()
        err = ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()
        med_f, best_f = _time(fused, a.iters, flush, world)
        med_l, best_l = _time(lib, a.iters, flush, world)
        t_flops = flops / (pk["bf16_tflops"] * 1e12) * 1e3
        t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_flops, t_link)
        rows.append({"case": name, "world": world, "T": T, "D": D, "F_local": fl, "fused_ms": med_f, "fused_ms_best": best_f,
                     "nccl_cublas_ms": med_l, "speedup": med_l / med_f, "roofline_ms": roof,
                     "roofline_bound": "flops" if t_flops >= t_link else "nvlink", "frac_of_roofline": roof / med_f,
                     "rel_err_vs_library": err, "comm_pairs": a.comm_pairs, "peaks": pk["source"]})
    tp.check()
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
