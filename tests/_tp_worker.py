"""Worker launched by test_gpu_multi.py under torchrun: fused tensor-parallel kernels vs a one-GPU fp32 reference."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.ops import functional as OF  # noqa: E402
from templar_b200.parallel.symmetric import SymmetricHeap  # noqa: E402
from templar_b200.parallel.tensor_parallel import (GatheredWeight, TensorParallel, column_parallel_linear,  # noqa: E402
                                                   row_parallel_linear)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    OF.set_gemm_backend("tcgen05_2sm")
    heap = SymmetricHeap.create(dev, rank, world, timeout_s=20.0)
    out = {}
    T, D, F = 256 * world * 2, 512, 1024          # tokens, model width, hidden width (full)
    tp = TensorParallel(heap, rows=T, width=D, n_comm_pairs=4)
    tr = T // world
    g = torch.Generator().manual_seed(11)
    X = (torch.randn(T, D, generator=g) * 0.5).to(dev)
    W1 = (torch.randn(F, D, generator=g) * 0.05).to(dev)     # column parallel: rows split
    W2 = (torch.randn(D, F, generator=g) * 0.05).to(dev)     # row parallel: columns split
    dY = (torch.randn(T, D, generator=g) * 0.5).to(dev)
    fl = F // world
    x_shard = X[rank * tr:(rank + 1) * tr].to(torch.bfloat16).requires_grad_()
    w1 = W1[rank * fl:(rank + 1) * fl].to(torch.bfloat16).contiguous().requires_grad_()
    w2 = W2[:, rank * fl:(rank + 1) * fl].to(torch.bfloat16).contiguous().requires_grad_()
    mg1 = torch.zeros(fl, D, device=dev)
    mg2 = torch.zeros(D, fl, device=dev)

    # fp32 reference of the same bf16-rounded operands on this GPU
    Xr = X.to(torch.bfloat16).float().requires_grad_()
    W1r = W1.to(torch.bfloat16).float().requires_grad_()
    W2r = W2.to(torch.bfloat16).float().requires_grad_()
    Hr = Xr @ W1r.t()
    Yr = Hr.to(torch.bfloat16).float() @ W2r.t()
    Yr.backward(dY.to(torch.bfloat16).float())

    for rep in range(3):                                       # repeated calls reuse buffers and flags
        x_shard.grad = None
        mg1.zero_(); mg2.zero_()
        h = column_parallel_linear(x_shard, w1, tp, mg1)       # [T, F/world]
        y = row_parallel_linear(h, w2, tp, mg2)                # [T/world, D]
        y.backward(dY[rank * tr:(rank + 1) * tr].to(torch.bfloat16))
        torch.cuda.synchronize()
        tp.check()

    def rel(a, b):
        return ((a.float() - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()

    out["h"] = rel(h, Hr[:, rank * fl:(rank + 1) * fl].detach())
    out["y"] = rel(y, Yr[rank * tr:(rank + 1) * tr].detach())
    out["dx"] = rel(x_shard.grad, Xr.grad[rank * tr:(rank + 1) * tr])
    out["dw1"] = rel(mg1, W1r.grad[rank * fl:(rank + 1) * fl])
    out["dw2"] = rel(mg2, W2r.grad[:, rank * fl:(rank + 1) * fl])
    # FSDP-style row-sharded weight gathered inside the GEMM that consumes it
    Wf = (torch.randn(256 * world, D, generator=g) * 0.05).to(dev).to(torch.bfloat16)
    gw = GatheredWeight(heap, 256 * world, D)
    gw.own.copy_(Wf[rank * 256:(rank + 1) * 256])
    xa = X.to(torch.bfloat16)
    for rep in range(2):
        yg = gw.linear(xa)
    torch.cuda.synchronize()
    out["fsdp_y"] = rel(yg, xa.float() @ Wf.float().t())
    out["fsdp_w"] = float((gw.full.float() - Wf.float()).abs().max())
    out["status"] = int(OF.status_word(dev).item())
    heap.barrier()
    torch.cuda.synchronize()
    heap.check_guards()           # no store of any rank ran past the end of a symmetric block of this rank
    out["guards_ok"] = True
    res = [None] * world
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
