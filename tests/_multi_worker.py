"""Worker launched by test_gpu_multi.py under torchrun (one process per GPU)."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.ops import functional as OF  # noqa: E402
from templar_b200.parallel.symmetric import SymmetricHeap  # noqa: E402
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine  # noqa: E402
from templar_b200.utils.synthetic import synthetic_payload  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    out = {}
    heap = SymmetricHeap.create(dev, rank, world, timeout_s=20.0)

    # 1. peer stores / loads and the flag barrier
    buf = heap.alloc(1024, torch.float32)
    buf.fill_(float(rank + 1))
    heap.barrier()
    from templar_b200.ops import native
    dst = [heap.peer_ptr(buf, (rank + 1) % world) + 512 * 4]
    native.check(native.lib().tplr_push_copy(buf.data_ptr(), native.ptr_array(dst), 1, 512 * 4, native.stream_ptr()), "push")
    heap.barrier()
    torch.cuda.synchronize()
    left = (rank - 1) % world
    out["push_ok"] = bool((buf[512:] == float(left + 1)).all().item() and (buf[:512] == float(rank + 1)).all().item())
    heap.check()

    # 2. a bounded wait that nothing satisfies: rank 0 waits on a barrier the others skip
    heap.timeout_ns = int(0.3e9)
    if rank == 0:
        heap.barrier()
        torch.cuda.synchronize()
        try:
            heap.check()
            out["timeout_detected"] = False
        except TimeoutError:
            out["timeout_detected"] = True
    else:
        heap._epoch += 1          # stay in step with rank 0's epoch counter without arriving
        out["timeout_detected"] = True
    heap.timeout_ns = int(20e9)
    dist.barrier()
    heap.barrier()                # the late arrival of the skipped epoch is harmless: epochs only grow
    torch.cuda.synchronize()
    heap.check()

    # 3. sharded window == single-rank window on the same global batch
    OF.set_gemm_backend(os.environ.get("TPLR_TEST_GEMM", "tcgen05_2sm"))
    args = ModelArgs(dim=256, n_layers=2, n_heads=4, vocab_size=1024, intermediate_size=512, max_seq_len=128)
    cfg = EngineConfig(topk=8, max_peers=4, inner_lr=1e-3, outer_lr=0.5)
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, 1024, (world, 2, 4, 129), generator=g)   # [rank, micro, batch, seq+1]

    def run(engine, my_ranks, hp):
        engine.snapshot()
        for m in range(2):
            for r in my_ranks:
                t = toks[r, m].to(dev)
                engine.micro_step(t[:, :-1], t[:, 1:], 0.5 / (1 if engine.dp_size > 1 else world))
        engine.optimizer_step()
        own = None
        if engine.heap is not None:
            own = (engine.heap.peer_ptr(engine.own_idx, 0), engine.heap.peer_ptr(engine.own_val, 0))
        engine.compress(own_slot_ptrs=own)
        for j in range(1, 4):
            if j % engine.world_size == engine.rank:
                engine.load_peer_payload(j // engine.world_size, synthetic_payload(engine.layout, 50 + j, device=dev))
        engine._barrier()
        engine.outer_step(4)
        torch.cuda.synchronize()

    model = build_model(args, device=dev, dtype=torch.bfloat16, seed=5)
    eng = WindowEngine(model, cfg, device=dev, rank=rank, world_size=world, heap=heap)
    run(eng, [rank], heap)
    heap.check()
    out["status"] = eng.check_status()
    ref_model = build_model(args, device=dev, dtype=torch.bfloat16, seed=5)
    ref = WindowEngine(ref_model, cfg, device=dev)
    run(ref, list(range(world)), None)
    lo, hi = eng.store.lo, eng.store.hi
    diff = (eng.store.master_shard - ref.store.master_shard[lo:hi]).abs().max().item()
    scale = ref.store.master_shard.abs().max().item()
    cdiff = (eng.store.compute.float() - ref.store.compute.float()).abs().max().item()
    out["master_max_diff"], out["compute_max_diff"], out["scale"] = diff, cdiff, scale
    moved = (ref.store.master_shard - ref.theta0).abs().max().item()
    out["moved"] = moved
    # index overlap of the staged peers: the ranks of the sharded engine count over their own chunks and sum
    ov, ov_ref = eng.index_overlap(4), ref.index_overlap(4)
    out["overlap_max_diff"] = (ov - ov_ref).abs().max().item()
    out["overlap_some"] = float(ov_ref.max().item())

    # 4. the same with 8-bit payload values: rank 0 encodes the assembled payload, every rank corrects its chunks
    import dataclasses
    qcfg = dataclasses.replace(cfg, quantize=True, quant_bins=256)
    qeng = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), qcfg, device=dev, rank=rank,
                        world_size=world, heap=heap)
    run(qeng, [rank], heap)
    heap.check()
    qref = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), qcfg, device=dev)
    run(qref, list(range(world)), None)
    lo, hi = qeng.store.lo, qeng.store.hi
    out["q_status"] = qeng.check_status()
    out["q_master_max_diff"] = (qeng.store.master_shard - qref.store.master_shard[lo:hi]).abs().max().item()
    out["q_ef_max_diff"] = (qeng.ef - qref.ef[lo:hi]).abs().max().item()
    out["q_ef_scale"] = qref.ef.abs().max().item()
    out["q_ef_vs_exact"] = (qref.ef - ref.ef).abs().max().item()       # the quantisation error is in the buffer
    if rank == 0:
        out["q_val_max_diff"] = (qeng.own_val - qref.own_val).abs().max().item()
        out["q_val_scale"] = qref.own_val.abs().max().item()
        out["q_codes_equal"] = float((qeng._q_codes == qref._q_codes).float().mean().item())

    # 5. Muon as the inner optimizer: direction shards exchanged over NVLink, Newton-Schulz on the own GEMM
    mcfg = dataclasses.replace(cfg, inner_optimizer="muon", inner_lr=0.02)
    meng = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), mcfg, device=dev, rank=rank,
                        world_size=world, heap=heap)
    start = meng.store.master_shard.clone()
    run(meng, [rank], heap)
    heap.check()
    mref = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), mcfg, device=dev)
    run(mref, list(range(world)), None)
    lo, hi = meng.store.lo, meng.store.hi
    md = (meng.store.master_shard - mref.store.master_shard[lo:hi]).abs()
    out["m_status"] = meng.check_status()
    out["m_mean_diff"], out["m_max_diff"] = md.mean().item(), md.max().item()
    out["m_moved_mean"] = (mref.store.master_shard[lo:hi] - start).abs().mean().item()
    out["m_vs_adamw"] = (mref.store.master_shard - ref.store.master_shard).abs().mean().item()
    # 6. sharded parameters (the FSDP role): weights gathered per block over NVLink on a side stream, weight
    #    gradients reduce-added into the owners' shards by the GEMM epilogue; two windows, so that the second one
    #    starts from gathered weights that the first one's outer step has replaced
    def shard_view(engine, full):
        return torch.cat([full[p.g_lo:p.g_hi] for p in engine.layout.pieces(engine.rank)])

    def local_view(engine, vec):
        return torch.cat([vec[p.local: p.local + (p.g_hi - p.g_lo)] for p in engine.layout.pieces(engine.rank)])

    for tag, extra in (("f", {"gather_buffers": 2}), ("fq", {"quantize": True, "quant_bins": 256}), ("fk", {"gather_buffers": 8}),
                       ("fd", {"gather_buffers": 2}), ("fm", {"inner_optimizer": "muon", "inner_lr": 0.02})):
        os.environ["TPLR_GATHER_ENGINE"] = "dma" if tag == "fd" else "sm"     # fd: gathers by the copy engines
        fcfg = dataclasses.replace(cfg, shard_params=True, **extra)
        fmodel = build_model(args, device=dev, dtype=torch.bfloat16, seed=5)
        fmodel.activation_checkpointing = tag == "fk"
        feng = WindowEngine(fmodel, fcfg, device=dev, rank=rank, world_size=world, heap=heap)
        fref = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5),
                            dataclasses.replace(cfg, **{k: v for k, v in extra.items() if k != "gather_buffers"}), device=dev)
        for _ in range(2):
            run(feng, [rank], heap)
            run(fref, list(range(world)), None)
        heap.check()
        out[tag + "_status"] = feng.check_status()
        out[tag + "_master_max_diff"] = (local_view(feng, feng.store.master_shard)
                                         - shard_view(feng, fref.store.master_shard)).abs().max().item()
        out[tag + "_ef_max_diff"] = (local_view(feng, feng.ef) - shard_view(feng, fref.ef)).abs().max().item()
        out[tag + "_ef_scale"] = fref.ef.abs().max().item()
        out[tag + "_scale"] = fref.store.master_shard.abs().max().item()
        out[tag + "_moved"] = (fref.store.master_shard - fref.theta0).abs().max().item()
        out[tag + "_master_mean_diff"] = (local_view(feng, feng.store.master_shard)
                                          - shard_view(feng, fref.store.master_shard)).abs().mean().item()
        out[tag + "_moved_mean"] = (fref.store.master_shard - fref.theta0).abs().mean().item()
        out[tag + "_gathers"] = feng.store.gather.gathers
        out[tag + "_no_full_buffers"] = feng.store.compute is None and feng.store.grad is None
        t = toks[0, 0].to(dev)
        with torch.no_grad():
            out[tag + "_loss_diff"] = abs(float(fmodel.loss(t[:, :-1], t[:, 1:])) - float(fref.model.loss(t[:, :-1], t[:, 1:])))

    # 7. co-located nodes: every rank is a whole node of its own (engine world_size 1, buffers on the shared heap);
    #    after compress + post + barrier each node aggregates all nodes' payloads by reading them from the owners'
    #    memory over NVLink.  Checked against one engine that has the same payloads staged in its slots.
    from templar_b200.parallel.peer_group import LocalPeerGroup

    ccfg = dataclasses.replace(cfg, max_peers=world)
    node = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), ccfg, device=dev, heap=heap)
    pg = LocalPeerGroup(100 + rank, rank=rank, world_size=world, heap=heap, device=dev)
    pg.attach(node)
    node.snapshot()
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    node.store.master_shard.add_(torch.randn(node.store.master_shard.shape, device=dev, generator=gen) * 1e-3)
    node.compress()
    pg.publish(42)
    pg.exchange()
    out["c_fresh"] = pg.fresh(42) == {100 + r: r for r in range(world)} and pg.fresh(41) == {}
    own_idx, own_val = node.own_idx.clone(), node.own_val.clone()
    node.outer_step(peers=[("rank", r) for r in range(world)], include_own=False)
    torch.cuda.synchronize()
    out["c_status"] = node.check_status()
    # the same aggregation from slots: payloads moved with NCCL
    idxs = [torch.empty_like(own_idx) for _ in range(world)]
    vals = [torch.empty_like(own_val) for _ in range(world)]
    dist.all_gather(idxs, own_idx)
    dist.all_gather(vals, own_val)
    cref = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), ccfg, device=dev)
    cref.snapshot()
    for r in range(world):
        cref.load_peer_payload(r, (idxs[r], vals[r]))
    cref.outer_step(world, include_own=False)
    torch.cuda.synchronize()
    out["c_master_max_diff"] = (node.store.master_shard - cref.store.master_shard).abs().max().item()
    out["c_moved"] = (cref.store.master_shard - cref.theta0).abs().max().item()
    pg.barrier()                 # nobody's buffers are reused while a peer may still read them

    # 8. replicas of the whole state (plain data parallelism): every rank is a copy of its own, the gradient is summed
    #    over the copies with NCCL in buckets; same window as the sharded engine of section 1
    reng = WindowEngine(build_model(args, device=dev, dtype=torch.bfloat16, seed=5), cfg, device=dev,
                        replicate_group=dist.group.WORLD, replicate_size=world)
    reng.REPLICATE_BUCKET = 1 << 20                       # several buckets even on this small model
    run(reng, [rank], None)
    out["r_status"] = reng.check_status()
    out["r_master_max_diff"] = (reng.store.master_shard - ref.store.master_shard).abs().max().item()
    out["r_moved"] = (ref.store.master_shard - ref.theta0).abs().max().item()

    heap.barrier()
    torch.cuda.synchronize()
    heap.check_guards()           # no store of any rank ran past the end of a symmetric block of this rank
    out["guards_ok"] = True
    res = [None] * world
    dist.all_gather_object(res, out)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
