"""Worker for test_distributed_cpu.py: the CPU/gloo plumbing run on world_size ranks.

One inner step on random tokens, sharded optimizer step, momentum/error-feedback + chunk-64 DCT +
top-k + 12-bit pack on each rank's shard, exchange of the two ranks' payloads, decompress, inverse
DCT, mean, outer step (SGD or sign), DCP save/load round trip.  Prints one RESULT line on rank 0.
"""

import asyncio
import json
import os
import sys
import time
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from templar_b200.backends.chain import StaticChain, StaticWallet  # noqa: E402
from templar_b200.backends.store import LocalFSStore  # noqa: E402
from templar_b200.models.llama import PRESETS, ModelArgs, build_model  # noqa: E402
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine  # noqa: E402


def main():
    model_name, batch, seq, update, workdir = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    t_all = time.perf_counter()
    args = PRESETS[model_name] if model_name in PRESETS else ModelArgs(dim=128, n_layers=2, n_heads=4, vocab_size=512,
                                                                     intermediate_size=256, max_seq_len=seq)
    model = build_model(args, seed=0)                     # fp32, same seed on every rank
    cfg = EngineConfig(topk=32, use_dct=True, momentum_decay=0.95, inner_lr=1e-3, weight_decay=0.1, outer_lr=0.4,
                       outer_update=update, max_peers=world)
    eng = WindowEngine(model, cfg, rank=rank, world_size=world)
    g = torch.Generator().manual_seed(100 + rank)
    tok = torch.randint(0, args.vocab_size, (batch, seq + 1), generator=g)
    t0 = time.perf_counter()
    eng.snapshot()
    loss0 = float(eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0))
    eng.optimizer_step()
    t_inner = time.perf_counter() - t0
    t0 = time.perf_counter()
    eng.compress()
    # exchange: every rank's payload part is summed into the full node payload (parts are disjoint)
    eng.merge_own_payload()
    # the "two peers": this node's payload and a second, perturbed copy standing for the other peer
    eng.peer_idx[1].copy_(eng.own_idx)
    eng.peer_val[1].copy_(eng.own_val * 0.5)
    t_compress = time.perf_counter() - t0
    t0 = time.perf_counter()
    eng.outer_step(2)
    t_outer = time.perf_counter() - t0
    loss1 = float(eng.micro_step(tok[:, :-1], tok[:, 1:], 1.0))
    eng.zero_grad()
    # all ranks hold the same compute weights afterwards
    flat = eng.store.compute.clone()
    ref = flat.clone()
    dist.broadcast(ref, 0)
    same = bool(torch.equal(flat, ref))
    # DCP round trip through the checkpointer (local file system store)
    store = LocalFSStore(os.path.join(workdir, "store"))
    chain = StaticChain(n=2, manual=True)
    comms = tplr.Comms(wallet=StaticWallet("hotkey-0"), config=SimpleNamespace(netuid=3, device="cpu"),
                       hparams=SimpleNamespace(topk_compression=32, blocks_per_window=4), uid=0, store=store, subtensor=chain)
    ck = tplr.DCPCheckpointer(comms, uid=0, version="test", repo_root=os.path.join(workdir, "repo"))

    async def ckpt():
        t = time.perf_counter()
        await ck.save_local(model=model, window=7, sync_window=7, global_step=3)
        await ck.upload(window=7, initial_sleep_s=0.0, pointer_poll_interval_s=0.2, pointer_poll_timeout_s=20.0,
                        delete_local_on_success=True)
        dist.barrier()
        before = eng.full_master().clone()
        eng.store.master_shard.zero_()
        eng.store.compute.zero_()
        comms.commitments = {}
        res = await ck.download_and_load(model=model, window=None, shared_fs=True, prefer_highest_staked=False)
        after = eng.full_master()
        return res, bool(torch.equal(before, after)), bool(torch.equal(eng.store.compute, flat)), time.perf_counter() - t
    res, master_ok, compute_ok, t_ckpt = asyncio.run(ckpt())
    out = {"rank": rank, "loss0": loss0, "loss1": loss1, "same_weights": same, "ckpt": list(res) if res else None,
           "master_roundtrip": master_ok, "compute_roundtrip": compute_ok, "status": eng.check_status(),
           "t_inner": t_inner, "t_compress": t_compress, "t_outer": t_outer, "t_ckpt": t_ckpt,
           "t_total": time.perf_counter() - t_all, "params": args.num_params()}
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print("RESULT " + json.dumps(gathered))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
