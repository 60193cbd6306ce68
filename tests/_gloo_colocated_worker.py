"""Worker for test_colocated_cpu.py: two miners as the two ranks of one launch (``--colocated``), exchanging gradients
through the peer group (on CPU an all-gather stands in for GPU peer memory) while still uploading for everybody
else; then, on rank 0 alone, the same two miners as ordinary in-process nodes that fetch from the object store."""

import asyncio
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from neurons.miner import Miner  # noqa: E402
from templar_b200.backends.chain import StaticChain  # noqa: E402
from templar_b200.backends.store import LocalFSStore, MemoryStore  # noqa: E402


class CountingStore(LocalFSStore):
    def __init__(self, root):
        super().__init__(root)
        self.fetched = []

    async def get_to_file(self, bucket, key, path):
        self.fetched.append(key)
        return await super().get_to_file(bucket, key, path)


async def windows(miners, n):
    for m in miners:
        m.loop = asyncio.get_running_loop()
        m.comms.commitments = await m.comms.get_commitments()
        m.comms.peers = [2, 3]
        m.gather_timeout = 5
        await m.dataset_manager.initialize_datasets(0)
        m.set_dataloader()
    out = []
    for w in range(1, n + 1):
        for m in miners:
            m.current_window = m.comms.current_window = w
        out.append(await asyncio.gather(*(m.run_window(w) for m in miners)))
    return out


def main():
    tmp = sys.argv[1]
    os.chdir(tmp)
    rank = int(os.environ["RANK"])
    chain = StaticChain(n=4, manual=True, state_file=os.path.join(tmp, "chain.json"))
    store = CountingStore(os.path.join(tmp, "store"))
    argv = ["--local", "--device", "cpu", "--colocated", "--uid", "2", "--peers", "2", "3"]
    m = Miner(config=Miner.miner_config(argv), store=store, subtensor=chain)
    assert m.uid == 2 + rank and m.world_size == 1 and m.group_world == 2 and m.peer_group.uids == [2, 3]
    dist.barrier()                       # both nodes have committed their buckets
    res = asyncio.run(windows([m], 2))
    weights = {k: v.clone() for k, v in m.engine.full_state_dict().items() if v.is_floating_point()}
    out = {"uid": m.uid, "success": [r[0]["gather_success_rate"] for r in res], "steps": res[-1][0]["global_step"],
           "gradient_downloads": [k for k in store.fetched if k.startswith("gradient-")],
           "uploaded": sorted(p.name for p in (store.root).rglob("gradient-*")),
           "ef": float(m.engine.ef.abs().max())}
    dist.barrier()
    if rank == 0:
        # the same two nodes without peer memory: ordinary in-process miners on an in-memory object store
        os.environ["WORLD_SIZE"] = "1"
        mem, chain2 = MemoryStore(), StaticChain(n=4, manual=True)
        plain = [Miner(config=Miner.miner_config(["--local", "--device", "cpu", "--uid", str(u), "--peers", "2", "3"]),
                       store=mem, subtensor=chain2) for u in (2, 3)]
        asyncio.run(windows(plain, 2))
        ref = plain[0].engine.full_state_dict()
        out["vs_object_store"] = max(float((weights[k] - ref[k]).abs().max()) for k in weights)
        out["moved"] = max(float((ref[k] - v).abs().max()) for k, v in
                           Miner(config=Miner.miner_config(["--local", "--device", "cpu", "--uid", "1"]), store=mem,
                                 subtensor=chain2).engine.full_state_dict().items() if k in weights)
    gathered = [None, None]
    dist.all_gather_object(gathered, out)
    both = [None, None]
    dist.all_gather_object(both, {k: v for k, v in weights.items()})
    if rank == 0:
        gathered[0]["peers_agree"] = max(float((both[0][k] - both[1][k]).abs().max()) for k in both[0])
        print("RESULT " + json.dumps(gathered))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
