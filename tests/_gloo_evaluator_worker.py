"""Worker for test_distributed_cpu.py: the evaluator on world_size gloo ranks.

The ranks share a local object store and a static chain through the environment.  A checkpoint of window 5 is saved
and uploaded by all ranks under the highest-staked validator's uid; then the evaluator runs once (newest checkpoint,
task harness as a child of rank 0 only, the other ranks waiting on the sentinel) and once more as a backfill over
windows 4..6, of which only 5 exists.  Prints one RESULT line on rank 0.
"""

import asyncio
import json
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import templar_b200 as tplr  # noqa: E402
from neurons.evaluator import Evaluator  # noqa: E402
from templar_b200.backends.chain import StaticWallet  # noqa: E402


def main():
    workdir = sys.argv[1]
    os.chdir(workdir)
    e = Evaluator(config=Evaluator.evaluator_config(
        ["--local", "--device", "cpu", "--uid", "1", "--tasks", "arc_easy", "--custom-eval-batches", "1", "--no-follow",
         "--cache-dir", os.path.join(workdir, "cache")]))
    rank, world = dist.get_rank(), dist.get_world_size()
    top = tplr.Comms(wallet=StaticWallet("hotkey-0"), config=e.config, hparams=e.hparams, uid=0, subtensor=e.subtensor)
    ck = tplr.DCPCheckpointer(top, uid=0, version=e.version, repo_root=os.path.join(workdir, "repo"))

    async def go():
        top.try_commit(top.wallet, top.bucket)             # the validator's bucket is on the chain
        dist.barrier()
        top.commitments = await top.get_commitments()
        if rank == 0:
            await top.post_start_window(3)
        await ck.save_local(model=e.model, window=5, sync_window=5, global_step=2)
        await ck.upload(window=5, initial_sleep_s=0.0, pointer_poll_interval_s=0.2, pointer_poll_timeout_s=20.0)
        dist.barrier()
        await e.run()
        first = {"evaluated": sorted(e.evaluated_windows), "counter": e.eval_counter, "start_window": e.start_window,
                 "baseline": e.baseline_evaluated}
        e.from_window, e.to_window, e.force_reval = 6, 4, True       # reversed on purpose
        done = await e.backfill_range()
        return first, done
    first, done = asyncio.run(go())
    leftovers = [f for f in os.listdir("/tmp") if f.startswith(f"tplr_lm_eval_done_{e.uid}_")]
    out = {"rank": rank, **first, "backfilled": done, "counter_after": e.eval_counter, "cache": e.cache.windows(),
           "export_complete": e.cache.exists(5), "sentinels_left": leftovers,
           "child_runs": len(open(os.path.join(workdir, "harness_calls.txt")).read().split()) if rank == 0 else None}
    e.cleanup()                                            # drains the metrics writer into its sink
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print("RESULT " + json.dumps(gathered))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
