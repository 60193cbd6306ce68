"""Worker for test_trainer_agreement.py: one rank's window clock advances in the middle of an accumulation
(and, in a second run, one rank is asked to stop there); both ranks must leave ``Trainer.inner_steps`` at the
same accumulation boundary, having made the same number of optimizer steps (gloo, 2 ranks)."""

import asyncio
import json
import os
import sys
import threading
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from neurons.trainer import Trainer  # noqa: E402
from templar_b200.distributed import dist_helper  # noqa: E402
from templar_b200.models.llama import ModelArgs, build_model  # noqa: E402
from templar_b200.parallel.window_engine import EngineConfig, WindowEngine  # noqa: E402


class FlippingLoader:
    """Yields ``n`` micro-batches; just before micro-batch ``at`` it runs ``hook`` (on one rank only)."""

    def __init__(self, n, at, hook, vocab):
        self.n, self.at, self.hook, self.vocab = n, at, hook, vocab

    def __iter__(self):
        g = torch.Generator().manual_seed(5)
        for i in range(self.n):
            if i == self.at and self.hook is not None:
                self.hook()
            yield torch.randint(0, self.vocab, (2, 16), generator=g)


def run_case(rank, world, mode):
    args = ModelArgs(dim=64, n_layers=1, n_heads=2, vocab_size=128, intermediate_size=128, max_seq_len=16)
    t = Trainer()
    t.hparams = SimpleNamespace(inner_steps=4, outer_learning_rate=0.4, optimizer={"type": "adamw", "adamw": {"learning_rate": 1e-3}},
                                anneal_mode={}, tokenizer=SimpleNamespace(pad_token_id=0))
    t.tokenizer = t.hparams.tokenizer
    t.device, t.rank, t.world_size, t.is_master = torch.device("cpu"), rank, world, rank == 0
    t.model = build_model(args, seed=3)
    t.engine = WindowEngine(t.model, EngineConfig(), rank=rank, world_size=world)
    t.init_optimizers_schedulers()
    t.sampler = SimpleNamespace(grad_accum_steps=3)
    t.stop_event = threading.Event()
    t.current_window = 10

    def hook():
        if mode == "window":
            t.current_window = 11
        else:
            t.stop_event.set()

    # micro-batch 4 is the second of the second accumulation group: rank 1 learns of the change there
    loader = FlippingLoader(12, 4, hook if rank == 1 else None, args.vocab_size)
    out = asyncio.run(t.inner_steps(loader, step_window=10))
    return {"inner_steps": out["inner_steps"], "batch_count": out["batch_count"], "adam_step": t.engine.adam_step}


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    dist_helper.rank, dist_helper.world_size = rank, world
    res = {mode: run_case(rank, world, mode) for mode in ("window", "stop")}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        print("RESULT " + json.dumps(gathered))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
