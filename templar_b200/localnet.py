"""A whole network on one machine, offline: one validator and N miners as separate processes.

    python -m templar_b200.localnet --miners 2 --windows 10 --block-time 1 [--device cpu] [--evaluator] [--dir D]

The nodes are the ordinary ``neurons/validator.py`` / ``neurons/miner.py`` / ``neurons/evaluator.py`` with
``--local``: the toy model of ``hparams/hparams-local-run.json``, the static chain (wall-clock blocks; the processes
share its commitments through one state file and its clock through one genesis time) and a directory as the object
store.  Nothing is wired by hand: the miners commit their buckets, the validator finds them active, publishes the
peer list and the start window, the miners pick the list up, everyone gathers the same payloads and applies the
same outer step, the validator scores the miners and uploads checkpoints, the evaluator follows the checkpoints.
The role of the reference's scripts/start.sh + ecosystem.config.js + scripts/local_miner_test.py for a run
without a chain node and a bucket.

``launch`` returns a summary read from the nodes' metrics files (windows done, gather success, the validator's
sync scores); the command prints it as JSON.  ``--device cuda`` puts node ``i`` on GPU ``i % device_count``.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def _records(path: Path) -> list[dict]:
    if not path.exists():
        return []
    out = []
    for line in path.read_text().splitlines():
        try:
            out.append(json.loads(line))
        except ValueError:
            continue
    return out


def summarise(root: Path, miner_uids: list[int]) -> dict:
    """What the run did, from the metrics files the nodes wrote under ``root``."""
    out: dict = {"miners": {}, "validator": {}, "evaluator": {}}
    for u in miner_uids:
        recs = [r for r in _records(root / f"miner{u}.jsonl") if r["measurement"].endswith("training_step_v2")]
        gathered = [r["fields"].get("gather_success_rate", 0.0) for r in recs]
        out["miners"][u] = {"windows": len(recs), "windows_with_gather": sum(1 for g in gathered if g and g > 0),
                            "last_loss": recs[-1]["fields"].get("loss") if recs else None,
                            "global_step": int(recs[-1]["fields"].get("global_step", 0)) if recs else 0}
    v = _records(root / "validator.jsonl")
    wins = [r for r in v if r["measurement"].endswith("validator_window_v2")]
    sync = [r for r in v if r["measurement"].endswith("validator_sync_score")]
    out["validator"] = {"windows": len(wins), "windows_with_scores": sum(1 for r in wins if r["fields"].get("n_scored", 0) > 0),
                        "max_gathered": max((int(r["fields"].get("n_gathered", 0)) for r in wins), default=0),
                        "last_sync": {r["tags"].get("uid", "?"): r["fields"] for r in sync[-2 * len(miner_uids):]}}
    ev = [r for r in _records(root / "evaluator.jsonl") if r["measurement"].endswith("custom_evaluation")]
    out["evaluator"] = {"evaluations": len(ev), "last": ev[-1]["fields"] if ev else None}
    return out


def launch(root: str | os.PathLike, miners: int = 2, windows: int = 10, block_time: float = 1.0, device: str = "cpu",
           evaluator: bool = False, timeout_s: float | None = None, hparams_file: str | None = None,
           extra_args: list[str] | None = None) -> dict:
    """Run the network under ``root`` until every node has done its windows (or ``timeout_s`` passed, after which the
    nodes are stopped).  Returns ``{"returncodes": {...}, "summary": {...}, "logs": {...}}``."""
    root = Path(root).resolve()
    root.mkdir(parents=True, exist_ok=True)
    env = dict(os.environ, TPLR_STORE="local", TPLR_STORE_ROOT=str(root / "store"),
               TPLR_STATIC_CHAIN_STATE=str(root / "chain.json"), TPLR_STATIC_CHAIN_GENESIS=repr(time.time()),
               PYTHONPATH=f"{REPO}{os.pathsep}{os.environ.get('PYTHONPATH', '')}")
    env.setdefault("TPLR_LOG_LEVEL", "INFO")
    if not device.startswith("cuda"):
        env.setdefault("OMP_NUM_THREADS", "2")                   # several nodes share the host's cores
    n_uids = max(8, miners + 2)
    miner_uids = list(range(2, 2 + miners))                      # uid 0 (highest stake) validates, uid 1 evaluates
    n_gpus = 0
    if device.startswith("cuda"):
        import torch

        n_gpus = torch.cuda.device_count()
    common = ["--local", "--device", device, "--block-time", str(block_time), "--static-n", str(n_uids), *(extra_args or [])]
    if hparams_file:
        common += ["--hparams-file", str(hparams_file)]
    procs: dict[str, subprocess.Popen] = {}
    logs: dict[str, Path] = {}

    def start(name: str, script: str, uid: int, args: list[str], slot: int) -> None:
        work = root / name
        work.mkdir(exist_ok=True)
        e = dict(env, TPLR_METRICS_JSONL=str(root / f"{name}.jsonl"))
        if n_gpus:
            e["CUDA_VISIBLE_DEVICES"] = str(slot % n_gpus)
        logs[name] = root / f"{name}.log"
        with open(logs[name], "w") as f:
            procs[name] = subprocess.Popen([sys.executable, str(REPO / "neurons" / script), "--uid", str(uid), *common, *args],
                                           cwd=work, env=e, stdout=f, stderr=subprocess.STDOUT)

    # the miners get a few windows more than the validator: the validator works one window behind them
    for i, u in enumerate(miner_uids):
        start(f"miner{u}", "miner.py", u, ["--max-windows", str(windows + 2)], i + 1)
    start("validator", "validator.py", 0, ["--max-windows", str(windows)], 0)
    if evaluator:
        start("evaluator", "evaluator.py", 1, ["--skip-lm-eval", "--eval-interval", str(max(1, int(4 * block_time))),
                                               "--custom-eval-batches", "1", "--max-windows", "2"], miners + 1)
    window_s = 4 * block_time
    deadline = time.time() + (timeout_s if timeout_s is not None else 60.0 + 3.0 * window_s * (windows + 6))
    rcs: dict[str, int | None] = {}
    try:
        for name, p in procs.items():
            try:
                rcs[name] = p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                rcs[name] = None
    finally:
        for name, p in procs.items():                            # stop exactly the processes started here
            if p.poll() is None:
                p.terminate()
        for name, p in procs.items():
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()
    return {"returncodes": rcs, "summary": summarise(root, miner_uids), "logs": {k: str(v) for k, v in logs.items()}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dir", default="./localnet")
    ap.add_argument("--miners", type=int, default=2)
    ap.add_argument("--windows", type=int, default=10)
    ap.add_argument("--block-time", type=float, default=1.0, help="seconds per block of the static chain (4 blocks per window)")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--evaluator", action="store_true")
    ap.add_argument("--timeout", type=float, default=None)
    ap.add_argument("--hparams-file", default=None)
    a = ap.parse_args(argv)
    res = launch(a.dir, a.miners, a.windows, a.block_time, a.device, a.evaluator, a.timeout, a.hparams_file)
    print(json.dumps(res, indent=1, default=str))
    ok = all(rc == 0 for rc in res["returncodes"].values())
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
