"""Real multi-process tier on CPU (gloo, world_size 2): sharded window + DCP round trip."""

import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(nproc, args, timeout=900, worker="_gloo_worker.py", port=29641):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, worker), *map(str, args)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, TPLR_LOG_LEVEL="WARNING"))
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, r.stdout[-2000:] + r.stderr[-4000:]
    return json.loads(lines[-1][7:])


@pytest.mark.parametrize("update", ["sgd", "sign"])
def test_two_rank_window_and_checkpoint_roundtrip(tmp_path, update):
    res = launch(2, ["small", 2, 64, update, tmp_path])
    assert len(res) == 2
    for r in res:
        assert r["same_weights"] and r["master_roundtrip"] and r["compute_roundtrip"], r
        assert r["ckpt"] == [7, 3] and r["status"] == 0
        assert r["loss0"] > 0 and abs(r["loss1"] - r["loss0"]) > 1e-6       # the outer step moved the model


def test_tensor_parallel_sharding_matches_unsharded_model():
    """Heads, hidden features and the (padded) vocabulary split over 2 ranks: same loss and the same
    parameter gradients as the unsharded model, with the projections on torch.distributed collectives."""
    res = launch(2, [], worker="_gloo_tp_worker.py", port=29643)
    assert len(res) == 2
    for r in res:
        assert r["vocab_padded"] == 512
        assert abs(r["loss"] - r["ref_loss"]) < 1e-4, r
        assert r["worst_rel"] < 1e-3, r
        assert r["ckpt_loss_diff"] < 1e-6 and r["ckpt_grad_diff"] < 1e-5, r      # activation checkpointing changes nothing


def test_sharded_quantised_compress_matches_unsharded():
    """2 gloo ranks: payload merged over the ranks, per-tensor statistics on whole tensors, every rank corrects the
    error feedback of its own chunks; same codes, tables, values and error feedback as one rank."""
    res = launch(2, [], worker="_gloo_quant_worker.py", port=29645)
    assert len(res) == 2
    for r in res:
        assert r["codes_equal"] == 1.0 and r["table"] < 1e-9 and r["val"] < 1e-9, r
        assert r["ef"] < 1e-6 * max(r["ef_scale"], 1e-3) + 2e-9, r


def test_evaluator_on_two_ranks_agrees_on_windows_and_runs_one_task_child(tmp_path):
    """Two gloo ranks of one evaluator: rank 0 decides which checkpoint is evaluated, only rank 0 starts the
    downstream-task child (which must not see the launcher's environment), the sentinel of the hand-over is gone
    afterwards, and a backfill over a range with one complete checkpoint evaluates exactly that one on both ranks."""
    import stat

    bindir = tmp_path / "bin"
    bindir.mkdir()
    harness = bindir / "lm_eval"
    harness.write_text(f"""#!/usr/bin/env python3
import json, os, sys
a = sys.argv[1:]
out, tasks = a[a.index("--output_path") + 1], a[a.index("--tasks") + 1].split(",")
assert not [k for k in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID") if k in os.environ]
assert "tensor_parallel_size=2" in a[a.index("--model_args") + 1]
open({str(tmp_path / 'harness_calls.txt')!r}, "a").write("x ")
os.makedirs(os.path.join(out, "m"), exist_ok=True)
json.dump({{"results": {{t: {{"acc,none": 0.4}} for t in tasks}}}}, open(os.path.join(out, "m", "results.json"), "w"))
""")
    harness.chmod(harness.stat().st_mode | stat.S_IXUSR)
    env = dict(os.environ, TPLR_LOG_LEVEL="WARNING", TPLR_STORE="local", TPLR_STORE_ROOT=str(tmp_path / "store"),
               TPLR_STATIC_CHAIN_STATE=str(tmp_path / "chain.json"), TPLR_METRICS_JSONL=str(tmp_path / "metrics.jsonl"),
               PATH=f"{bindir}{os.pathsep}{os.environ['PATH']}")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(HERE, "_gloo_evaluator_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert r.returncode == 0 and lines, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads(lines[-1][7:])
    assert len(res) == 2
    for x in res:
        assert x["evaluated"] == [5] and x["counter"] == 1 and x["start_window"] == 3 and not x["baseline"], x
        assert x["backfilled"] == [5] and x["counter_after"] == 2 and x["sentinels_left"] == [], x
        assert x["cache"] == [5] and x["export_complete"], x
    assert res[0]["child_runs"] == 2                           # once per evaluation, rank 0 only
    recs = [json.loads(l) for l in (tmp_path / "metrics.jsonl").read_text().splitlines()]
    scores = [x for x in recs if x["measurement"].endswith("benchmark_task")]
    assert len(scores) == 2 and all(x["fields"]["score"] == 0.4 and x["tags"]["metric"] == "acc,none" for x in scores)
