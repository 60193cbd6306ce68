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
